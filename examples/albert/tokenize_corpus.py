#!/usr/bin/env python
"""Turn plain text into the token file that ``run_trainer.py --dataset_path`` reads.

The reference's counterpart (examples/albert/tokenize_wikitext103.py) downloads WikiText-103 and the ALBERT tokenizer;
this script works offline on any UTF-8 text files: it loads a SentencePiece model (``--spm_model``, e.g. ALBERT's
``spiece.model``) or trains one on the corpus itself (``--train_vocab_size``), cuts the text into sentences, packs
consecutive sentences of a document into sequences of ``[CLS] ... [SEP]`` of at most ``--seq_length`` tokens, pads with
``<pad>`` and writes ``{"input_ids": int64 [n, seq_length], "vocab_size": V, "special_ids": {...}}`` with ``torch.save``.
Blank lines separate documents; sequences never straddle two documents.

    python examples/albert/tokenize_corpus.py --text wiki.train.txt --spm_model spiece.model --out tokens.pt
    python examples/albert/run_trainer.py --dataset_path tokens.pt ...
"""
import argparse
import re
import tempfile
from pathlib import Path
from typing import Iterable, Iterator, List

import sentencepiece as spm
import torch

# ids of the ALBERT vocabulary; a model trained here gets the same layout
SPECIAL = {"<pad>": 0, "<unk>": 1, "[CLS]": 2, "[SEP]": 3, "[MASK]": 4}
_SENTENCE_END = re.compile(r"(?<=[.!?])\s+")


def documents(paths: Iterable[Path]) -> Iterator[List[str]]:
    """Yield each document as a list of sentences; headings of the WikiText kind (``= Title =``) are dropped."""
    for path in paths:
        sentences: List[str] = []
        with open(path, encoding="utf-8") as lines:
            for line in lines:
                line = line.strip()
                if not line:
                    if sentences:
                        yield sentences
                        sentences = []
                    continue
                if line.startswith("=") and line.endswith("="):
                    continue
                sentences.extend(piece for piece in _SENTENCE_END.split(line) if piece)
        if sentences:
            yield sentences


def train_tokenizer(paths: List[Path], vocab_size: int, workdir: Path) -> spm.SentencePieceProcessor:
    prefix = str(workdir / "corpus_spm")
    spm.SentencePieceTrainer.train(
        input=",".join(map(str, paths)), model_prefix=prefix, vocab_size=vocab_size, model_type="unigram",
        pad_id=SPECIAL["<pad>"], unk_id=SPECIAL["<unk>"], bos_id=-1, eos_id=-1, pad_piece="<pad>", unk_piece="<unk>",
        user_defined_symbols=["[CLS]", "[SEP]", "[MASK]"], hard_vocab_limit=False, minloglevel=2)
    return spm.SentencePieceProcessor(model_file=prefix + ".model")


def pack(tokenizer: spm.SentencePieceProcessor, docs: Iterable[List[str]], seq_length: int) -> torch.Tensor:
    cls_id, sep_id, pad_id = (tokenizer.piece_to_id(p) for p in ("[CLS]", "[SEP]", "<pad>"))
    budget = seq_length - 2
    rows: List[List[int]] = []

    def close(tokens: List[int]) -> None:
        if tokens:
            row = [cls_id] + tokens + [sep_id]
            rows.append(row + [pad_id] * (seq_length - len(row)))

    for sentences in docs:
        current: List[int] = []
        for ids in tokenizer.encode(sentences):
            while len(ids) > budget:  # a sentence longer than a whole sequence is cut into full sequences
                close(current)
                current = []
                close(ids[:budget])
                ids = ids[budget:]
            if len(current) + len(ids) > budget:
                close(current)
                current = []
            current.extend(ids)
        close(current)
    return torch.tensor(rows, dtype=torch.int64).reshape(-1, seq_length)


def main(argv=None) -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--text", nargs="+", type=Path, required=True, help="UTF-8 text files; blank lines separate documents")
    parser.add_argument("--out", type=Path, required=True, help="where to write the token file")
    parser.add_argument("--spm_model", type=Path, default=None, help="a SentencePiece model to tokenize with")
    parser.add_argument("--train_vocab_size", type=int, default=30000,
                        help="without --spm_model: train a unigram model of (at most) this size on the corpus")
    parser.add_argument("--seq_length", type=int, default=512)
    args = parser.parse_args(argv)

    with tempfile.TemporaryDirectory() as workdir:
        if args.spm_model is not None:
            tokenizer = spm.SentencePieceProcessor(model_file=str(args.spm_model))
        else:
            tokenizer = train_tokenizer(args.text, args.train_vocab_size, Path(workdir))
        special_ids = {piece: tokenizer.piece_to_id(piece) for piece in SPECIAL}
        missing = [piece for piece, index in special_ids.items() if piece != "<unk>" and index == tokenizer.unk_id()]
        if missing:
            raise SystemExit(f"the tokenizer has no pieces {missing}; ALBERT's spiece.model has all of them")
        input_ids = pack(tokenizer, documents(args.text), args.seq_length)
    torch.save({"input_ids": input_ids, "vocab_size": tokenizer.get_piece_size(), "special_ids": special_ids}, args.out)
    filled = (input_ids != special_ids["<pad>"]).float().mean().item() if len(input_ids) else 0.0
    print(f"{len(input_ids)} sequences of {args.seq_length} tokens ({100 * filled:.1f} % filled), "
          f"vocabulary {tokenizer.get_piece_size()} -> {args.out}")


if __name__ == "__main__":
    main()
