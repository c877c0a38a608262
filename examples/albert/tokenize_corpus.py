#!/usr/bin/env python
"""Turn plain text into the token file that ``run_trainer.py --dataset_path`` reads.

The reference's counterpart (examples/albert/tokenize_wikitext103.py) downloads WikiText-103 and the ALBERT tokenizer;
this script works offline on any UTF-8 text files: it loads a SentencePiece model (``--spm_model``, e.g. ALBERT's
``spiece.model``) or trains one on the corpus itself (``--train_vocab_size``), cuts the text into sentences, packs
consecutive sentences of a document into sequences of ``[CLS] ... [SEP]`` of at most ``--seq_length`` tokens, pads with
``<pad>`` and writes ``{"input_ids": int64 [n, seq_length], "vocab_size": V, "special_ids": {...}}`` with ``torch.save``.
Blank lines separate documents; sequences never straddle two documents. ``--sentence_order`` makes rows of two
segments (``[CLS] A [SEP] B [SEP]``, swapped in half of the rows) and adds ``token_type_ids`` and
``sentence_order_label``, which switches the trainer to both of ALBERT's objectives.

    python examples/albert/tokenize_corpus.py --text wiki.train.txt --spm_model spiece.model --out tokens.pt
    python examples/albert/run_trainer.py --dataset_path tokens.pt ...
"""
import argparse
import random
import re
import tempfile
from pathlib import Path
from typing import Dict, Iterable, Iterator, List

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


def pack(tokenizer: spm.SentencePieceProcessor, docs: Iterable[List[str]], seq_length: int, sentence_order: bool = False,
         seed: int = 0) -> Dict[str, torch.Tensor]:
    """Pack sentences into rows of ``seq_length`` ids. Plain rows are ``[CLS] tokens [SEP] <pad>...``. With
    ``sentence_order`` a row is ``[CLS] A [SEP] B [SEP]``: a run of sentences cut at a sentence boundary, the halves
    swapped in every other row on average; ``token_type_ids`` marks B and ``sentence_order_label`` is 1 for swapped."""
    cls_id, sep_id, pad_id = (tokenizer.piece_to_id(p) for p in ("[CLS]", "[SEP]", "<pad>"))
    budget = seq_length - (3 if sentence_order else 2)
    rng = random.Random(seed)
    rows: List[List[int]] = []
    types: List[List[int]] = []
    orders: List[int] = []

    def close(sentences: List[List[int]]) -> None:
        tokens = [t for sentence in sentences for t in sentence]
        if not tokens:
            return
        if not sentence_order:
            row = [cls_id] + tokens + [sep_id]
            rows.append(row + [pad_id] * (seq_length - len(row)))
            return
        if len(sentences) > 1:
            cut = rng.randint(1, len(sentences) - 1)
            first = [t for sentence in sentences[:cut] for t in sentence]
        elif len(tokens) > 1:
            first = tokens[:len(tokens) // 2]  # a lone sentence is cut in the middle
        else:
            return
        second = tokens[len(first):]
        swapped = rng.random() < 0.5
        if swapped:
            first, second = second, first
        row = [cls_id] + first + [sep_id] + second + [sep_id]
        kinds = [0] * (len(first) + 2) + [1] * (len(second) + 1)
        rows.append(row + [pad_id] * (seq_length - len(row)))
        types.append(kinds + [0] * (seq_length - len(kinds)))
        orders.append(int(swapped))

    for sentences in docs:
        current: List[List[int]] = []
        used = 0
        for ids in tokenizer.encode(sentences):
            while len(ids) > budget:  # a sentence longer than a whole sequence is cut into full sequences
                close(current)
                current, used = [], 0
                close([ids[:budget]])
                ids = ids[budget:]
            if used + len(ids) > budget:
                close(current)
                current, used = [], 0
            if ids:
                current.append(ids)
                used += len(ids)
        close(current)
    out = {"input_ids": torch.tensor(rows, dtype=torch.int64).reshape(-1, seq_length)}
    if sentence_order:
        out["token_type_ids"] = torch.tensor(types, dtype=torch.int64).reshape(-1, seq_length)
        out["sentence_order_label"] = torch.tensor(orders, dtype=torch.int64)
    return out


def main(argv=None) -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--text", nargs="+", type=Path, required=True, help="UTF-8 text files; blank lines separate documents")
    parser.add_argument("--out", type=Path, required=True, help="where to write the token file")
    parser.add_argument("--spm_model", type=Path, default=None, help="a SentencePiece model to tokenize with")
    parser.add_argument("--train_vocab_size", type=int, default=30000,
                        help="without --spm_model: train a unigram model of (at most) this size on the corpus")
    parser.add_argument("--seq_length", type=int, default=512)
    parser.add_argument("--sentence_order", action="store_true",
                        help="rows of two segments with token types and sentence-order labels (ALBERT's second objective)")
    parser.add_argument("--seed", type=int, default=0, help="decides where rows are cut and which are swapped")
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
        packed = pack(tokenizer, documents(args.text), args.seq_length, args.sentence_order, args.seed)
    input_ids = packed["input_ids"]
    torch.save({**packed, "vocab_size": tokenizer.get_piece_size(), "special_ids": special_ids}, args.out)
    filled = (input_ids != special_ids["<pad>"]).float().mean().item() if len(input_ids) else 0.0
    print(f"{len(input_ids)} sequences of {args.seq_length} tokens ({100 * filled:.1f} % filled), "
          f"vocabulary {tokenizer.get_piece_size()} -> {args.out}")


if __name__ == "__main__":
    main()
