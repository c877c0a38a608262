"""Model families against plain PyTorch fp32 restatements of the same architecture."""
import pytest
import torch
import torch.nn.functional as F

from hivemind_b200.models.gpt2 import GPT2Config, GPT2LMHeadModel, make_lm_batch


def _gpt2_reference_loss(cfg: GPT2Config, p, input_ids, labels):
    """Textbook pre-LayerNorm GPT-2 in fp64 over a dict of parameters named like the model's."""
    b, s = input_ids.shape
    x = p["wte"][input_ids] + p["wpe"][:s]
    mask = torch.ones(s, s, dtype=torch.bool, device=x.device).tril()
    for i in range(cfg.n_layer):
        g = lambda name: p[f"blocks.{i}.{name}"]
        h = F.layer_norm(x, (cfg.n_embd,), g("ln_1_weight"), g("ln_1_bias"), cfg.layer_norm_eps)
        qkv = (h @ g("qkv_weight").T + g("qkv_bias")).view(b, s, 3, cfg.n_head, -1)
        q, k, v = (qkv[:, :, j].transpose(1, 2) for j in range(3))
        att = (q @ k.transpose(-1, -2)) / q.shape[-1] ** 0.5
        att = att.masked_fill(~mask, float("-inf")).softmax(-1)
        ctx = (att @ v).transpose(1, 2).reshape(b, s, cfg.n_embd)
        x = x + ctx @ g("attn_out_weight").T + g("attn_out_bias")
        h = F.layer_norm(x, (cfg.n_embd,), g("ln_2_weight"), g("ln_2_bias"), cfg.layer_norm_eps)
        h = F.gelu(h @ g("ffn_weight").T + g("ffn_bias"), approximate="tanh")
        x = x + h @ g("ffn_out_weight").T + g("ffn_out_bias")
    x = F.layer_norm(x, (cfg.n_embd,), p["ln_f_weight"], p["ln_f_bias"], cfg.layer_norm_eps)
    logits = x @ p["wte"][:cfg.vocab_size].T
    return F.cross_entropy(logits.view(b * s, -1), labels.reshape(-1), ignore_index=-100)


def _autograd_reference(model, batch):
    params = {name: q.detach().double().requires_grad_(True) for name, q in model.named_parameters()}
    loss = _gpt2_reference_loss(model.cfg, params, batch["input_ids"], batch["labels"])
    loss.backward()
    return loss.detach(), {name: q.grad for name, q in params.items()}


def _check_model(device, loss_tol, grad_tol):
    torch.manual_seed(0)
    cfg = GPT2Config.tiny()
    model = GPT2LMHeadModel(cfg).to(device)
    with torch.no_grad():  # make the biases and norms non-trivial
        for name, q in model.named_parameters():
            if q.ndim == 1:
                q.add_(0.1 * torch.randn_like(q))
    batch = {k: v.to(device) for k, v in make_lm_batch(cfg, 3, 48, generator=torch.Generator().manual_seed(1)).items()}
    loss = model(batch["input_ids"], batch["labels"])
    loss.backward()
    ref_loss, ref_grads = _autograd_reference(model, batch)
    assert abs(loss.item() - ref_loss.item()) <= loss_tol * abs(ref_loss.item()), (loss.item(), ref_loss.item())
    for name, q in model.named_parameters():
        assert q.grad is not None, name
        ref = ref_grads[name].to(q.grad.dtype)
        err = (q.grad - ref).norm() / ref.norm().clamp_min(1e-6)
        assert err.item() <= grad_tol, (name, err.item())
    assert model.wte.grad[cfg.vocab_size:].abs().max().item() < 1e-6  # padded vocabulary rows get no gradient
    # the default labels are the inputs shifted by one
    assert torch.allclose(model(batch["input_ids"]).float(), loss.detach().float(), rtol=5 * loss_tol + 1e-6)
    assert model.logits(batch["input_ids"]).shape == (3, 48, cfg.vocab_size)


def test_gpt2_matches_reference_cpu():
    _check_model(torch.device("cpu"), loss_tol=1e-5, grad_tol=1e-4)


@pytest.mark.gpu
def test_gpt2_matches_reference_gpu():
    from hivemind_b200.ops import _lib
    before = _lib.launch_count()
    _check_model(torch.device("cuda"), loss_tol=5e-3, grad_tol=6e-2)
    assert _lib.launch_count() > before  # the native kernels ran, not a fallback


def test_layer_norm_return_sum_cpu():
    from hivemind_b200.ops.norm_act import layer_norm
    x, r = torch.randn(5, 32, requires_grad=True), torch.randn(5, 32, requires_grad=True)
    g, b = torch.randn(32, requires_grad=True), torch.randn(32, requires_grad=True)
    y, z = layer_norm(x, g, b, 1e-5, residual=r, return_sum=True)
    assert torch.allclose(z, x + r)
    assert torch.allclose(y, F.layer_norm(x + r, (32,), g, b, 1e-5), atol=1e-6)


@pytest.mark.gpu
def test_layer_norm_return_sum_gpu():
    from hivemind_b200.ops.norm_act import layer_norm
    torch.manual_seed(0)
    x = torch.randn(300, 1024, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    r = torch.randn(300, 1024, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(1024, device="cuda", requires_grad=True)
    b = torch.randn(1024, device="cuda", requires_grad=True)
    y, z = layer_norm(x, g, b, 1e-5, residual=r, return_sum=True)
    wy, wz = torch.randn_like(y), torch.randn_like(z)
    ((y * wy).sum() + (z * wz).sum()).backward()
    xf, rf = x.detach().float().requires_grad_(True), r.detach().float().requires_grad_(True)
    gf, bf = g.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    zf = xf + rf
    yf = F.layer_norm(zf, (1024,), gf, bf, 1e-5)
    ((yf * wy.float()).sum() + (zf * wz.float()).sum()).backward()
    assert torch.allclose(z.float(), zf, atol=2e-2)
    assert torch.allclose(y.float(), yf, atol=5e-2, rtol=2e-2)
    for got, ref in ((x.grad, xf.grad), (r.grad, rf.grad), (g.grad, gf.grad), (b.grad, bf.grad)):
        assert ((got.float() - ref).norm() / ref.norm()).item() < 2e-2


def _albert_reference_hidden(cfg, p, ids, token_type_ids=None):
    """Textbook ALBERT encoder (factorised embeddings, one shared post-LayerNorm block) in the precision of ``p``."""
    b, s = ids.shape
    e, h = cfg.embedding_size, cfg.hidden_size
    types = p["token_type_embeddings"][0] if token_type_ids is None else p["token_type_embeddings"][token_type_ids]
    x = p["word_embeddings"][ids] + p["position_embeddings"][:s] + types
    x = F.layer_norm(x, (e,), p["emb_ln_weight"], p["emb_ln_bias"], cfg.layer_norm_eps)
    x = x @ p["emb_proj_weight"].T + p["emb_proj_bias"]
    g = lambda name: p[f"layer.{name}"]
    for _ in range(cfg.num_hidden_layers):
        qkv = (x @ g("qkv_weight").T + g("qkv_bias")).view(b, s, 3, cfg.num_attention_heads, -1)
        q, k, v = (qkv[:, :, j].transpose(1, 2) for j in range(3))
        att = ((q @ k.transpose(-1, -2)) / q.shape[-1] ** 0.5).softmax(-1)
        ctx = (att @ v).transpose(1, 2).reshape(b, s, h)
        x = F.layer_norm(x + ctx @ g("attn_out_weight").T + g("attn_out_bias"), (h,), g("attn_ln_weight"),
                         g("attn_ln_bias"), cfg.layer_norm_eps)
        inter = F.gelu(x @ g("ffn_weight").T + g("ffn_bias"), approximate="tanh")
        x = F.layer_norm(x + inter @ g("ffn_out_weight").T + g("ffn_out_bias"), (h,), g("ffn_ln_weight"),
                         g("ffn_ln_bias"), cfg.layer_norm_eps)
    return x


def _albert_reference_loss(cfg, p, batch, token_type_ids=None, sentence_order_label=None):
    """Masked-LM loss with the tied decoder, plus the sentence-order loss when its labels are given; fp64."""
    ids, labels = batch["input_ids"], batch["labels"]
    b, s = ids.shape
    x = _albert_reference_hidden(cfg, p, ids, token_type_ids)
    z = F.gelu(x @ p["head_dense_weight"].T + p["head_dense_bias"], approximate="tanh")
    z = F.layer_norm(z, (cfg.embedding_size,), p["head_ln_weight"], p["head_ln_bias"], cfg.layer_norm_eps)
    logits = z @ p["word_embeddings"].T + p["decoder_bias"]
    loss = F.cross_entropy(logits.view(b * s, -1), labels.reshape(-1), ignore_index=-100)
    if sentence_order_label is not None:
        pooled = torch.tanh(x[:, 0] @ p["pooler_weight"].T + p["pooler_bias"])
        loss = loss + F.cross_entropy(pooled @ p["sop_weight"].T + p["sop_bias"], sentence_order_label)
    return loss


def _check_albert(device, loss_tol, grad_tol):
    from hivemind_b200.models.albert import AlbertConfig, AlbertForMaskedLM, make_mlm_batch

    torch.manual_seed(0)
    cfg = AlbertConfig.tiny()
    model = AlbertForMaskedLM(cfg).to(device)
    with torch.no_grad():
        for name, q in model.named_parameters():
            if q.ndim == 1:
                q.add_(0.1 * torch.randn_like(q))
    batch = {k: v.to(device) for k, v in make_mlm_batch(cfg, 3, 40, generator=torch.Generator().manual_seed(1)).items()}
    loss = model(batch["input_ids"], batch["labels"], masked_positions=batch["masked_positions"])
    loss.backward()
    params = {name: q.detach().double().requires_grad_(True) for name, q in model.named_parameters()}
    ref_loss = _albert_reference_loss(cfg, params, batch)
    ref_loss.backward()
    assert abs(loss.item() - ref_loss.item()) <= loss_tol * abs(ref_loss.item()), (loss.item(), ref_loss.item())
    for name, q in model.named_parameters():
        if name == "token_type_embeddings":
            ref = params[name].grad[:1].to(q.grad.dtype)  # only segment 0 is used
            got = q.grad[:1]
        else:
            ref, got = params[name].grad.to(q.grad.dtype), q.grad
        err = (got - ref).norm() / ref.norm().clamp_min(1e-6)
        assert err.item() <= grad_tol, (name, err.item())
    # finding the labelled rows on the fly gives the same loss as passing their positions
    again = model(batch["input_ids"], batch["labels"])
    assert torch.allclose(again.float(), loss.detach().float(), rtol=5 * loss_tol + 1e-6)


def _check_albert_pretraining(device, loss_tol, grad_tol):
    """Both objectives (masked LM + sentence order) with two segment types against the fp64 restatement."""
    from hivemind_b200.models.albert import AlbertConfig, AlbertForPreTraining, make_mlm_batch

    torch.manual_seed(0)
    cfg = AlbertConfig.tiny()
    model = AlbertForPreTraining(cfg).to(device)
    with torch.no_grad():
        for name, q in model.named_parameters():
            if q.ndim == 1:
                q.add_(0.1 * torch.randn_like(q))
    batch = {k: v.to(device) for k, v in make_mlm_batch(cfg, 5, 48, generator=torch.Generator().manual_seed(2)).items()}
    token_types = (torch.arange(48, device=device).unsqueeze(0) >= torch.tensor([[20], [24], [30], [10], [40]], device=device)).long()
    order = torch.tensor([0, 1, 1, 0, 1], device=device)
    loss = model(batch["input_ids"], batch["labels"], masked_positions=batch["masked_positions"],
                 token_type_ids=token_types, sentence_order_label=order)
    loss.backward()
    params = {name: q.detach().double().requires_grad_(True) for name, q in model.named_parameters()}
    ref_loss = _albert_reference_loss(cfg, params, batch, token_types, order)
    ref_loss.backward()
    assert abs(loss.item() - ref_loss.item()) <= loss_tol * abs(ref_loss.item()), (loss.item(), ref_loss.item())
    for name, q in model.named_parameters():
        ref = params[name].grad.to(q.grad.dtype)
        err = (q.grad - ref).norm() / ref.norm().clamp_min(1e-6)
        assert err.item() <= grad_tol, (name, err.item())
    # without sentence-order labels the model is the masked-LM model
    mlm_only = model(batch["input_ids"], batch["labels"], masked_positions=batch["masked_positions"], token_type_ids=token_types)
    ref_mlm = _albert_reference_loss(cfg, params, batch, token_types)
    assert abs(mlm_only.item() - ref_mlm.item()) <= loss_tol * abs(ref_mlm.item())


def test_albert_pretraining_matches_reference_cpu():
    _check_albert_pretraining(torch.device("cpu"), loss_tol=1e-5, grad_tol=1e-4)


@pytest.mark.gpu
def test_albert_pretraining_matches_reference_gpu():
    _check_albert_pretraining(torch.device("cuda"), loss_tol=5e-3, grad_tol=6e-2)


def test_albert_matches_reference_cpu():
    _check_albert(torch.device("cpu"), loss_tol=1e-5, grad_tol=1e-4)


@pytest.mark.gpu
def test_albert_matches_reference_gpu():
    _check_albert(torch.device("cuda"), loss_tol=5e-3, grad_tol=6e-2)


def test_producer_bias_contract_on_the_pytorch_path():
    """linear(skip_bias_grad=True) leaves the bias gradient to layer_norm(producer_bias=...), exactly once."""
    import torch.nn.functional as F

    from hivemind_b200.ops.gemm import linear
    from hivemind_b200.ops.norm_act import layer_norm

    torch.manual_seed(0)
    x = torch.randn(6, 5, 16, requires_grad=True)
    w = torch.randn(24, 16, requires_grad=True)
    bias = torch.randn(24, requires_grad=True)
    g, b = torch.rand(24, requires_grad=True), torch.randn(24, requires_grad=True)
    res = torch.randn(6, 5, 24, requires_grad=True)
    y = layer_norm(linear(x, w, bias, skip_bias_grad=True), g, b, 1e-5, residual=res, producer_bias=bias)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr, biasr, gr, br, resr = (t.detach().clone().requires_grad_() for t in (x, w, bias, g, b, res))
    F.layer_norm(F.linear(xr, wr, biasr) + resr, (24,), gr, br, 1e-5).backward(dy)
    for mine, ref in ((x, xr), (w, wr), (bias, biasr), (g, gr), (b, br), (res, resr)):
        assert torch.allclose(mine.grad, ref.grad, atol=1e-4, rtol=1e-4)


def test_feed_forward_on_the_pytorch_path_is_two_linears():
    import torch.nn.functional as F

    from hivemind_b200.ops.gemm import feed_forward

    torch.manual_seed(1)
    x = torch.randn(4, 7, 16, requires_grad=True)
    w1, b1 = torch.randn(32, 16, requires_grad=True), torch.randn(32, requires_grad=True)
    w2, b2 = torch.randn(16, 32, requires_grad=True), torch.randn(16, requires_grad=True)
    out, skip = feed_forward(x, w1, b1, w2, b2, passthrough=True)
    (out + skip).sum().backward()
    refs = [t.detach().clone().requires_grad_() for t in (x, w1, b1, w2, b2)]
    xr, w1r, b1r, w2r, b2r = refs
    (F.linear(F.gelu(F.linear(xr, w1r, b1r), approximate="tanh"), w2r, b2r) + xr).sum().backward()
    for mine, ref in zip((x, w1, b1, w2, b2), refs):
        assert torch.allclose(mine.grad, ref.grad, atol=1e-4, rtol=1e-4)
