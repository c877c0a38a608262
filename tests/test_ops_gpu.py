"""Numerics of the sm_100a kernels against plain PyTorch fp32 references of the same ops."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("h", [128, 1024, 1536])
def test_layernorm_fwd_bwd(dtype, h):
    from hivemind_b200.ops.norm_act import layer_norm

    torch.manual_seed(0)
    rows = 777
    x = torch.randn(rows, h, device=_dev(), dtype=dtype, requires_grad=True)
    r = torch.randn(rows, h, device=_dev(), dtype=dtype, requires_grad=True)
    g = (torch.rand(h, device=_dev()) + 0.5).requires_grad_()
    b = torch.randn(h, device=_dev()).requires_grad_()
    y = layer_norm(x, g, b, 1e-12, residual=r)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, rr, gr, br = (t.detach().float().requires_grad_() for t in (x, r, g, b))
    yr = F.layer_norm(xr + rr, (h,), gr, br, 1e-12)
    yr.backward(dy.float())
    tol = 3e-2 if dtype == torch.bfloat16 else 1e-4
    assert torch.allclose(y.float(), yr, atol=tol, rtol=tol)
    assert torch.allclose(x.grad.float(), xr.grad, atol=tol, rtol=tol)
    assert torch.allclose(r.grad.float(), rr.grad, atol=tol, rtol=tol)
    assert torch.allclose(g.grad, gr.grad, atol=tol * 30, rtol=tol)
    assert torch.allclose(b.grad, br.grad, atol=tol * 30, rtol=tol)


@pytest.mark.parametrize("h,rows", [(256, 3001), (768, 1111), (1024, 20000), (2048, 515), (128, 999)])
@pytest.mark.parametrize("grads_exist", [False, True])
def test_layernorm_backward_delivers_the_gradient_of_the_producing_bias(h, rows, grads_exist):
    """linear(skip_bias_grad) -> layer_norm(producer_bias): one pass gives dx, dgamma, dbeta and the bias gradient."""
    from hivemind_b200.ops.gemm import linear
    from hivemind_b200.ops.norm_act import layer_norm

    torch.manual_seed(1)
    dev = _dev()
    inp = torch.randn(rows, 64, device=dev, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(h, 64, device=dev) * 0.2).requires_grad_()
    bias = torch.randn(h, device=dev).requires_grad_()
    r = torch.randn(rows, h, device=dev, dtype=torch.bfloat16, requires_grad=True)
    g = (torch.rand(h, device=dev) + 0.5).requires_grad_()
    b = torch.randn(h, device=dev).requires_grad_()
    if grads_exist:  # fp32 .grad buffers with content: the kernels add to them in place
        for t in (w, bias, g, b):
            t.grad = torch.ones_like(t)
    y = layer_norm(linear(inp, w, bias, skip_bias_grad=True), g, b, 1e-12, residual=r, producer_bias=bias)
    dy = torch.randn_like(y)
    y.backward(dy)
    ir, wr, biasr, rr, gr, br = (t.detach().float().requires_grad_() for t in (inp, w, bias, r, g, b))
    lin = F.linear(ir, wr.bfloat16().float(), biasr).bfloat16().float()
    yr = F.layer_norm(lin + rr, (h,), gr, br, 1e-12)
    yr.backward(dy.float())
    base = 1.0 if grads_exist else 0.0
    scale = math.sqrt(rows)
    assert torch.allclose(r.grad.float(), rr.grad, atol=3e-2, rtol=3e-2)
    assert torch.allclose(bias.grad - base, biasr.grad, atol=0.03 * scale, rtol=2e-2)
    assert torch.allclose(g.grad - base, gr.grad, atol=0.03 * scale, rtol=2e-2)
    assert torch.allclose(b.grad - base, br.grad, atol=0.03 * scale, rtol=2e-2)
    assert torch.allclose(w.grad - base, wr.grad, atol=0.03 * scale, rtol=3e-2)
    assert torch.allclose(inp.grad.float(), ir.grad, atol=5e-2, rtol=5e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_bias_gelu(dtype):
    from hivemind_b200.ops.norm_act import bias_gelu

    torch.manual_seed(1)
    x = torch.randn(513, 4096, device=_dev(), dtype=dtype, requires_grad=True)
    b = torch.randn(4096, device=_dev(), requires_grad=True)
    y = bias_gelu(x, b)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, br = x.detach().float().requires_grad_(), b.detach().clone().requires_grad_()
    yr = F.gelu(xr + br, approximate="tanh")
    yr.backward(dy.float())
    tol = 3e-2 if dtype == torch.bfloat16 else 2e-3
    assert torch.allclose(y.float(), yr, atol=tol, rtol=tol)
    assert torch.allclose(x.grad.float(), xr.grad, atol=tol, rtol=tol)
    assert torch.allclose(b.grad, br.grad, atol=0.5 if dtype == torch.bfloat16 else 1e-2, rtol=tol)


def test_multi_tensor_elementwise():
    from hivemind_b200.ops import multi_tensor as mt

    torch.manual_seed(2)
    shapes = [(1000,), (17, 33), (4096, 64), (3,), (1,)]
    acc = [torch.randn(s, device=_dev()) for s in shapes]
    grads = [torch.randn(s, device=_dev()).to(torch.bfloat16 if i % 2 else torch.float32) for i, s in enumerate(shapes)]
    ref = [a.clone() + 0.25 * g.float() for a, g in zip(acc, grads)]
    mt.axpy_(acc, grads, 0.25)
    for a, r in zip(acc, ref):
        assert torch.allclose(a, r, atol=1e-6)
    out = [torch.empty(s, device=_dev(), dtype=torch.bfloat16) for s in shapes]
    mt.scale_copy_(out, acc, 0.5)
    for o, a in zip(out, acc):
        assert torch.allclose(o.float(), (a * 0.5).to(torch.bfloat16).float())
    assert mt.all_finite(acc)
    acc[2][5, 7] = float("inf")
    assert not mt.all_finite(acc)
    acc[2][5, 7] = 0.0
    sq = mt.sumsq(acc)
    for i, a in enumerate(acc):
        assert torch.allclose(sq[i], a.pow(2).sum(), rtol=1e-4)
    total = math.sqrt(float(sq[-1]))
    norm = mt.clip_grad_norm_(acc, total / 2)
    assert abs(float(norm) - total) / total < 1e-4
    assert abs(math.sqrt(float(mt.sumsq(acc)[-1])) - total / 2) / total < 1e-3
    mt.zero_(acc)
    assert all(float(a.abs().sum()) == 0 for a in acc)
    local = [torch.randn(s, device=_dev()) for s in shapes]
    new = [torch.randn(s, device=_dev()) for s in shapes]
    old = [torch.randn(s, device=_dev()) for s in shapes]
    ref = [l + (n - o) for l, n, o in zip(local, new, old)]
    mt.delta_update_(local, new, old)
    for l, r in zip(local, ref):
        assert torch.allclose(l, r, atol=1e-6)


def _clone_all(ts):
    return [t.clone() for t in ts]


@pytest.mark.parametrize("decoupled", [False, True])
def test_adam_matches_torch(decoupled):
    from hivemind_b200.ops import multi_tensor as mt

    torch.manual_seed(3)
    shapes = [(1024, 128), (77,), (30000, 16)]
    params = [torch.randn(s, device=_dev()) for s in shapes]
    ref_params = [p.clone().requires_grad_() for p in params]
    opt_cls = torch.optim.AdamW if decoupled else torch.optim.Adam
    ref_opt = opt_cls(ref_params, lr=1e-2, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.1)
    m = [torch.zeros_like(p) for p in params]
    v = [torch.zeros_like(p) for p in params]
    for step in range(1, 4):
        grads = [torch.randn_like(p) for p in params]
        for rp, g in zip(ref_params, grads):
            rp.grad = g.clone()
        ref_opt.step()
        mt.adam_step_(params, grads, m, v, step=step, lr=1e-2, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.1,
                      decoupled=decoupled)
    for p, rp in zip(params, ref_params):
        assert torch.allclose(p, rp.detach(), atol=2e-5, rtol=1e-4)


def test_lamb_matches_reference_formula():
    from hivemind_b200.ops import multi_tensor as mt

    torch.manual_seed(4)
    shapes = [(512, 256), (1024,), (100, 100)]
    params = [torch.randn(s, device=_dev()) for s in shapes]
    cpu_params = [p.cpu().clone() for p in params]
    state = [[torch.zeros_like(p) for p in params] for _ in range(3)]
    cpu_state = [[torch.zeros_like(p) for p in cpu_params] for _ in range(3)]
    lp = [torch.empty_like(p, dtype=torch.bfloat16) for p in params]
    for step in range(1, 4):
        grads = [torch.randn_like(p) for p in params]
        kw = dict(step=step, lr=1.76e-3, betas=(0.9, 0.999), eps=1e-6, weight_decay=0.01, clamp_value=10000.0)
        mt.lamb_step_(params, grads, state[0], state[1], state[2], model_copies=lp, **kw)
        mt.lamb_step_(cpu_params, [g.cpu() for g in grads], cpu_state[0], cpu_state[1], cpu_state[2], **kw)
    for p, cp, l in zip(params, cpu_params, lp):
        assert torch.allclose(p.cpu(), cp, atol=1e-5, rtol=1e-4)
        assert torch.allclose(l.float(), p.to(torch.bfloat16).float())


def test_sgd_momentum():
    from hivemind_b200.ops import multi_tensor as mt

    torch.manual_seed(5)
    params = [torch.randn(300, 70, device=_dev())]
    ref = [params[0].clone().requires_grad_()]
    opt = torch.optim.SGD(ref, lr=0.1, momentum=0.9, weight_decay=0.01, nesterov=True)
    buf = [torch.zeros_like(params[0])]
    for step in range(3):
        g = [torch.randn_like(params[0])]
        ref[0].grad = g[0].clone()
        opt.step()
        mt.sgd_step_(params, g, buf, lr=0.1, momentum=0.9, weight_decay=0.01, nesterov=True, first_step=step == 0)
    assert torch.allclose(params[0], ref[0].detach(), atol=1e-5)


GEMM_CASES = [
    # m, n, k, a_mn, b_mn
    (128, 256, 64, False, False),
    (256, 512, 256, False, False),
    (300, 1000, 520, False, False),
    (256, 256, 192, False, True),
    (256, 256, 192, True, True),
    (200, 328, 136, True, False),
    (1024, 4096, 1024, False, False),
    (4096, 1024, 2048, True, True),
]


@pytest.mark.parametrize("m,n,k,a_mn,b_mn", GEMM_CASES)
@pytest.mark.parametrize("block_n", [None, 64, 128])
def test_tc_gemm_bf16(m, n, k, a_mn, b_mn, block_n):
    from hivemind_b200.ops.gemm import check_kernel_errors, tc_gemm

    torch.manual_seed(m + n + k)
    a = torch.randn((k, m) if a_mn else (m, k), device=_dev(), dtype=torch.bfloat16)
    b = torch.randn((k, n) if b_mn else (n, k), device=_dev(), dtype=torch.bfloat16)
    d = tc_gemm(a, b, a_mn=a_mn, b_mn=b_mn, block_n=block_n)
    check_kernel_errors()
    ref = (a.t() if a_mn else a).float() @ (b if b_mn else b.t()).float()
    err = (d.float() - ref).abs().max().item()
    assert err <= 2e-2 * math.sqrt(k) + 1e-2 * ref.abs().max().item(), err


@pytest.mark.parametrize("m,n,k,a_mn,b_mn", [c for c in GEMM_CASES if c[0] >= 256 and c[1] >= 256] + [
    (2048, 768, 4096, False, True), (1024, 1024, 2048, True, True), (260, 304, 72, False, False)])
def test_tc_gemm_pair_bf16(m, n, k, a_mn, b_mn):
    """The two-CTA (cta_group::2) kernel against fp32 matmul, all operand layouts."""
    from hivemind_b200.ops.gemm import check_kernel_errors, tc_gemm

    torch.manual_seed(m + n + k)
    a = torch.randn((k, m) if a_mn else (m, k), device=_dev(), dtype=torch.bfloat16)
    b = torch.randn((k, n) if b_mn else (n, k), device=_dev(), dtype=torch.bfloat16)
    d = tc_gemm(a, b, a_mn=a_mn, b_mn=b_mn, pair=True)
    check_kernel_errors()
    ref = (a.t() if a_mn else a).float() @ (b if b_mn else b.t()).float()
    err = (d.float() - ref).abs().max().item()
    assert err <= 2e-2 * math.sqrt(k) + 1e-2 * ref.abs().max().item(), err


def test_tc_gemm_pair_epilogues():
    from hivemind_b200.ops.gemm import check_kernel_errors, tc_gemm

    torch.manual_seed(8)
    m, n, k = 640, 768, 320
    a = torch.randn(m, k, device=_dev(), dtype=torch.bfloat16)
    b = torch.randn(n, k, device=_dev(), dtype=torch.bfloat16) * 0.1
    bias = torch.randn(n, device=_dev())
    aux = torch.empty(m, n, device=_dev(), dtype=torch.bfloat16)
    d = tc_gemm(a, b, bias=bias, gelu=True, aux=aux, pair=True)
    check_kernel_errors()
    pre = a.float() @ b.float().t() + bias
    assert torch.allclose(aux.float(), pre, atol=5e-2, rtol=2e-2)
    assert torch.allclose(d.float(), F.gelu(pre, approximate="tanh"), atol=5e-2, rtol=2e-2)
    acc = torch.ones(m, n, device=_dev())
    tc_gemm(a, b, out=acc, reduce_add=True, splits=3, pair=True)
    check_kernel_errors()
    assert torch.allclose(acc, 1 + a.float() @ b.float().t(), atol=5e-2, rtol=2e-2)


def test_tc_gemm_epilogues():
    from hivemind_b200.ops.gemm import check_kernel_errors, tc_gemm

    torch.manual_seed(7)
    m, n, k = 384, 768, 256
    a = torch.randn(m, k, device=_dev(), dtype=torch.bfloat16)
    b = torch.randn(n, k, device=_dev(), dtype=torch.bfloat16) * 0.1
    bias = torch.randn(n, device=_dev())
    aux = torch.empty(m, n, device=_dev(), dtype=torch.bfloat16)
    d = tc_gemm(a, b, bias=bias, gelu=True, aux=aux)
    check_kernel_errors()
    pre = a.float() @ b.float().t() + bias
    assert torch.allclose(aux.float(), pre, atol=5e-2, rtol=2e-2)
    assert torch.allclose(d.float(), F.gelu(pre, approximate="tanh"), atol=5e-2, rtol=2e-2)
    # fp32 output with reduce-add and split-K
    acc = torch.ones(m, n, device=_dev())
    tc_gemm(a, b, out=acc, reduce_add=True, splits=4)
    check_kernel_errors()
    assert torch.allclose(acc, 1 + a.float() @ b.float().t(), atol=5e-2, rtol=2e-2)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (True, True), (True, False)])
@pytest.mark.parametrize("n", [32, 64, 128])
def test_tc_gemm_tf32(a_mn, b_mn, n):
    from hivemind_b200.ops.gemm import check_kernel_errors, tc_gemm

    torch.manual_seed(11)
    m, k = 520, 328
    a = torch.randn((k, m) if a_mn else (m, k), device=_dev())
    b = torch.randn((k, n) if b_mn else (n, k), device=_dev())
    d = tc_gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    check_kernel_errors()
    ref = (a.t() if a_mn else a).double() @ (b if b_mn else b.t()).double()
    assert d.dtype == torch.float32
    assert (d.double() - ref).abs().max().item() < 5e-2 * math.sqrt(k) / 10 + 2e-2


def test_linear_autograd():
    from hivemind_b200.ops.gemm import check_kernel_errors, linear

    torch.manual_seed(13)
    x = torch.randn(6, 100, 256, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(512, 256, device=_dev()) * 0.05).requires_grad_()
    b = torch.randn(512, device=_dev()).requires_grad_()
    for act in (None, "gelu"):
        x.grad = w.grad = b.grad = None
        y = linear(x, w, b, activation=act)
        dy = torch.randn_like(y)
        y.backward(dy)
        check_kernel_errors()
        xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
        yr = F.linear(xr, wr.to(torch.bfloat16).float(), br)
        if act:
            yr = F.gelu(yr, approximate="tanh")
        yr.backward(dy.float())
        assert torch.allclose(y.float(), yr, atol=5e-2, rtol=3e-2)
        assert torch.allclose(x.grad.float(), xr.grad, atol=5e-2, rtol=3e-2)
        assert torch.allclose(w.grad, wr.grad, atol=0.35, rtol=3e-2)
        assert torch.allclose(b.grad, br.grad, atol=0.35, rtol=3e-2)
    # accumulation straight into an existing fp32 .grad buffer
    w.grad = torch.ones_like(w)
    before = w.grad.data_ptr()
    linear(x, w, b).sum().backward()
    assert w.grad.data_ptr() == before
    ref = 1 + x.detach().float().reshape(-1, 256).sum(0).expand(512, 256)
    assert torch.allclose(w.grad, ref, atol=0.5, rtol=3e-2)


@pytest.mark.parametrize("m,n,k,a_mn,b_mn", [(512, 384, 1024, False, False), (1000, 264, 4096, False, True),
                                             (256, 1024, 16384, True, True)])
def test_tc_gemm_bf16_inputs_fp32_output_is_exact_up_to_fp32_accumulation(m, n, k, a_mn, b_mn):
    """bf16 products are exact in fp32, so against fp64 the only error is the fp32 accumulation: a bound relative to
    sum |a||b| (not to the size of the output) that a dropped k-block, a wrong swizzle or a stale accumulator breaks."""
    from hivemind_b200.ops.gemm import check_kernel_errors, tc_gemm

    torch.manual_seed(m + k)
    a = torch.randn((k, m) if a_mn else (m, k), device=_dev(), dtype=torch.bfloat16)
    b = torch.randn((k, n) if b_mn else (n, k), device=_dev(), dtype=torch.bfloat16)
    d = tc_gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    check_kernel_errors()
    a64 = (a.t() if a_mn else a).double()
    b64 = (b if b_mn else b.t()).double()
    ref, mass = a64 @ b64, a64.abs() @ b64.abs()
    assert d.dtype == torch.float32
    assert ((d.double() - ref).abs() <= 1e-5 * mass + 1e-30).all(), ((d.double() - ref).abs() / mass).max().item()
    # split-K with fp32 reduce-add keeps the same bound
    acc = torch.zeros(m, n, device=_dev(), dtype=torch.float32)
    tc_gemm(a, b, a_mn=a_mn, b_mn=b_mn, out=acc, reduce_add=True, splits=4)
    assert ((acc.double() - ref).abs() <= 1e-5 * mass + 1e-30).all()


@pytest.mark.parametrize("m,n,k", [(300, 256, 512), (4096, 1024, 3072), (129, 72, 64)])
def test_tc_gemm_addend_epilogue(m, n, k):
    from hivemind_b200.ops.gemm import check_kernel_errors, tc_gemm

    torch.manual_seed(5)
    a = torch.randn(m, k, device=_dev(), dtype=torch.bfloat16)
    b = torch.randn(k, n, device=_dev(), dtype=torch.bfloat16)
    wide = torch.randn(m, n + 8, device=_dev(), dtype=torch.bfloat16) * 30
    add = wide[:, :n]  # a strided addend: rows 16-byte aligned, not contiguous
    out = tc_gemm(a, b, b_mn=True, out_dtype=torch.bfloat16, add=add, pair=False)
    check_kernel_errors()
    ref = a.double() @ b.double() + add.double()
    err = (out.double() - ref).abs()
    assert (err <= 0.01 * ref.abs() + 0.02 * math.sqrt(k)).all()
    plain = tc_gemm(a, b, b_mn=True, out_dtype=torch.bfloat16, pair=False)
    assert ((out.float() - plain.float()) - add.float()).abs().max().item() < 0.02 * ref.abs().max().item()


def test_linear_passthrough_adds_the_residual_gradient_in_the_gemm():
    from hivemind_b200.ops.gemm import check_kernel_errors, linear

    torch.manual_seed(14)
    x = torch.randn(4, 130, 256, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(384, 256, device=_dev()) * 0.05).requires_grad_()
    b = torch.randn(384, device=_dev()).requires_grad_()
    y, skip = linear(x, w, b, passthrough=True)
    dy, dskip = torch.randn_like(y), torch.randn_like(skip)
    torch.autograd.backward([y, skip], [dy, dskip])
    check_kernel_errors()
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = F.linear(xr, wr.to(torch.bfloat16).float(), br)
    torch.autograd.backward([yr, xr * 1.0], [dy.float(), dskip.float()])
    assert torch.allclose(x.grad.float(), xr.grad, atol=6e-2, rtol=3e-2)
    assert torch.allclose(w.grad, wr.grad, atol=0.35, rtol=3e-2)
    # only the passed-through tensor used: the gradient goes straight through
    x.grad = None
    _, skip = linear(x, w, b, passthrough=True)
    skip.backward(dskip)
    assert torch.equal(x.grad, dskip)


@pytest.mark.parametrize("passthrough", [False, True])
def test_feed_forward_node_matches_fp32_math(passthrough):
    from hivemind_b200.ops.gemm import check_kernel_errors, feed_forward

    torch.manual_seed(15)
    dev = _dev()
    x = torch.randn(3, 200, 256, device=dev, dtype=torch.bfloat16, requires_grad=True)
    w1 = (torch.randn(1024, 256, device=dev) * 0.05).requires_grad_()
    b1 = torch.randn(1024, device=dev).requires_grad_()
    w2 = (torch.randn(256, 1024, device=dev) * 0.05).requires_grad_()
    b2 = torch.randn(256, device=dev).requires_grad_()
    res = feed_forward(x, w1, b1, w2, b2, passthrough=passthrough)
    out, skip = res if passthrough else (res, None)
    dout = torch.randn_like(out)
    dskip = torch.randn_like(x) if passthrough else None
    torch.autograd.backward([out] + ([skip] if passthrough else []), [dout] + ([dskip] if passthrough else []))
    check_kernel_errors()
    xr, w1r, b1r, w2r, b2r = (t.detach().float().requires_grad_() for t in (x, w1, b1, w2, b2))
    inter = F.gelu(F.linear(xr, w1r.bfloat16().float(), b1r), approximate="tanh")
    outr = F.linear(inter, w2r.bfloat16().float(), b2r)
    torch.autograd.backward([outr] + ([xr * 1.0] if passthrough else []),
                            [dout.float()] + ([dskip.float()] if passthrough else []))
    assert torch.allclose(out.float(), outr, atol=6e-2, rtol=3e-2)
    assert torch.allclose(x.grad.float(), xr.grad, atol=6e-2, rtol=3e-2)
    for mine, ref in ((w1, w1r), (b1, b1r), (w2, w2r), (b2, b2r)):
        assert torch.allclose(mine.grad, ref.grad, atol=0.4, rtol=3e-2), (mine.grad - ref.grad).abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ffn_expert_block_on_cuda_matches_its_fp32_formula(dtype):
    """The ``ffn`` expert of the MoE server (one feed-forward node + LayerNorm with the producer's bias gradient)."""
    from hivemind_b200.moe.server.layers.common import FeedforwardBlock

    torch.manual_seed(21)
    block = FeedforwardBlock(256).to(_dev())
    x = torch.randn(300, 256, device=_dev(), dtype=dtype, requires_grad=True)
    y = block(x)
    dy = torch.randn_like(y)
    y.backward(dy)
    ref = FeedforwardBlock(256).to(_dev())
    ref.load_state_dict(block.state_dict())
    xr = x.detach().float().requires_grad_()
    inner = F.gelu(F.linear(xr, ref.ffn.weight, ref.ffn.bias), approximate="tanh")
    yr = F.layer_norm(xr + F.linear(inner, ref.ffn_output.weight, ref.ffn_output.bias), (256,), ref.layer_norm.weight,
                      ref.layer_norm.bias, 1e-12)
    yr.backward(dy.float())
    assert y.dtype == dtype and torch.allclose(y.float(), yr, atol=6e-2, rtol=3e-2)
    assert torch.allclose(x.grad.float(), xr.grad, atol=8e-2, rtol=5e-2)
    for mine, theirs in zip(block.parameters(), ref.parameters()):
        assert torch.allclose(mine.grad.float(), theirs.grad, atol=0.5, rtol=5e-2), (mine.grad.float() - theirs.grad).abs().max()


def test_orthogonalize_matches_gram_schmidt():
    from hivemind_b200.ops.powersgd import orthogonalize_batch_
    from hivemind_b200.utils.math import orthogonalize_reference_

    torch.manual_seed(17)
    mats = [torch.randn(m, 32, device=_dev()) for m in (1024, 4096, 50257, 100)]
    mats[1][:, 5] = 0  # a dead column stays dead
    refs = [orthogonalize_reference_(m.double().cpu().clone()) for m in mats]
    orthogonalize_batch_(mats)
    for got, ref in zip(mats, refs):
        assert torch.allclose(got.cpu().double(), ref, atol=2e-4), (got.cpu().double() - ref).abs().max()
        gram = got.t() @ got
        live = gram.diag() > 0.5
        assert torch.allclose(gram[live][:, live], torch.eye(int(live.sum()), device=_dev()), atol=1e-4)


@pytest.mark.parametrize("m,n,r", [(1024, 4096, 32), (50257, 1024, 32), (1000, 520, 8), (768, 768, 64)])
def test_powersgd_products(m, n, r):
    from hivemind_b200.ops import powersgd as ps
    from hivemind_b200.ops.gemm import check_kernel_errors

    torch.manual_seed(19)
    M = torch.randn(m, n, device=_dev())
    Q = torch.randn(n, r, device=_dev())
    P = torch.empty(m, r, device=_dev())
    ps.compute_p_(P, M, Q)
    check_kernel_errors()
    ref_p = M.double() @ Q.double()
    assert (P.double() - ref_p).abs().max().item() <= 2e-3 * ref_p.abs().max().item() + 1e-2
    Q2 = torch.empty(n, r, device=_dev())
    ps.compute_q_(Q2, M, P)
    check_kernel_errors()
    ref_q = M.double().t() @ P.double()
    assert (Q2.double() - ref_q).abs().max().item() <= 2e-3 * ref_q.abs().max().item() + 1e-2
    out = torch.empty(m, n, device=_dev())
    ps.reconstruct_(out, P, Q)
    check_kernel_errors()
    ref_o = P.double() @ Q.double().t()
    assert (out.double() - ref_o).abs().max().item() <= 2e-3 * ref_o.abs().max().item() + 1e-2


@pytest.mark.parametrize("count,m,n,r", [(3, 1024, 512, 32), (5, 256, 1024, 8), (2, 3072, 1024, 32)])
def test_powersgd_stacked_products_match_per_matrix_math(count, m, n, r):
    """One grouped launch per product for a stack of equally shaped matrices (tf32) against fp64 matrix products."""
    from hivemind_b200.ops import powersgd as ps
    from hivemind_b200.ops.gemm import check_kernel_errors

    torch.manual_seed(23)
    M = torch.randn(count, m, n, device=_dev())
    Q = torch.randn(count, n, r, device=_dev())
    P = torch.full((count, m, r), float("nan"), device=_dev())
    assert ps.can_stack(m, n, r)
    ps.compute_p_stacked_(P, M, Q)
    check_kernel_errors()
    ref_p = M.double() @ Q.double()
    assert (P.double() - ref_p).abs().max().item() <= 2e-3 * ref_p.abs().max().item() + 1e-2
    Q2 = torch.full((count, n, r), float("nan"), device=_dev())
    ps.compute_q_stacked_(Q2, M, P)
    check_kernel_errors()
    ref_q = M.double().transpose(1, 2) @ P.double()
    assert (Q2.double() - ref_q).abs().max().item() <= 2e-3 * ref_q.abs().max().item() + 1e-2
    out = torch.full((count, m, n), float("nan"), device=_dev())
    ps.reconstruct_stacked_(out, P, Q)
    check_kernel_errors()
    ref_o = P.double() @ Q.double().transpose(1, 2)
    assert (out.double() - ref_o).abs().max().item() <= 2e-3 * ref_o.abs().max().item() + 1e-2


def test_powersgd_round_on_rank_deficient_gradient_matches_gram_schmidt_math():
    """A gradient of true rank 8 compressed with r = 32: P = M Q has 24 dependent columns. The reference normalises
    whatever Gram-Schmidt leaves of them (hivemind/utils/math.py:6-14), the batched CholeskyQR2 kernel drops them;
    what matters is the gradient that comes out, g^ = P (M^T P)^T, which must be the same (here: M itself, since its
    column space is captured either way)."""
    from hivemind_b200.ops import powersgd as ps
    from hivemind_b200.utils.math import orthogonalize_reference_

    torch.manual_seed(29)
    m, n, r = 1024, 512, 32
    M = (torch.randn(m, 8, device=_dev()) @ torch.randn(8, n, device=_dev())) / 8 ** 0.5
    Q = torch.randn(n, r, device=_dev())
    P = torch.empty(m, r, device=_dev())
    ps.compute_p_(P, M, Q)
    # reference math in fp64 on the host
    P_ref = orthogonalize_reference_((M.double() @ Q.double()).cpu())
    g_ref = P_ref @ (M.double().cpu().t() @ P_ref).t()
    # device path
    ps.orthogonalize_batch_([P])
    Q2 = torch.empty(n, r, device=_dev())
    ps.compute_q_(Q2, M, P)
    g = torch.empty(m, n, device=_dev())
    ps.reconstruct_(g, P, Q2)
    scale = M.abs().max().item()
    # the oracle recovers M up to what fp32 rounding of M adds outside its eight directions (about 6e-4 here)
    assert (g_ref - M.double().cpu()).abs().max().item() < 2e-3 * scale
    assert (g.double().cpu() - g_ref).abs().max().item() < 5e-3 * scale, (g.double().cpu() - g_ref).abs().max().item()
