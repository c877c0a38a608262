"""The tcgen05 attention kernels against a plain PyTorch fp32 attention of the same inputs, and the CPU path."""
import math

import pytest
import torch

from hivemind_b200.ops.attention import attention, kernel_supports, reference_attention


def test_reference_attention_matches_sdpa_on_cpu():
    torch.manual_seed(0)
    b, s, nh, d = 2, 37, 3, 16
    qkv = torch.randn(b, s, 3 * nh * d, requires_grad=True)
    for causal in (False, True):
        got = attention(qkv, nh, causal=causal)  # CPU tensors take the PyTorch formula
        q, k, v = (t.transpose(1, 2) for t in qkv.view(b, s, 3, nh, d).unbind(2))
        want = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=causal)
        want = want.transpose(1, 2).reshape(b, s, nh * d)
        assert torch.allclose(got, want, atol=1e-5, rtol=1e-5)
    assert not kernel_supports(qkv, nh)


def _fp32_oracle(qkv, dout, nh, causal):
    ref_in = qkv.detach().float().requires_grad_()
    ref = reference_attention(ref_in, nh, causal)
    ref.backward(dout.float())
    return ref.detach(), ref_in.grad


@pytest.mark.gpu
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("shape", [(2, 128, 2), (3, 512, 4), (2, 1024, 2), (2, 200, 3), (1, 64, 1), (2, 333, 2)])
def test_attention_kernel_forward_backward(shape, causal):
    b, s, nh = shape
    dev = torch.device("cuda", 0)
    torch.manual_seed(s + nh + int(causal))
    qkv = (torch.randn(b, s, 3 * nh * 64, device=dev) * 1.5).to(torch.bfloat16).requires_grad_()
    assert kernel_supports(qkv, nh)
    out = attention(qkv, nh, causal=causal)
    dout = torch.randn_like(out)
    out.backward(dout)
    torch.cuda.synchronize()
    ref, ref_grad = _fp32_oracle(qkv, dout, nh, causal)
    assert out.shape == (b, s, nh * 64) and out.dtype == torch.bfloat16
    # bf16 outputs: half a unit in the last place of values around 1 is 4e-3; P is rounded to bf16 before P V
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2), float((out.float() - ref).abs().max())
    err = (out.float() - ref).pow(2).mean().sqrt() / ref.pow(2).mean().sqrt()
    assert err < 1e-2, f"relative rms error of the forward output {err}"
    grad = qkv.grad.float()
    hidden = nh * 64
    for name, lo in (("dq", 0), ("dk", hidden), ("dv", 2 * hidden)):
        g, r = grad[..., lo:lo + hidden], ref_grad[..., lo:lo + hidden]
        rel = (g - r).pow(2).mean().sqrt() / r.pow(2).mean().sqrt()
        assert rel < 2e-2, f"{name}: relative rms error {rel}"
        assert torch.allclose(g, r, atol=0.05 * float(r.abs().max()), rtol=5e-2), f"{name}: {float((g - r).abs().max())}"


@pytest.mark.gpu
def test_attention_kernel_custom_scale_and_repeatability():
    dev = torch.device("cuda", 0)
    torch.manual_seed(5)
    qkv = torch.randn(2, 256, 3 * 2 * 64, device=dev).to(torch.bfloat16)
    a = attention(qkv, 2, causal=True, scale=0.05)
    b = attention(qkv, 2, causal=True, scale=0.05)
    assert torch.equal(a, b)
    ref = reference_attention(qkv.float(), 2, True, 0.05)
    assert torch.allclose(a.float(), ref, atol=2e-2, rtol=2e-2)
    assert not torch.allclose(a.float(), reference_attention(qkv.float(), 2, True, 1 / math.sqrt(64)), atol=2e-2)
