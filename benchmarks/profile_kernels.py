"""Runs ONE kernel of the package a few times on a small, fixed case, for timing with CUDA events or for a profiler.

    python benchmarks/profile_kernels.py --kernel gemm --m 16384 --n 4096 --k 1024
    python benchmarks/profile_kernels.py --kernel ln_bwd --rows 32768 --hidden 1024

Prints the mean device time of the timed launches (CUDA events; an L2-sized buffer is rewritten between launches)
and the implied throughput. Under a profiler, capture by kernel name (tc_gemm_kernel, ln_bwd_kernel, ...).
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from hivemind_b200.ops.gemm import check_kernel_errors, linear, tc_gemm
from hivemind_b200.ops.norm_act import layer_norm


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--kernel", required=True,
                        choices=["gemm", "gemm_dw", "gemm_compare", "ln_fwd", "ln_bwd", "gelu_bwd", "attention_compare",
                                 "codec", "lamb", "powersgd", "ffn"])
    parser.add_argument("--codec", default="uniform8", help="codec mode: float16, meanstd16, uniform8, quantile8 or blockwise8")
    parser.add_argument("--mb", type=float, default=256.0, help="codec / lamb modes: megabytes of fp32 data")
    parser.add_argument("--batch", type=int, default=32)
    parser.add_argument("--seq", type=int, default=512)
    parser.add_argument("--heads", type=int, default=16)
    parser.add_argument("--causal", action="store_true")
    parser.add_argument("--skip-library", action="store_true", help="attention_compare: time only this package's kernels")
    parser.add_argument("--m", type=int, default=16384)
    parser.add_argument("--n", type=int, default=4096)
    parser.add_argument("--k", type=int, default=1024)
    parser.add_argument("--rows", type=int, default=32768)
    parser.add_argument("--hidden", type=int, default=1024)
    parser.add_argument("--iters", type=int, default=5)
    parser.add_argument("--warmup", type=int, default=2)
    parser.add_argument("--pair", action="store_true", help="gemm kernels: use the two-CTA (cta_group::2) kernel")
    args = parser.parse_args()
    dev = torch.device("cuda")
    torch.manual_seed(0)
    flush = torch.empty(256 * 2 ** 20, dtype=torch.uint8, device=dev)  # larger than the 126 MB L2

    if args.kernel == "gemm_compare":
        # one-CTA kernel, two-CTA kernel and torch.matmul (cuBLAS) on the same tensors, back to back
        a = torch.randn(args.m, args.k, device=dev, dtype=torch.bfloat16)
        b = torch.randn(args.n, args.k, device=dev, dtype=torch.bfloat16)
        out = torch.empty(args.m, args.n, device=dev, dtype=torch.bfloat16)
        variants = {"one_cta": lambda: tc_gemm(a, b, out=out, pair=False), "two_cta": lambda: tc_gemm(a, b, out=out, pair=True),
                    "cublas": lambda: torch.matmul(a, b.t(), out=out)}
        result = {}
        for name, fn in variants.items():
            for _ in range(max(args.warmup, 3)):
                fn()
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(args.iters):
                fn()
            stop.record()
            torch.cuda.synchronize()
            result[name] = 2.0 * args.m * args.n * args.k / (start.elapsed_time(stop) / args.iters / 1e3) / 1e12
        check_kernel_errors()
        print(json.dumps({"kernel": "gemm_compare", "tflops": result, "m": args.m, "n": args.n, "k": args.k,
                          "iters": args.iters, "note": "launches back to back, no L2 flush"}))
        return
    if args.kernel == "attention_compare":
        # this package's tcgen05 attention and PyTorch's scaled_dot_product_attention (library kernels) on the same
        # packed projections, forward and forward+backward, L2 rewritten before every timed call
        from hivemind_b200.ops.attention import attention

        b, s, nh = args.batch, args.seq, args.heads
        qkv = torch.randn(b, s, 3 * nh * 64, device=dev, dtype=torch.bfloat16, requires_grad=True)
        dout = torch.randn(b, s, nh * 64, device=dev, dtype=torch.bfloat16)

        def ours():
            return attention(qkv, nh, causal=args.causal)

        def library():
            q, k, v = (t.transpose(1, 2) for t in qkv.view(b, s, 3, nh, 64).unbind(2))
            ctx = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=args.causal)
            return ctx.transpose(1, 2).reshape(b, s, nh * 64)

        def timed(fn):
            for _ in range(max(args.warmup, 3)):
                fn()
            torch.cuda.synchronize()
            total = 0.0
            for _ in range(args.iters):
                flush.fill_(1)
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                fn()
                stop.record()
                torch.cuda.synchronize()
                total += start.elapsed_time(stop)
            return total / args.iters

        flops_fwd = 4.0 * b * nh * s * s * 64 * (0.5 if args.causal else 1.0)
        result = {}
        for name, fn in (("ours", ours),) if args.skip_library else (("ours", ours), ("library", library)):
            fwd_ms = timed(fn)
            both_ms = timed(lambda: torch.autograd.grad(fn(), qkv, dout))
            result[name] = {"fwd_ms": fwd_ms, "fwd_tflops": flops_fwd / fwd_ms / 1e9, "fwd_bwd_ms": both_ms,
                            "bwd_ms": both_ms - fwd_ms, "bwd_tflops": 2.5 * flops_fwd / max(both_ms - fwd_ms, 1e-6) / 1e9}
        check_kernel_errors()
        print(json.dumps({"kernel": "attention_compare", "batch": b, "seq": s, "heads": nh, "causal": args.causal,
                          "result": result, "note": "library = scaled_dot_product_attention including the transposes "
                                                    "and the stacked q/k/v gradient that surround it in a model"}))
        return
    if args.kernel == "codec":
        # whole-tensor encoders of ops/codec.py (statistics / borders / encode kernels of ops/csrc/codec.cu)
        from hivemind_b200.compression.quantization import dynamic_code_table
        from hivemind_b200.ops import codec as codecs

        x = torch.randn(int(args.mb * 2 ** 20 / 4), device=dev)
        code = dynamic_code_table().to(dev) if args.codec == "blockwise8" else None
        run = {"float16": lambda: codecs.encode_float16(x), "meanstd16": lambda: codecs.encode_scaled_float16(x),
               "uniform8": lambda: codecs.encode_uniform8(x), "quantile8": lambda: codecs.encode_quantile8(x),
               "blockwise8": lambda: codecs.encode_blockwise8(x, code)}[args.codec]
        work = 4.0 * x.numel() * (1.5 if args.codec in ("float16", "meanstd16") else 1.25)  # read fp32, write the code
        unit = "GB/s"
    elif args.kernel == "lamb":
        # one fused LAMB step over ALBERT-large-like parameters (fp32 master weights, bf16 model copy)
        from hivemind_b200.optim.fused import FusedLAMB

        n = int(args.mb * 2 ** 20 / 4)
        params = [torch.randn(n // 8, device=dev, requires_grad=True) for _ in range(8)]
        for p in params:
            p.grad = torch.randn_like(p)
        opt = FusedLAMB(params, lr=1e-3, weight_decay=0.01)
        run = opt.step
        work = 4.0 * n * 7  # read p, g, m, v; write p, m, v
        unit = "GB/s"
    elif args.kernel == "powersgd":
        # one PowerSGD compression of a stack of 24 matrices of 1024 x 4096 at rank 32: P = M Q, orthogonalise, Q = M^T P
        from hivemind_b200.ops import powersgd as ps

        groups, rows, cols, r = 24, 1024, 4096, 32
        m = torch.randn(groups, rows, cols, device=dev)
        q = torch.randn(groups, cols, r, device=dev)
        p_ = torch.empty(groups, rows, r, device=dev)

        def run():
            ps.compute_p_stacked_(p_, m, q)
            ps.orthogonalize_batch_(list(p_.unbind(0)))
            ps.compute_q_stacked_(q, m, p_)

        work = 2 * 2.0 * groups * rows * cols * r
        unit = "TFLOP/s"
    elif args.kernel == "ffn":
        # forward + backward of the feed-forward node (four GEMMs each way, GELU derivative and residual gradient in
        # GEMM epilogues) on ALBERT-large's shapes
        from hivemind_b200.ops.gemm import feed_forward

        x = torch.randn(args.rows // 2, args.hidden, device=dev, dtype=torch.bfloat16, requires_grad=True)
        w1 = (torch.randn(4 * args.hidden, args.hidden, device=dev) * 0.02).requires_grad_()
        w2 = (torch.randn(args.hidden, 4 * args.hidden, device=dev) * 0.02).requires_grad_()
        b1, b2 = torch.zeros(4 * args.hidden, device=dev, requires_grad=True), torch.zeros(args.hidden, device=dev, requires_grad=True)
        for t in (w1, w2, b1, b2):
            t.grad = torch.zeros_like(t)
        w1_lp, w2_lp = w1.detach().bfloat16(), w2.detach().bfloat16()
        dout = torch.randn(args.rows // 2, args.hidden, device=dev, dtype=torch.bfloat16)

        def run():
            out, skip = feed_forward(x, w1, b1, w2, b2, w1_lp=w1_lp, w2_lp=w2_lp, passthrough=True)
            torch.autograd.backward([out, skip], [dout, dout])

        work = 6 * 2.0 * (args.rows // 2) * args.hidden * 4 * args.hidden
        unit = "TFLOP/s"
    elif args.kernel == "gemm":
        a = torch.randn(args.m, args.k, device=dev, dtype=torch.bfloat16)
        b = torch.randn(args.n, args.k, device=dev, dtype=torch.bfloat16)
        out = torch.empty(args.m, args.n, device=dev, dtype=torch.bfloat16)
        run = lambda: tc_gemm(a, b, out=out, pair=args.pair)
        work = 2.0 * args.m * args.n * args.k
        unit = "TFLOP/s"
    elif args.kernel == "gemm_dw":
        a = torch.randn(args.k, args.m, device=dev, dtype=torch.bfloat16)  # [tokens, out]
        b = torch.randn(args.k, args.n, device=dev, dtype=torch.bfloat16)  # [tokens, in]
        out = torch.zeros(args.m, args.n, device=dev, dtype=torch.float32)
        run = lambda: tc_gemm(a, b, a_mn=True, b_mn=True, out=out, reduce_add=True, splits=4, pair=args.pair)
        work = 2.0 * args.m * args.n * args.k
        unit = "TFLOP/s"
    else:
        x = torch.randn(args.rows, args.hidden, device=dev, dtype=torch.bfloat16, requires_grad=True)
        res = torch.randn(args.rows, args.hidden, device=dev, dtype=torch.bfloat16)
        gamma = torch.ones(args.hidden, device=dev, requires_grad=True)
        beta = torch.zeros(args.hidden, device=dev, requires_grad=True)
        nbytes = args.rows * args.hidden * 2
        if args.kernel == "ln_fwd":
            run = lambda: layer_norm(x.detach(), gamma.detach(), beta.detach(), 1e-12, residual=res)
            work = 4.0 * nbytes  # read x, residual; write y, z
        elif args.kernel == "ln_bwd":
            y = layer_norm(x, gamma, beta, 1e-12, residual=res)
            dy = torch.randn_like(y)
            run = lambda: torch.autograd.grad(y, x, dy, retain_graph=True)
            work = 3.0 * nbytes  # read dy, z; write dx
        else:
            bias = torch.zeros(args.hidden, device=dev, requires_grad=True)
            w = torch.randn(args.hidden, 64, device=dev, requires_grad=True)
            inp = torch.randn(args.rows, 64, device=dev, dtype=torch.bfloat16)
            y = linear(inp, w, bias, activation="gelu")
            dy = torch.randn_like(y)
            run = lambda: torch.autograd.grad(y, w, dy, retain_graph=True)
            work = 3.0 * nbytes
        unit = "GB/s"

    for _ in range(args.warmup):
        run()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(args.iters):
        flush.fill_(1)
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        run()
        stop.record()
        torch.cuda.synchronize()
        total += start.elapsed_time(stop)
    check_kernel_errors()
    ms = total / args.iters
    scale = 1e12 if unit == "TFLOP/s" else 1e9
    print(json.dumps({"kernel": args.kernel, "ms": ms, "throughput": work / (ms / 1e3) / scale, "unit": unit,
                      "note": "ln_bwd / gelu_bwd times include the other kernels of that autograd node",
                      "args": vars(args)}))


if __name__ == "__main__":
    main()
