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
                        choices=["gemm", "gemm_dw", "gemm_compare", "ln_fwd", "ln_bwd", "gelu_bwd"])
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
    if args.kernel == "gemm":
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
