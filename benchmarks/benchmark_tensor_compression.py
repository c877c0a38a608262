"""Time, distortion and size of every wire codec on one tensor (reference: benchmarks/benchmark_tensor_compression.py).

On a CUDA tensor (``--device cuda``) the encoders are the device kernels of ``hivemind_b200.ops.codec``; on CPU the
PyTorch reference codecs. Prints one JSON line per codec.
"""
import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch

from hivemind_b200.compression import deserialize_torch_tensor, serialize_torch_tensor
from hivemind_b200.proto.runtime_pb2 import CompressionType


def benchmark_compression(tensor: torch.Tensor, compression_type: int):
    if tensor.is_cuda:
        torch.cuda.synchronize()
    started = time.perf_counter()
    serialized = serialize_torch_tensor(tensor, compression_type)
    restored = deserialize_torch_tensor(serialized)
    elapsed = time.perf_counter() - started
    error = (tensor.detach().float().cpu() - restored.float()).square().mean().item()
    return elapsed, error, serialized.ByteSize()


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--size", type=int, default=10_000_000)
    parser.add_argument("--seed", type=int, default=7348)
    parser.add_argument("--num_iters", type=int, default=30)
    parser.add_argument("--device", default="cpu")
    args = parser.parse_args()
    torch.manual_seed(args.seed)
    x = torch.randn(args.size, dtype=torch.float32, device=args.device)
    for name, compression_type in CompressionType.items():
        results = [benchmark_compression(x, compression_type) for _ in range(args.num_iters)]
        seconds = sum(r[0] for r in results) / len(results)
        print(json.dumps({"benchmark": "tensor_compression", "compression": name, "seconds": seconds,
                          "mse": sum(r[1] for r in results) / len(results), "bytes": int(results[0][2]),
                          "input_gb_per_s": x.numel() * 4 / seconds / 1e9, "device": args.device,
                          "elements": args.size}), flush=True)
