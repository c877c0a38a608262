"""The allocation-free clipping entry point, called through its exported C symbol.

It exists for programs that cannot allocate device memory when they call into the library (a runtime that owns all
of HBM through its own pool, a plain C host). The test compares it with the regular path
(``multi_tensor.clip_grad_norm_``: caller-allocated sums) on two calls in a row — the second one with other data and
fewer tensors, which would go wrong if the shared scratch array were not cleared — and checks that oversized calls
are refused. This file sorts last on purpose, so that a failure here cannot hide another test's result.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, tensors, max_norm):
    from hivemind_b200.ops import multi_tensor as mt

    table = mt.make_table(tensors)  # the table is an input of the call; preparing it is the caller's business
    norm_out = torch.zeros(1, device=tensors[0].device)
    fn = lib.hm_mt_clip_grad_norm_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_void_p,
                   ctypes.c_void_p]
    stream = torch.cuda.current_stream(tensors[0].device).cuda_stream
    rc = fn(table.tensors_dev.data_ptr(), table.chunks_dev.data_ptr(), table.num_chunks, len(tensors), max_norm,
            norm_out.data_ptr(), stream)
    return rc, norm_out


def test_noalloc_clip_matches_regular_path_twice_in_a_row():
    from hivemind_b200.ops import _lib
    from hivemind_b200.ops import multi_tensor as mt

    lib = ctypes.CDLL(str(_lib._build.KERNELS_SO))  # resolved through the exported symbol, not a Python wrapper
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    rounds = [([(1000, 33), (77,), (40000,), (5, 5, 5)], 1.5), ([(513,), (64, 64)], 0.25)]
    for shapes, max_norm in rounds:
        grads = [torch.randn(s, device=dev) * 3 for s in shapes]
        expected = [g.clone() for g in grads]
        expected_norm = mt.clip_grad_norm_(expected, max_norm)
        rc, norm = _call_noalloc(lib, grads, max_norm)
        torch.cuda.synchronize()
        assert rc == 0
        assert torch.allclose(norm[0], expected_norm, rtol=1e-4)
        for got, want in zip(grads, expected):
            assert torch.allclose(got, want, rtol=1e-4, atol=1e-6)
        total = torch.sqrt(sum(g.float().pow(2).sum() for g in grads))
        assert abs(float(total) - max_norm) <= 1e-3 * max_norm
    # a call that fits keeps working when nothing needs clipping
    small = [torch.full((10,), 0.01, device=dev)]
    rc, norm = _call_noalloc(lib, small, 100.0)
    torch.cuda.synchronize()
    assert rc == 0 and torch.allclose(small[0], torch.full((10,), 0.01, device=dev))


def test_noalloc_clip_refuses_more_tensors_than_its_scratch_holds():
    from hivemind_b200.ops import _lib

    lib = ctypes.CDLL(str(_lib._build.KERNELS_SO))
    fn = lib.hm_mt_clip_grad_norm_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_void_p,
                   ctypes.c_void_p]
    rc = fn(None, None, 0, 4097, 1.0, None, None)
    assert rc == -20
