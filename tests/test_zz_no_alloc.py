"""The allocation-free sampler against the regular one.

Some users of this library cannot allocate device memory when they sample (a serving loop with a
fixed memory plan, or a host runtime that owns all device memory), so they cannot give
``b200_sample_topk`` its scratch buffer.  ``b200_sample_topk_noalloc`` keeps the scratch inside the
library.  This test calls it through its exported C symbol, twice in a row (the second call finds
the first call's leftovers in the shared scratch), and checks that it picks the same tokens as the
regular entry point, and that it refuses a problem larger than its built-in scratch.

The file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _fn():
    from openagents_b200 import _native
    L = _native.cuda()
    f = L.b200_sample_topk_noalloc
    f.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_int, ctypes.c_float,
                  ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    f.restype = ctypes.c_int
    return f


def test_noalloc_sampler_matches_regular_sampler_twice():
    from openagents_b200.ops import cuda_ops as ops
    f = _fn()
    dev = "cuda"
    st = torch.cuda.current_stream().cuda_stream
    for call, (T, V, k, p, temp) in enumerate([(4, 50257, 8, 0.9, 0.8), (3, 32000, 5, 1.0, 1.3)]):
        g = torch.Generator(device=dev).manual_seed(100 + call)
        logits = torch.randn(T, V, generator=g, device=dev) * 3
        u = torch.rand(T, generator=g, device=dev)
        ref = torch.zeros(T, dtype=torch.int32, device=dev)
        scratch = torch.empty((T, V), device=dev)
        ops.sample_topk(logits, temp, k, p, u, ref, scratch)
        out = torch.full((T,), -1, dtype=torch.int32, device=dev)
        before = torch.cuda.memory_allocated()
        rc = f(logits.data_ptr(), T, V, temp, k, p, u.data_ptr(), out.data_ptr(), st)
        torch.cuda.synchronize()
        assert rc == 0
        assert torch.cuda.memory_allocated() == before
        assert torch.equal(out, ref), (call, out.tolist(), ref.tolist())
        assert all(int(out[t]) in logits[t].topk(k).indices.tolist() for t in range(T))


def test_noalloc_sampler_rejects_oversize_and_bad_arguments():
    f = _fn()
    x = torch.zeros(8, device="cuda")
    o = torch.zeros(8, dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    assert f(x.data_ptr(), 64, 128256, 1.0, 4, 1.0, x.data_ptr(), o.data_ptr(), st) == -1     # 8.2M floats > 2M
    assert f(x.data_ptr(), 1, 8, 1.0, 0, 1.0, x.data_ptr(), o.data_ptr(), st) == -2
    assert f(x.data_ptr(), 0, 8, 1.0, 1, 1.0, x.data_ptr(), o.data_ptr(), st) == -2
    assert f(x.data_ptr(), 1, 8, 1.0, 9, 1.0, x.data_ptr(), o.data_ptr(), st) == -2            # more candidates than entries


def test_noalloc_sampler_gives_a_defined_id_for_rows_without_finite_logits():
    f = _fn()
    V = 4096
    logits = torch.full((2, V), float("nan"), device="cuda")
    logits[1] = float("-inf")
    logits[1, 77] = 0.5                      # one finite entry: it must win whatever top_k says
    u = torch.rand(2, device="cuda")
    out = torch.full((2,), -1, dtype=torch.int32, device="cuda")
    rc = f(logits.data_ptr(), 2, V, 1.0, 8, 1.0, u.data_ptr(), out.data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 0 and out.tolist() == [0, 77]
    torch.cuda.synchronize()
