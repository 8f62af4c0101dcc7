"""HBM and NVLink bandwidth probes: the denominators of every roofline fraction the framework reports.

    python -m openagents_b200.utils.bandwidth_probe                       # one GPU: STREAM triad
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m openagents_b200.utils.bandwidth_probe                          # + peer pull / push / multicast push

Triad: ``a = b + s * c`` over three fp32 arrays of 1 GiB each (3 x 4 bytes per element cross HBM).
Peer copy: rank r reads from / writes to rank (r + 1) % world through the symmetric heap with plain
16-byte loads and stores issued by a kernel (the same instructions the fused kernels use), and with one
``multimem.st`` per 16 bytes where NVSwitch multicast is available.  CUDA events, best of 10, maximum
over ranks.  Reference for the memory case: apps/openagents.com/workers/api/src/cs336-a2-device-benchmark.ts:193-210
(STREAM triad, 2 M doubles x 8 passes on the host); the device-capability dataset stores the result
(apps/openagents.com/workers/api/src/training-device-capability.ts:24-29).
"""
from __future__ import annotations

import ctypes
import json
import os

import torch

from ..ops import cuda_ops as ops


def _best(fn, iters=10):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    best = 1e30
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) * 1e-3)
    return best


def stream_triad_gbs(device, n: int = 1 << 28) -> float:
    a, b, c = (torch.empty(n, dtype=torch.float32, device=device) for _ in range(3))
    b.fill_(1.0)
    c.fill_(2.0)
    lib = ops.lib()
    lib.b200_stream_triad.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_float, ctypes.c_size_t, ctypes.c_void_p]
    st = lambda: ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    s = _best(lambda: ops._check(lib.b200_stream_triad(a.data_ptr(), b.data_ptr(), c.data_ptr(), 3.0, n, st()), "stream_triad"))
    assert abs(float(a[12345]) - 7.0) < 1e-6
    return 3 * 4 * n / s / 1e9


def peer_copy_gbs(heap, peer: int, nbytes: int = 1 << 28) -> dict:
    lib = ops.lib()
    lib.b200_sym_peer_copy.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
    src, src_off = heap.alloc_tensor((nbytes,), torch.uint8)
    dst, dst_off = heap.alloc_tensor((nbytes,), torch.uint8)
    src.fill_(heap.rank + 1)
    heap.barrier()
    st = lambda: ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    out = {}
    modes = [("pull", 0), ("push", 1)] + ([("multicast_push", 2)] if heap.uses_multicast else [])
    for name, mode in modes:
        s = _best(lambda: ops._check(lib.b200_sym_peer_copy(ctypes.addressof(heap.table), peer, src_off, dst_off, nbytes, mode, st()), "peer_copy"))
        heap.barrier()
        out[name] = nbytes / s / 1e9
    return out


def main():
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    res = {"hbm_triad_gbs": round(stream_triad_gbs(dev), 1)}
    if world > 1:
        import torch.distributed as dist
        from ..parallel.symm import SymmHeap
        dist.init_process_group("nccl", device_id=dev)
        heap = SymmHeap((1 << 29) + (1 << 20), dev)
        res.update({f"nvlink_{k}_gbs": v for k, v in peer_copy_gbs(heap, (rank + 1) % world).items()})
        t = torch.tensor([res[k] for k in sorted(res)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)            # slowest rank = time maximum over ranks
        res = {k: round(float(v), 1) for k, v in zip(sorted(res), t.tolist())}
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps({"n_gpus": world, **res}))


if __name__ == "__main__":
    main()
