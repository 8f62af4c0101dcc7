"""Device-time micro-benchmarks of the tensor-parallel building blocks, one process per GPU:

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m openagents_b200.utils.tp_microbench

Each case is captured in a CUDA graph of 20 back-to-back launches and replayed, so the figure is the
steady-state cost of one launch in a stream of them (CUDA events on rank 0; every rank runs the same
sequence).  Cases: the stand-alone flag barrier, the row-parallel mat-vec with the all-reduce fused into
its epilogue against the same mat-vec with a local residual add, and the same pair for the 64-token
tensor-core GEMM.  The difference between a fused case and its local twin is what the collective costs.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    from ..models.config import LLAMA3_8B
    from ..models.engine import LlamaEngine
    from ..models.qweight import RandomSource
    from ..models.weights import PLAN_Q4_K
    from ..ops import cuda_ops as ops
    from ..parallel.tp import TPComm
    comm = TPComm(rank, world, dev)
    cfg = LLAMA3_8B.with_(n_layers=1)
    eng = LlamaEngine(cfg, RandomSource(cfg, PLAN_Q4_K, 0, dev), device=dev, max_batch=64, max_ctx=256, max_tokens=256, tp_rank=rank,
                      tp_world=world, comm=comm)
    L = eng.layers[0]
    x, x1 = eng.x[:64], eng.x[:1]
    hb = torch.randn(64, L.wdown.K, device=dev).bfloat16()
    hq = torch.randn(64, L.wo.K, device=dev).bfloat16()
    for t in (eng.fq, eng.fs, eng.xq, eng.xs):
        t.zero_()
    eng.fd.fill_(1.0)
    eng.xd.fill_(1.0)
    mv = lambda w, q, d, s, f, epi, **kw: ops.matvec(w.wt, w.main, w.plane2, w.N, w.K, 1, xq=q, xd=d, xs16=s, xf=f, epi=epi, y=x1, ldy=eng.d, **kw)
    cases = {
        "barrier": lambda: comm.heap.barrier(ch=2),
        "matvec wo   + fused all-reduce (1 token)": lambda: comm.matvec_allreduce(L.wo, 1, eng.xq, eng.xd, eng.xs, eng.xf, x1, eng.d),
        "matvec wo   local residual add": lambda: mv(L.wo, eng.xq, eng.xd, eng.xs, eng.xf, ops.EPI_RESID, resid=x1),
        "matvec down + fused all-reduce (1 token)": lambda: comm.matvec_allreduce(L.wdown, 1, eng.fq, eng.fd, eng.fs, eng.gu, x1, eng.d),
        "matvec down local residual add": lambda: mv(L.wdown, eng.fq, eng.fd, eng.fs, eng.gu, ops.EPI_RESID, resid=x1),
        "gemm wo   + fused all-reduce (64 tokens)": lambda: comm.gemm_allreduce(hq, eng._dense(L.wo), 64, x, status=eng.status),
        "gemm wo   local residual add": lambda: ops.gemm_bf16(hq, eng._dense(L.wo), 64, L.wo.N, L.wo.K, out_f32=x, resid_f32=x, ldc=eng.d, status=eng.status),
        "gemm down + fused all-reduce (64 tokens)": lambda: comm.gemm_allreduce(hb, eng._dense(L.wdown), 64, x, status=eng.status),
        "gemm down local residual add": lambda: ops.gemm_bf16(hb, eng._dense(L.wdown), 64, L.wdown.N, L.wdown.K, out_f32=x, resid_f32=x, ldc=eng.d,
                                                              status=eng.status),
    }
    reps = 20
    for name, fn in cases.items():
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            fn()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                for _ in range(reps):
                    fn()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(10):
            g.replay()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) * 1000 / (10 * reps)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            print(f"{name:45s} {t.item():7.1f} us", flush=True)
    if rank == 0:
        print("heap status", comm.heap.status(), "multicast", comm.heap.uses_multicast)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
