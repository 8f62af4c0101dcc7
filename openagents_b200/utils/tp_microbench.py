"""Device-time micro-benchmarks of the tensor-parallel building blocks, one process per GPU:

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m openagents_b200.utils.tp_microbench

Each case is captured in a CUDA graph of 20 back-to-back launches and replayed, so the figure is the
steady-state cost of one launch in a stream of them (CUDA events, maximum over ranks; every rank runs the same
sequence).  A row-parallel projection is timed TOGETHER with the RMSNorm that consumes its result, in two forms: the
slot all-reduce (the projection keeps its partial result local; the norm pushes each row into every rank's slots, raises
and awaits the row's flag and sums) and the same pair with a local residual add (no communication).  The difference to the local pair is what
the collective costs; the roofline column is the larger of the packed weight bytes over the measured copy bandwidth
and the bytes that must arrive over NVLink over 770 GB/s.
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
    hn = torch.empty((64, eng.d), dtype=torch.bfloat16, device=dev)
    for t in (eng.fq, eng.fs, eng.xq, eng.xs):
        t.zero_()
    eng.fd.fill_(1.0)
    eng.xd.fill_(1.0)
    table, slot = comm.heap.table, (comm.heap.table, eng.slots_off, eng.slot_rows, eng.xpart)
    gain = L.ffn_norm
    eps = cfg.norm_eps

    def mv(w, q, d, s_, f, epi, **kw):
        ops.matvec(w.wt, w.main, w.plane2, w.N, w.K, 1, xq=q, xd=d, xs16=s_, xf=f, epi=epi, ldy=eng.d, **kw)

    def norm(rows, **kw):
        ops.rmsnorm(rows, gain, eps, hb=hn[: rows.shape[0]], **kw)

    def pair_mv(w, q, d, s_, f, mode):
        if mode == "slots":
            mv(w, q, d, s_, f, ops.EPI_STORE, y=eng.xpart)
            norm(x1, slots=slot)
        elif mode == "allreduce":
            comm.matvec_allreduce(w, 1, q, d, s_, f, x1, eng.d, wait_ready=True)
            norm(x1, signal_sym=table)
        else:
            mv(w, q, d, s_, f, ops.EPI_RESID, resid=x1, y=x1)
            norm(x1)

    def pair_q(w, a_, mode):
        if mode == "slots":
            ops.qgemm(w, a_, 64, out_f32=eng.xpart, ldo=eng.d, epi=ops.QEPI_ADD, status=eng.status)
            norm(x, slots=slot)
        elif mode == "allreduce":
            comm.gemm_allreduce(a_, eng._dense(w), 64, x, status=eng.status, wait_ready=True)
            norm(x, signal_sym=table)
        else:
            ops.qgemm(w, a_, 64, out_f32=x, ldo=eng.d, epi=ops.QEPI_ADD, status=eng.status)
            norm(x)

    cases = {"barrier": (lambda: comm.heap.barrier(ch=2), 0, 0)}
    for wname, w, q, d_, s_, f, a_ in (("wo", L.wo, eng.xq, eng.xd, eng.xs, eng.xf, hq), ("down", L.wdown, eng.fq, eng.fd, eng.fs, eng.gu, hb)):
        for mode in ("slots", "local"):
            cases[f"{wname:4s} mat-vec (1 token) + norm, {mode}"] = ((lambda w=w, q=q, d_=d_, s_=s_, f=f, mode=mode: pair_mv(w, q, d_, s_, f, mode)),
                                                                    w.nbytes(), (world - 1) * eng.d * 4 if mode != "local" else 0)
            cases[f"{wname:4s} GEMM (64 tokens) + norm, {mode}"] = ((lambda w=w, a_=a_, mode=mode: pair_q(w, a_, mode)),
                                                                   w.nbytes(), (world - 1) * 64 * eng.d * 4 if mode != "local" else 0)
    reps = 20
    hbm = 6546e9
    for name, (fn, wbytes, link_bytes) in cases.items():
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            fn()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=s):
                for _ in range(reps):
                    fn()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(10):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) * 1000 / (10 * reps)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            roof = max(wbytes / hbm, link_bytes / 770e9) * 1e6
            print(f"{name:45s} {t.item():7.1f} us" + (f"   roofline {roof:5.1f} us  ({roof / t.item():4.2f})" if roof else ""), flush=True)
    if rank == 0:
        print("heap status", comm.heap.status(), "multicast", comm.heap.uses_multicast)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
