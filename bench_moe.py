#!/usr/bin/env python
"""Expert-parallel MoE serving benchmark (gpt-oss-20b shape): prefill of one 4096-token chunk per rank,
then decode at a global batch of 256 sequences.

    python bench_moe.py --gpus N --steps K --warmup W        # N > 1: launched with torch.distributed.run

Attention is data-parallel (each rank serves ``256 / N`` sequences), experts are sharded ``32 / N`` per
rank; every layer runs the fused router+dispatch kernel and the two grouped tcgen05 GEMMs.  Synthetic
token ids, seeded N(0, 0.02) weights, MXFP4 expert blocks expanded to bf16 at load.  Prints one JSON
line on rank 0; timing is CUDA events on the launching stream, maximum over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import time


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--batch", type=int, default=256, help="global decode batch")
    ap.add_argument("--prefill", type=int, default=4096)
    ap.add_argument("--context", type=int, default=4096, help="tokens each decode sequence holds before the timed steps")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (debugging only; marks the run invalid)")
    return ap.parse_args()


def run(args) -> dict | None:
    """The benchmark proper; the process group (when WORLD_SIZE > 1) must already exist.  Returns the record on rank 0."""
    K, W = args.steps, max(args.warmup, 3)

    import torch
    import torch.distributed as dist
    from bench import ClockSampler
    from openagents_b200.models.config import GPT_OSS_20B
    from openagents_b200.models.engine import PAGE
    from openagents_b200.models.moe_engine import MoEEngine
    from openagents_b200.models.qweight import RandomSource
    from openagents_b200.models.weights import PLAN_MOE

    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local)
    cfg, valid = GPT_OSS_20B, True
    if args.layers:
        cfg, valid = cfg.with_(n_layers=args.layers), False
    B = args.batch // world
    P = args.prefill
    max_ctx = max(P, args.context + 2 * (K + W) + 8) + PAGE
    n_pages = B * ((args.context + 2 * (K + W) + 8 + PAGE) // PAGE + 1) + P // PAGE + 8
    t0 = time.time()
    eng = MoEEngine(cfg, RandomSource(cfg, PLAN_MOE, 0, dev), device=dev, max_batch=B + 1, max_ctx=max_ctx, n_pages=n_pages,
                    max_tokens=P, ep_rank=rank, ep_world=world)
    load_s = time.time() - t0

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    g = torch.Generator().manual_seed(77 + rank)
    # ---- prefill: one chunk of P tokens per rank (all ranks at once: the experts see P * world tokens)
    prompt = torch.randint(0, cfg.vocab, (P,), generator=g).tolist()
    eng.begin(B)
    eng.forward_tokens([B], [prompt[:64]])
    eng.end(B)
    ttft = []
    for rep in range(3):
        eng.begin(B)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        eng.forward_tokens([B], [prompt])
        e1.record()
        barrier()
        ttft.append(max_over_ranks(e0.elapsed_time(e1)))
        eng.end(B)
    prefill_ms = min(ttft[1:])

    # ---- decode sequences: B per rank, `context` tokens each (untimed prefill in groups)
    per = max(1, P // args.context)
    first = []
    for b0 in range(0, B, per):
        ids = list(range(b0, min(B, b0 + per)))
        for i in ids:
            eng.begin(i)
        _, nxt = eng.forward_tokens(ids, [torch.randint(0, cfg.vocab, (args.context,), generator=g).tolist() for _ in ids])
        first += nxt.tolist()
    eng.check_status()
    seqs = list(range(B))
    hist = eng.decode_steps(seqs, first, W)
    last = hist[W - 1].tolist()
    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    marks = {0: e0}
    hist = eng.decode_steps(seqs, last, K, on_replay=lambda i: marks[i].record() if i in marks else None)
    e1.record()
    barrier()
    clocks = sampler.stop()
    dev_ms = max_over_ranks(e0.elapsed_time(e1)) / K
    launches = eng.launches_per_decode * K
    last = hist[K - 1].tolist()
    eng.check_status()

    # ---- end to end through engine.decode(): per step H2D of the ids/positions, D2H of the new ids
    for _ in range(W):
        _, nxt = eng.decode(seqs, last)
        last = nxt.tolist()
    barrier()
    h2d_before = eng.h2d_bytes
    t0 = time.perf_counter()
    for _ in range(K):
        _, nxt = eng.decode(seqs, last)
        last = nxt.tolist()
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1000) / K
    eng.check_status()
    h2d = (eng.h2d_bytes - h2d_before) // K        # counted by the engine from the tensors it copies: ids, pos, slot,
                                                   # lengths every step, page-table rows when a sequence takes a new page
    if rank != 0:
        return None
    if True:
        return ({
            "metric": "gpt_oss_20b_moe_decode_tok_s_bs256", "value": round(args.batch / dev_ms * 1000, 1), "unit": "tokens/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": round(dev_ms, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"model": cfg.name, "weights": "experts MXFP4 (expanded to bf16 at load), attention/router bf16/fp32, seeded N(0,0.02)",
                       "global_batch": args.batch, "decode_context": args.context, "prefill_tokens_per_rank": P,
                       "parallelism": f"ep{world} (data-parallel attention)", "placement_digest": eng.placement_digest(),
                       "l2": "inputs larger than L2 (expert weights >> 126 MB)", "valid": valid},
            "clocks": clocks,
            "e2e": {"value": round(args.batch / e2e_ms * 1000, 1), "unit": "tokens/s", "ms_per_step": round(e2e_ms, 4),
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * B},
            "gpu_launches": launches,
            "extra": {"prefill_ms_per_chunk": round(prefill_ms, 3), "prefill_tok_s": round(P * world / prefill_ms * 1000, 1),
                      "load_s": round(load_s, 1), "weight_bytes_per_gpu": eng.weight_bytes()}})


def main():
    args = parse()
    import torch
    import torch.distributed as dist
    world, local = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    out = run(args)
    if out is not None:
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
