#!/usr/bin/env python
"""Training throughput: GPT-2-small-shape LM, data parallel with the sharded AdamW, global batch
512 sequences of 1024 tokens, bf16 compute with fp32 master weights, synthetic uniform token ids.

    python bench_train.py --steps K --warmup W                       (one GPU)
    python -m torch.distributed.run --nproc-per-node N ... bench_train.py --steps K --warmup W

A step is one optimizer step over the whole global batch (forward, backward, gradient
reduce-scatter, AdamW, parameter all-gather).  Each step's token ids are copied from pinned host
memory and the loss is read back, inside the timed region.  Prints one JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os


def run(steps: int, warmup: int, global_batch: int = 512, micro_batch: int = 16, seq_len: int = 1024, baseline: bool = True) -> dict | None:
    """Time ``steps`` optimizer steps after ``warmup``; the process group (when WORLD_SIZE > 1) must already exist.
    ``baseline``: afterwards time the same model, batch and optimizer on plain PyTorch (``baseline/gpt2_torch.py``: autocast,
    SDPA, fused AdamW, DDP) on the same GPUs and report the ratio as ``vs_baseline``.  Returns the result record on rank 0,
    None elsewhere."""
    import torch
    import torch.distributed as dist
    from bench import ClockSampler
    from openagents_b200.models.config import GPT2_SMALL
    from openagents_b200.train.trainer import TrainConfig, Trainer, synthetic_batch

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    cfg = TrainConfig(model=GPT2_SMALL, global_batch=global_batch, micro_batch=micro_batch, seq_len=seq_len)
    tr = Trainer(cfg, dev, rank, world)
    batches = [synthetic_batch(cfg, tr.accum, s, rank, dev) for s in range(2)]
    batches = [(a.pin_memory(), b.pin_memory()) for a, b in batches]

    def step(i):
        tok, tgt = batches[i % 2]
        tok, tgt = tok.to(dev, non_blocking=True), tgt.to(dev, non_blocking=True)      # host -> device, every step
        return float(tr.train_step(tok, tgt).item())                                    # device -> host read of the loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    losses = [step(i) for i in range(warmup)]
    tr.check_status()
    n0 = tr.model.kernel_launches
    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        losses.append(step(warmup + i))
    e1.record()
    barrier()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    tr.check_status()
    launches = tr.model.kernel_launches - n0
    accum = tr.accum
    base = None
    if baseline:
        del tr
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        try:
            from baseline.gpt2_torch import run_train_baseline
            b = run_train_baseline(cfg.model, dev, rank, world, batches, accum, max(1, min(steps, 2)), 2, lr=cfg.lr, betas=cfg.betas,
                                   wd=cfg.weight_decay, clip=cfg.grad_clip, barrier=barrier)
            bms = b["ms_per_step"]
            if world > 1:
                t = torch.tensor([bms], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                bms = float(t.item())
            base = {"tok_s": round(cfg.global_batch * cfg.seq_len / (bms * 1e-3), 1), "ms_per_step": round(bms, 2),
                    "last_loss": round(b["losses"][-1], 4),
                    "stack": "torch.nn + bf16 autocast + SDPA + fused AdamW" + (" + DDP (NCCL)" if world > 1 else "")}
        except Exception as e:      # noqa: BLE001 - the product number stands even if the comparison arm fails
            base = {"error": f"{type(e).__name__}: {e}"[:200]}
    if rank != 0:
        return None
    toks = cfg.global_batch * cfg.seq_len
    # 6 * params * tokens (matmul FLOPs incl. the tied LM head) + attention 12 * L * T * d per token
    m = cfg.model
    flops = 6.0 * (12 * m.n_layers * m.d_model ** 2 + m.vocab * m.d_model) * toks + 12.0 * m.n_layers * cfg.seq_len * m.d_model * toks
    return {
        "metric": "gpt2_small_train_tok_s", "value": round(toks / (ms * 1e-3), 1), "unit": "tokens/s", "n_gpus": world,
        "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 2), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": (round(toks / (ms * 1e-3) / base["tok_s"], 4) if base and "tok_s" in base else None),
        "dtype": "bf16", "data": "synthetic",
        "config": {"model": m.name, "global_batch": cfg.global_batch, "seq_len": cfg.seq_len, "micro_batch": cfg.micro_batch,
                   "parallelism": f"dp{world}+zero{cfg.zero_stage}", "optimizer": "AdamW lr 6e-4 betas (0.9,0.95) wd 0.1 clip 1.0",
                   "timed_region": "includes per-step H2D of token ids from pinned memory and D2H of the loss"},
        "clocks": clocks, "gpu_launches": launches,
        "extra": {"model_tflops_per_gpu": round(flops / (ms * 1e-3) / 1e12 / world, 1), "first_loss": round(losses[0], 4),
                  "last_loss": round(losses[-1], 4),
                  "h2d_bytes_per_step": 2 * 8 * accum * cfg.micro_batch * cfg.seq_len, "d2h_bytes_per_step": 4 * accum,
                  "baseline": base}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--global-batch", type=int, default=512)
    ap.add_argument("--micro-batch", type=int, default=16)
    ap.add_argument("--seq-len", type=int, default=1024)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--no-baseline", action="store_true", help="skip the plain-PyTorch comparison arm that runs after the timed steps")
    args = ap.parse_args()
    import torch
    import torch.distributed as dist
    world, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    out = run(args.steps, max(args.warmup, 3), args.global_batch, args.micro_batch, args.seq_len, baseline=not args.no_baseline)
    if out is not None:
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
