"""The training comparison arm: the same GPT-2-shape model, batch and optimizer on plain PyTorch.

``torch.nn`` modules with fp32 parameters under bf16 autocast, ``F.scaled_dot_product_attention`` (causal),
``torch.optim.AdamW(fused=True)``, gradient clipping by global norm, gradient accumulation over the micro-batches of a
step and ``DistributedDataParallel`` (NCCL all-reduce) over the ranks.  None of this package's kernels are on this path.
It exists so that the trainer's tokens/s has a labelled baseline measured on the same GPUs in the same process.
"""
from __future__ import annotations

import contextlib
import math
import time

import torch
import torch.nn as nn
import torch.nn.functional as F


class Block(nn.Module):
    def __init__(self, d: int, n_heads: int, ffn: int, eps: float):
        super().__init__()
        self.h = n_heads
        self.ln1, self.ln2 = nn.LayerNorm(d, eps=eps), nn.LayerNorm(d, eps=eps)
        self.qkv, self.proj = nn.Linear(d, 3 * d), nn.Linear(d, d)
        self.up, self.down = nn.Linear(d, ffn), nn.Linear(ffn, d)

    def forward(self, x):
        B, T, d = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(B, T, 3, self.h, d // self.h).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, T, d)
        x = x + self.proj(a)
        return x + self.down(F.gelu(self.up(self.ln2(x)), approximate="tanh"))


class TorchGPT2(nn.Module):
    def __init__(self, cfg):
        super().__init__()
        d = cfg.d_model
        self.vocab = cfg.vocab
        vp = (cfg.vocab + 63) // 64 * 64               # same padded vocabulary as the product trainer
        self.wte, self.wpe = nn.Embedding(vp, d), nn.Embedding(cfg.context, d)
        self.blocks = nn.ModuleList(Block(d, cfg.n_heads, cfg.ffn, cfg.norm_eps) for _ in range(cfg.n_layers))
        self.lnf = nn.LayerNorm(d, eps=cfg.norm_eps)
        for p in self.parameters():
            if p.dim() > 1:
                nn.init.normal_(p, 0.0, 0.02)

    def forward(self, tokens, targets):
        T = tokens.shape[1]
        x = self.wte(tokens) + self.wpe(torch.arange(T, device=tokens.device))
        for b in self.blocks:
            x = b(x)
        logits = F.linear(self.lnf(x), self.wte.weight)[..., : self.vocab]          # tied LM head
        return F.cross_entropy(logits.float().view(-1, self.vocab), targets.reshape(-1))


def run_train_baseline(model_cfg, device, rank: int, world: int, batches, accum: int, steps: int, warmup: int, lr=6e-4, betas=(0.9, 0.95),
                       wd=0.1, clip=1.0, barrier=None) -> dict:
    """``batches``: list of pinned ``(tokens, targets)`` of shape [accum, micro_batch, seq_len] (int64), cycled.  Returns
    ms per optimizer step (device time, this rank) and the losses."""
    torch.manual_seed(0)
    model = TorchGPT2(model_cfg).to(device)
    ddp = model
    if world > 1:
        from torch.nn.parallel import DistributedDataParallel as DDP
        ddp = DDP(model, device_ids=[device.index] if device.type == "cuda" else None, gradient_as_bucket_view=True)
    decay = [p for n, p in model.named_parameters() if p.dim() > 1]
    plain = [p for n, p in model.named_parameters() if p.dim() <= 1]
    opt = torch.optim.AdamW([{"params": decay, "weight_decay": wd}, {"params": plain, "weight_decay": 0.0}], lr=lr, betas=betas,
                            eps=1e-8, fused=True)
    on_gpu = device.type == "cuda"

    def step(i):
        tok, tgt = batches[i % len(batches)]
        tok, tgt = tok.to(device, non_blocking=True), tgt.to(device, non_blocking=True)
        total = 0.0
        for a in range(accum):
            sync = contextlib.nullcontext() if (world == 1 or a == accum - 1) else ddp.no_sync()
            with sync:
                with torch.autocast(device.type, dtype=torch.bfloat16):
                    loss = ddp(tok[a], tgt[a]) / accum
                loss.backward()
            total = total + loss.detach()
        torch.nn.utils.clip_grad_norm_(model.parameters(), clip)
        opt.step()
        opt.zero_grad(set_to_none=True)
        return float(total.item())

    losses = [step(i) for i in range(warmup)]
    if barrier:
        barrier()
    if on_gpu:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    t0 = time.perf_counter()
    for i in range(steps):
        losses.append(step(warmup + i))
    if on_gpu:
        e1.record()
    if barrier:
        barrier()
    elif on_gpu:
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps if on_gpu else (time.perf_counter() - t0) * 1e3 / steps
    del opt, ddp, model
    if on_gpu:
        torch.cuda.empty_cache()
    return {"ms_per_step": ms, "losses": losses, "first_loss_expected": math.log(model_cfg.vocab)}
