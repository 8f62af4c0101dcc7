"""Baseline arm of the decode benchmark: a Llama-shaped decoder in plain PyTorch.

Same configuration, same seeded Q4_K / Q6_K weights as the product run, but served the stock way: every weight is
dequantized once to bf16, projections are ``torch.matmul`` (cuBLAS), attention is
``torch.nn.functional.scaled_dot_product_attention`` over a contiguous bf16 KV cache, tensor parallelism is the
Megatron split with ``torch.distributed.all_reduce`` (NCCL) after the two row-parallel projections, and the decode
step is replayed from a CUDA graph (as a production PyTorch server would).  Nothing from ``openagents_b200``'s engine,
kernels or communicator runs here; only its weight generator and block codecs are used, so both arms see the same
numbers in the weights.
"""
from __future__ import annotations


import torch
import torch.distributed as dist
import torch.nn.functional as F


class TorchLlama:
    def __init__(self, cfg, src, device, rank: int = 0, world: int = 1, max_batch: int = 64, max_ctx: int = 4096, group=None):
        self.cfg, self.dev, self.rank, self.world, self.group = cfg, device, rank, world, group
        self.Hq, self.Hkv, self.hd = cfg.n_heads // world, cfg.n_kv_heads // world, cfg.head_dim
        self.F = cfg.ffn // world
        bf = torch.bfloat16

        def w(name):
            return src.get(name).to_float().to(device)

        def rows(x, n):      # column-parallel: split the output rows
            return x[rank * n:(rank + 1) * n]

        def cols(x, n):      # row-parallel: split the input columns
            return x[:, rank * n:(rank + 1) * n]

        self.emb = w("token_embd.weight").to(bf)
        self.layers = []
        for i in range(cfg.n_layers):
            p = f"blk.{i}."
            q, k, v = w(p + "attn_q.weight"), w(p + "attn_k.weight"), w(p + "attn_v.weight")
            wqkv = torch.cat([rows(q, self.Hq * self.hd), rows(k, self.Hkv * self.hd), rows(v, self.Hkv * self.hd)]).to(bf).contiguous()
            wo = cols(w(p + "attn_output.weight"), self.Hq * self.hd).to(bf).contiguous()
            wgu = torch.cat([rows(w(p + "ffn_gate.weight"), self.F), rows(w(p + "ffn_up.weight"), self.F)]).to(bf).contiguous()
            wd = cols(w(p + "ffn_down.weight"), self.F).to(bf).contiguous()
            self.layers.append((w(p + "attn_norm.weight").to(bf), wqkv, wo, w(p + "ffn_norm.weight").to(bf), wgu, wd))
        self.out_norm = w("output_norm.weight").to(bf)
        out = w("token_embd.weight" if cfg.tied_embeddings else "output.weight")
        self.V_local = out.shape[0] // world
        self.wout = rows(out, self.V_local).to(bf).contiguous()
        self.kc = [torch.zeros((max_batch, self.Hkv, max_ctx, self.hd), dtype=bf, device=device) for _ in range(cfg.n_layers)]
        self.vc = [torch.zeros_like(k) for k in self.kc]
        self.max_ctx = max_ctx
        half = self.hd // 2
        inv = cfg.rope_theta ** (-torch.arange(half, device=device, dtype=torch.float64) * 2.0 / self.hd)
        ang = torch.arange(max_ctx, device=device, dtype=torch.float64)[:, None] * inv[None]
        self.cos, self.sin = ang.cos().float(), ang.sin().float()
        self.pairs = cfg.rope_style == "pairs"

    def weight_bytes(self) -> int:
        n = self.emb.numel() + self.wout.numel()
        for l in self.layers:
            n += sum(t.numel() for t in l)
        return 2 * n

    def _norm(self, x, g):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.cfg.norm_eps)).to(x.dtype) * g

    def _rope(self, x, pos):           # x [B, T, H, hd], pos [B, T]
        c, s = self.cos[pos][:, :, None], self.sin[pos][:, :, None]
        xf = x.float()
        if self.pairs:
            a, b = xf[..., 0::2], xf[..., 1::2]
            return torch.stack((a * c - b * s, a * s + b * c), dim=-1).flatten(-2).to(x.dtype)
        a, b = xf[..., : self.hd // 2], xf[..., self.hd // 2:]
        return torch.cat((a * c - b * s, a * s + b * c), dim=-1).to(x.dtype)

    @torch.no_grad()
    def forward(self, ids, pos, row0, mask):
        """ids, pos [B, T]; the batch uses cache rows [row0, row0 + B); mask [B, 1, T, ctx] (True = attend)."""
        B, T = ids.shape
        x = self.emb[ids]
        for li, (g1, wqkv, wo, g2, wgu, wd) in enumerate(self.layers):
            h = self._norm(x, g1)
            qkv = h @ wqkv.t()
            q, k, v = qkv.split([self.Hq * self.hd, self.Hkv * self.hd, self.Hkv * self.hd], dim=-1)
            q = self._rope(q.view(B, T, self.Hq, self.hd), pos).transpose(1, 2)
            k = self._rope(k.view(B, T, self.Hkv, self.hd), pos).transpose(1, 2)
            v = v.view(B, T, self.Hkv, self.hd).transpose(1, 2)
            idx = pos[:, None, :, None].expand(B, self.Hkv, T, self.hd)
            kc, vc = self.kc[li][row0:row0 + B], self.vc[li][row0:row0 + B]       # views: the cache is updated in place
            kc.scatter_(2, idx, k)
            vc.scatter_(2, idx, v)
            o = F.scaled_dot_product_attention(q, kc, vc, attn_mask=mask, enable_gqa=True)
            a = o.transpose(1, 2).reshape(B, T, self.Hq * self.hd) @ wo.t()
            if self.world > 1:
                dist.all_reduce(a, group=self.group)
            x = x + a
            h = self._norm(x, g2)
            gu = h @ wgu.t()
            m = (F.silu(gu[..., : self.F]) * gu[..., self.F:]) @ wd.t()
            if self.world > 1:
                dist.all_reduce(m, group=self.group)
            x = x + m
        logits = self._norm(x[:, -1], self.out_norm) @ self.wout.t()
        val, idx = logits.float().max(-1)
        if self.world > 1:          # vocabulary is sharded: merge the per-shard winners
            vals = [torch.empty_like(val) for _ in range(self.world)]
            ids_ = [torch.empty_like(idx) for _ in range(self.world)]
            dist.all_gather(vals, val, group=self.group)
            dist.all_gather(ids_, idx + self.rank * self.V_local, group=self.group)
            vals, ids_ = torch.stack(vals), torch.stack(ids_)
            idx = ids_.gather(0, vals.argmax(0, keepdim=True))[0]
        return idx


class DecodeGraph:
    """One decode step of a fixed batch, replayed from a CUDA graph: inputs are the previous step's tokens (on the
    device) and positions; the cache is written in place; every cache row up to ``ctx`` positions is attended through a
    mask, so the graph does not depend on the step number."""

    def __init__(self, model: TorchLlama, B: int):
        self.m, self.B = model, B
        dev = model.dev
        self.ids = torch.zeros((B, 1), dtype=torch.long, device=dev)
        self.pos = torch.zeros((B, 1), dtype=torch.long, device=dev)
        self.mask = torch.zeros((B, 1, 1, model.max_ctx), dtype=torch.bool, device=dev)
        self.out = torch.zeros(B, dtype=torch.long, device=dev)
        self.graph = None

    def _body(self):
        ar = torch.arange(self.m.max_ctx, device=self.m.dev)
        self.mask.copy_(ar[None, None, None, :] <= self.pos[:, None, :, None])
        self.out.copy_(self.m.forward(self.ids, self.pos, 0, self.mask))
        self.ids.copy_(self.out[:, None])
        self.pos.add_(1)

    def capture(self):
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        saved = (self.ids.clone(), self.pos.clone())
        with torch.cuda.stream(s):
            self._body()                     # warm-up (allocations, cuBLAS handles, NCCL)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        self.ids.copy_(saved[0])
        self.pos.copy_(saved[1])
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=s):
            self._body()
        self.ids.copy_(saved[0])
        self.pos.copy_(saved[1])

    def step(self):
        self.graph.replay()


def run_decode_baseline(cfg, src, dev, rank, world, B, P, K, W, prompts, barrier, max_over_ranks, sampler=None, group=None, total_batch=None):
    """Prefill ``B`` prompts of ``P`` tokens (untimed), then time ``K`` greedy decode steps of the whole batch after ``W``
    warm-up steps.  Returns (tokens/s, ms per step, end-to-end tokens/s with per-step host copies, clocks).  ``rank`` /
    ``world`` / ``group`` describe ONE tensor-parallel replica; with several replicas side by side ``B`` is this replica's
    share and ``total_batch`` the number of sequences all replicas advance per step."""
    total_batch = total_batch or B
    model = TorchLlama(cfg, src, dev, rank, world, max_batch=B, max_ctx=P + 2 * (K + W) + 16, group=group)
    first = torch.zeros(B, dtype=torch.long, device=dev)
    ar = torch.arange(model.max_ctx, device=dev)
    for b0 in range(0, B, 4):
        ids = prompts[b0:b0 + 4].to(dev)
        n = ids.shape[0]
        pos = torch.arange(P, device=dev)[None].expand(n, P)
        mask = (ar[None, None, None, :] <= pos[:, None, :, None])
        first[b0:b0 + n] = model.forward(ids, pos, b0, mask)
    g = DecodeGraph(model, B)
    g.ids.copy_(first[:, None])
    g.pos.fill_(P)
    g.capture()
    for _ in range(W):
        g.step()
    barrier()
    if sampler is not None:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        g.step()
    e1.record()
    barrier()
    clocks = sampler.stop() if sampler is not None else None
    ms = max_over_ranks(e0.elapsed_time(e1)) / K
    # end to end: the step's input ids come from pinned host memory and the sampled ids go back to the host every step
    import time
    host_ids = torch.zeros((B, 1), dtype=torch.long).pin_memory()
    host_ids.copy_(g.ids.cpu())
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        g.ids.copy_(host_ids, non_blocking=True)
        g.step()
        host_ids.copy_(g.out[:, None].cpu())
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3) / K
    res = {"value": total_batch / (ms * 1e-3), "ms_per_step": ms, "e2e_value": total_batch / (e2e_ms * 1e-3), "e2e_ms_per_step": e2e_ms, "clocks": clocks,
           "weight_bytes_per_gpu": model.weight_bytes()}
    del g, model
    torch.cuda.empty_cache()
    return res
