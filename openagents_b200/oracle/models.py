"""Whole-model CPU reference forwards over a dict of fp32 tensors (GGUF tensor names)."""
from __future__ import annotations

import torch

from ..models.config import ModelConfig
from . import nn


class KVCacheRef:
    """Contiguous per-layer K/V lists; the simplest cache with the same semantics as the paged one."""

    def __init__(self, n_layers: int):
        self.k = [None] * n_layers
        self.v = [None] * n_layers

    def append(self, layer: int, k, v):
        self.k[layer] = k if self.k[layer] is None else torch.cat((self.k[layer], k), 0)
        self.v[layer] = v if self.v[layer] is None else torch.cat((self.v[layer], v), 0)
        return self.k[layer], self.v[layer]

    @property
    def length(self) -> int:
        return 0 if self.k[0] is None else self.k[0].shape[0]

    def truncate(self, n: int):
        """Keep the first ``n`` positions (a rejected speculative tail is dropped)."""
        for i in range(len(self.k)):
            if self.k[i] is not None:
                self.k[i], self.v[i] = self.k[i][:n], self.v[i][:n]


def _lin(x, w, b=None):
    y = x @ w.t()
    return y if b is None else y + b


def llama_forward(cfg: ModelConfig, W: dict, tokens: torch.Tensor, cache: KVCacheRef | None = None):
    """tokens: [T] ids appended after whatever the cache holds.  Returns logits [T, V]."""
    cache = cache if cache is not None else KVCacheRef(cfg.n_layers)
    p0 = cache.length
    T = tokens.shape[0]
    pos = torch.arange(p0, p0 + T, device=tokens.device)
    x = W["token_embd.weight"][tokens]
    for i in range(cfg.n_layers):
        pre = f"blk.{i}."
        h = nn.rmsnorm(x, W[pre + "attn_norm.weight"], cfg.norm_eps)
        q = _lin(h, W[pre + "attn_q.weight"], W.get(pre + "attn_q.bias")).view(T, cfg.n_heads, cfg.head_dim)
        k = _lin(h, W[pre + "attn_k.weight"], W.get(pre + "attn_k.bias")).view(T, cfg.n_kv_heads, cfg.head_dim)
        v = _lin(h, W[pre + "attn_v.weight"], W.get(pre + "attn_v.bias")).view(T, cfg.n_kv_heads, cfg.head_dim)
        q = nn.rope(q, pos, cfg.rope_theta, cfg.rope_style)
        k = nn.rope(k, pos, cfg.rope_theta, cfg.rope_style)
        K, V = cache.append(i, k, v)
        kpos = torch.arange(K.shape[0], device=tokens.device)
        window = cfg.sliding_window if cfg.layer_uses_window(i) else 0
        sinks = W.get(pre + "attn_sinks.weight") if cfg.attn_sinks else None
        a = nn.attention(q, K, V, pos, kpos, window=window, sinks=sinks).reshape(T, cfg.q_dim)
        x = x + _lin(a, W[pre + "attn_output.weight"], W.get(pre + "attn_output.bias"))
        h = nn.rmsnorm(x, W[pre + "ffn_norm.weight"], cfg.norm_eps)
        if cfg.n_experts:
            x = x + moe_ffn(cfg, W, pre, h)
        else:
            g = _lin(h, W[pre + "ffn_gate.weight"])
            u = _lin(h, W[pre + "ffn_up.weight"])
            x = x + _lin(nn.swiglu(g, u), W[pre + "ffn_down.weight"])
    x = nn.rmsnorm(x, W["output_norm.weight"], cfg.norm_eps)
    out_w = W["token_embd.weight"] if cfg.tied_embeddings else W["output.weight"]
    return x @ out_w.t()


def moe_ffn(cfg: ModelConfig, W: dict, pre: str, h: torch.Tensor) -> torch.Tensor:
    """Top-k routed SwiGLU experts; weights stacked as [E, out, in]."""
    logits = _lin(h, W[pre + "ffn_gate_inp.weight"], W.get(pre + "ffn_gate_inp.bias"))
    p, idx = nn.topk_router(logits, cfg.top_k)
    out = torch.zeros_like(h)
    Wg, Wu, Wd = W[pre + "ffn_gate_exps.weight"], W[pre + "ffn_up_exps.weight"], W[pre + "ffn_down_exps.weight"]
    for e in range(cfg.n_experts):
        sel = (idx == e)
        rows = sel.any(-1).nonzero().flatten()
        if rows.numel() == 0:
            continue
        wt = (p * sel)[rows].sum(-1, keepdim=True)
        he = h[rows]
        y = nn.swiglu(he @ Wg[e].t(), he @ Wu[e].t()) @ Wd[e].t()
        out.index_add_(0, rows, wt * y)
    return out


def gpt2_forward(cfg: ModelConfig, W: dict, tokens: torch.Tensor) -> torch.Tensor:
    """tokens: [B, T].  Pre-LN GPT-2 with tied embeddings.  Returns logits [B, T, V]."""
    B, T = tokens.shape
    x = W["token_embd.weight"][tokens] + W["position_embd.weight"][:T]
    pos = torch.arange(T, device=tokens.device)
    for i in range(cfg.n_layers):
        pre = f"blk.{i}."
        h = nn.layernorm(x, W[pre + "attn_norm.weight"], W[pre + "attn_norm.bias"], cfg.norm_eps)
        qkv = _lin(h, W[pre + "attn_qkv.weight"], W[pre + "attn_qkv.bias"])
        q, k, v = qkv.split(cfg.d_model, dim=-1)
        outs = []
        for b in range(B):
            o = nn.attention(q[b].view(T, cfg.n_heads, cfg.head_dim), k[b].view(T, cfg.n_heads, cfg.head_dim),
                             v[b].view(T, cfg.n_heads, cfg.head_dim), pos, pos)
            outs.append(o.reshape(T, cfg.d_model))
        a = torch.stack(outs)
        x = x + _lin(a, W[pre + "attn_output.weight"], W[pre + "attn_output.bias"])
        h = nn.layernorm(x, W[pre + "ffn_norm.weight"], W[pre + "ffn_norm.bias"], cfg.norm_eps)
        x = x + _lin(nn.gelu_tanh(_lin(h, W[pre + "ffn_up.weight"], W[pre + "ffn_up.bias"])),
                     W[pre + "ffn_down.weight"], W[pre + "ffn_down.bias"])
    x = nn.layernorm(x, W["output_norm.weight"], W["output_norm.bias"], cfg.norm_eps)
    return x @ W["token_embd.weight"].t()


def greedy_generate(cfg: ModelConfig, W: dict, prompt: torch.Tensor, n_new: int):
    """Greedy decode with a contiguous cache.  Returns (token ids [n_new], logits [n_new, V])."""
    cache = KVCacheRef(cfg.n_layers)
    logits = llama_forward(cfg, W, prompt, cache)[-1]
    ids, all_logits = [], []
    for _ in range(n_new):
        all_logits.append(logits)
        nxt = int(torch.argmax(logits))
        ids.append(nxt)
        logits = llama_forward(cfg, W, torch.tensor([nxt]), cache)[-1]
    return torch.tensor(ids), torch.stack(all_logits)
