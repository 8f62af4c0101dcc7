"""Plain PyTorch fp32/fp64 restatement of the transformer math, used as the test oracle.

The normalisation, attention, SwiGLU and cross-entropy formulas are the ones of the reference's
CPU workload (apps/openagents.com/workers/api/src/cs336-a1-real-gradient-workload.ts:351-375
RMSNorm, :478-518 causal softmax attention, :532-549 SwiGLU, :580-595 cross-entropy), widened with
RoPE, grouped-query heads, sliding windows with sink logits, LayerNorm + GELU and a top-k router.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rmsnorm(x: torch.Tensor, g: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * g


def layernorm(x, g, b, eps: float = 1e-5):
    mu = x.mean(-1, keepdim=True)
    var = (x - mu).pow(2).mean(-1, keepdim=True)
    return (x - mu) * torch.rsqrt(var + eps) * g + b


def gelu_tanh(x):
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x.pow(3))))


def swiglu(gate, up):
    return F.silu(gate) * up


def rope(x: torch.Tensor, pos: torch.Tensor, theta: float, style: str = "pairs") -> torch.Tensor:
    """x: [..., T, H, D]; pos: [T] (or broadcastable to x[..., :, 0, 0])."""
    D = x.shape[-1]
    inv = theta ** (-torch.arange(0, D, 2, dtype=torch.float64, device=x.device) / D)
    ang = pos.to(torch.float64)[..., None] * inv          # [T, D/2]
    cos, sin = ang.cos().to(x.dtype)[..., None, :], ang.sin().to(x.dtype)[..., None, :]
    if style == "pairs":
        x1, x2 = x[..., 0::2], x[..., 1::2]
        out = torch.stack((x1 * cos - x2 * sin, x1 * sin + x2 * cos), dim=-1)
        return out.flatten(-2)
    x1, x2 = x[..., : D // 2], x[..., D // 2:]
    return torch.cat((x1 * cos - x2 * sin, x1 * sin + x2 * cos), dim=-1)


def attention(q, k, v, q_pos, k_pos, window: int = 0, sinks: torch.Tensor | None = None,
              causal: bool = True, scale: float | None = None):
    """q: [Tq, H, D]; k, v: [Tk, Hkv, D]; positions are absolute token indices.

    ``window`` > 0 keeps keys with q_pos - k_pos < window.  ``sinks`` ([H]) adds one learned logit
    per head to the softmax denominator only.
    """
    Tq, H, D = q.shape
    Hkv = k.shape[1]
    rep = H // Hkv
    k = k.repeat_interleave(rep, dim=1)
    v = v.repeat_interleave(rep, dim=1)
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    s = torch.einsum("qhd,khd->hqk", q, k) * scale
    dist = q_pos[:, None] - k_pos[None, :]
    mask = torch.zeros_like(dist, dtype=torch.bool)
    if causal:
        mask |= dist < 0
    if window > 0:
        mask |= dist >= window
    s = s.masked_fill(mask[None], float("-inf"))
    if sinks is not None:
        s = torch.cat((s, sinks.to(s.dtype)[:, None, None].expand(H, Tq, 1)), dim=-1)
        p = torch.softmax(s, dim=-1)[..., :-1]
    else:
        p = torch.softmax(s, dim=-1)
    return torch.einsum("hqk,khd->qhd", p, v)


def cross_entropy(logits, targets):
    return F.cross_entropy(logits.float(), targets, reduction="mean")


def topk_router(logits: torch.Tensor, k: int):
    """Top-k over expert logits, then softmax over the selected k (gpt-oss convention)."""
    vals, idx = torch.topk(logits, k, dim=-1)
    return torch.softmax(vals, dim=-1), idx
