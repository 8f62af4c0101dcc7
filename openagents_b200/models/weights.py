"""Tensor inventories, seeded random initialisation and GGUF save/load of whole models.

Weights are N(0, 0.02) from a seeded generator (one stream per tensor, so the values do not depend
on creation order); norm gains are ones and stay F32 in the file.
"""
from __future__ import annotations

import zlib
from dataclasses import dataclass

import torch

from ..gguf import GGUFFile, GGUFWriter, GgmlType, type_block
from .config import ModelConfig


@dataclass
class TensorSpec:
    name: str
    shape: tuple[int, ...]
    kind: str   # "matrix" | "embed" | "output" | "norm" | "bias" | "expert" | "router" | "sink" | "pos"


def tensor_specs(cfg: ModelConfig) -> list[TensorSpec]:
    d, f, V = cfg.d_model, cfg.ffn, cfg.vocab
    s: list[TensorSpec] = [TensorSpec("token_embd.weight", (V, d), "embed")]
    if cfg.arch == "gpt2":
        s.append(TensorSpec("position_embd.weight", (cfg.context, d), "pos"))
    for i in range(cfg.n_layers):
        p = f"blk.{i}."
        if cfg.arch == "gpt2":
            s += [TensorSpec(p + "attn_norm.weight", (d,), "norm"), TensorSpec(p + "attn_norm.bias", (d,), "bias"),
                  TensorSpec(p + "attn_qkv.weight", (3 * d, d), "matrix"), TensorSpec(p + "attn_qkv.bias", (3 * d,), "bias"),
                  TensorSpec(p + "attn_output.weight", (d, d), "matrix"), TensorSpec(p + "attn_output.bias", (d,), "bias"),
                  TensorSpec(p + "ffn_norm.weight", (d,), "norm"), TensorSpec(p + "ffn_norm.bias", (d,), "bias"),
                  TensorSpec(p + "ffn_up.weight", (f, d), "matrix"), TensorSpec(p + "ffn_up.bias", (f,), "bias"),
                  TensorSpec(p + "ffn_down.weight", (d, f), "matrix"), TensorSpec(p + "ffn_down.bias", (d,), "bias")]
            continue
        s += [TensorSpec(p + "attn_norm.weight", (d,), "norm"),
              TensorSpec(p + "attn_q.weight", (cfg.q_dim, d), "matrix"),
              TensorSpec(p + "attn_k.weight", (cfg.kv_dim, d), "matrix"),
              TensorSpec(p + "attn_v.weight", (cfg.kv_dim, d), "matrix"),
              TensorSpec(p + "attn_output.weight", (d, cfg.q_dim), "matrix")]
        if cfg.qkv_bias:
            s += [TensorSpec(p + "attn_q.bias", (cfg.q_dim,), "bias"), TensorSpec(p + "attn_k.bias", (cfg.kv_dim,), "bias"),
                  TensorSpec(p + "attn_v.bias", (cfg.kv_dim,), "bias"), TensorSpec(p + "attn_output.bias", (d,), "bias")]
        if cfg.attn_sinks:
            s.append(TensorSpec(p + "attn_sinks.weight", (cfg.n_heads,), "sink"))
        s.append(TensorSpec(p + "ffn_norm.weight", (d,), "norm"))
        if cfg.n_experts:
            E = cfg.n_experts
            s += [TensorSpec(p + "ffn_gate_inp.weight", (E, d), "router"),
                  TensorSpec(p + "ffn_gate_exps.weight", (E, f, d), "expert"),
                  TensorSpec(p + "ffn_up_exps.weight", (E, f, d), "expert"),
                  TensorSpec(p + "ffn_down_exps.weight", (E, d, f), "expert")]
        else:
            s += [TensorSpec(p + "ffn_gate.weight", (f, d), "matrix"),
                  TensorSpec(p + "ffn_up.weight", (f, d), "matrix"),
                  TensorSpec(p + "ffn_down.weight", (d, f), "matrix")]
    s.append(TensorSpec("output_norm.weight", (d,), "norm"))
    if cfg.arch == "gpt2":
        s.append(TensorSpec("output_norm.bias", (d,), "bias"))
    if not cfg.tied_embeddings:
        s.append(TensorSpec("output.weight", (V, d), "output"))
    return s


@dataclass(frozen=True)
class QuantPlan:
    """Which block format each tensor kind is stored in."""
    matrix: GgmlType = GgmlType.Q8_0
    embed: GgmlType = GgmlType.Q8_0
    output: GgmlType = GgmlType.Q8_0
    expert: GgmlType = GgmlType.MXFP4
    router: GgmlType = GgmlType.F32

    def type_for(self, spec: TensorSpec) -> GgmlType:
        if spec.kind in ("norm", "bias", "sink", "pos"):
            return GgmlType.F32
        t = {"matrix": self.matrix, "embed": self.embed, "output": self.output,
             "expert": self.expert, "router": self.router}[spec.kind]
        be, _ = type_block(t)
        # A row that does not divide into blocks falls back to F16, as GGUF converters do.
        return t if spec.shape[-1] % be == 0 else GgmlType.F16


PLAN_Q8_0 = QuantPlan()
PLAN_Q4_K = QuantPlan(matrix=GgmlType.Q4_K, embed=GgmlType.Q6_K, output=GgmlType.Q6_K)
PLAN_BF16 = QuantPlan(matrix=GgmlType.BF16, embed=GgmlType.BF16, output=GgmlType.BF16, expert=GgmlType.BF16)
PLAN_F32 = QuantPlan(matrix=GgmlType.F32, embed=GgmlType.F32, output=GgmlType.F32, expert=GgmlType.F32)
PLAN_MOE = QuantPlan(matrix=GgmlType.BF16, embed=GgmlType.BF16, output=GgmlType.BF16, expert=GgmlType.MXFP4)


def init_tensor(spec: TensorSpec, seed: int, device="cpu", std: float = 0.02) -> torch.Tensor:
    if spec.kind == "norm":
        return torch.ones(spec.shape, dtype=torch.float32, device=device)
    if spec.kind == "bias":
        return torch.zeros(spec.shape, dtype=torch.float32, device=device)
    g = torch.Generator(device=device)
    g.manual_seed((seed * 1000003 + zlib.crc32(spec.name.encode())) & 0x7FFFFFFF)
    return torch.randn(spec.shape, generator=g, dtype=torch.float32, device=device) * std


def random_weights(cfg: ModelConfig, seed: int = 0) -> dict[str, torch.Tensor]:
    return {s.name: init_tensor(s, seed) for s in tensor_specs(cfg)}


def save_gguf(path: str, cfg: ModelConfig, weights: dict[str, torch.Tensor], plan: QuantPlan = PLAN_Q8_0,
              extra_meta: dict | None = None):
    w = GGUFWriter(path)
    for k, v in cfg.to_gguf_metadata().items():
        w.add_meta(k, v)
    w.add_meta("general.file_type", int(plan.matrix))
    for k, v in (extra_meta or {}).items():
        w.add_meta(k, v)
    for spec in tensor_specs(cfg):
        x = weights[spec.name].detach().to(torch.float32).cpu().numpy()
        w.add_tensor(spec.name, x, plan.type_for(spec))
    w.write()


def load_gguf_float(path: str) -> tuple[ModelConfig, dict[str, torch.Tensor]]:
    """Load and dequantize every tensor to fp32 (CPU backend and oracle)."""
    with GGUFFile(path) as f:
        cfg = ModelConfig.from_gguf_metadata(f.metadata)
        W = {n: torch.from_numpy(t.to_float().copy()) for n, t in f.tensors.items()}
    return cfg, W
