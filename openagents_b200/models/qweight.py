"""Device-resident weights in the layouts the kernels read, and where they come from.

A ``WeightSource`` hands out tensors in standard GGUF bytes (so sharding is plain byte slicing);
``QWeight.from_ggml`` repacks them once into the engine layout.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..gguf import GGUFFile, GgmlType, type_block
from ..gguf import torch_codecs as tc
from ..ops import cuda_ops as ops
from .config import ModelConfig
from .weights import QuantPlan, init_tensor, tensor_specs


@dataclass
class RawTensor:
    """A tensor in standard GGUF bytes: ``data`` is uint8, ``shape`` row-major."""
    type: GgmlType
    shape: tuple[int, ...]
    data: torch.Tensor

    def rows(self, lo: int, hi: int) -> "RawTensor":
        """Slice of the slowest axis (exact for every block format)."""
        per = self.data.numel() // self.shape[0]
        return RawTensor(self.type, (hi - lo,) + tuple(self.shape[1:]), self.data[lo * per: hi * per])

    def cols(self, lo: int, hi: int) -> "RawTensor":
        """Slice of the last axis of a 2-D tensor; ``lo``/``hi`` must fall on block boundaries."""
        be, bb = type_block(self.type)
        N, K = self.shape
        if lo % be or hi % be:
            raise ValueError(f"column slice [{lo},{hi}) is not aligned to the {self.type.name} block of {be}")
        d = self.data.reshape(N, K // be, bb)[:, lo // be: hi // be].contiguous()
        return RawTensor(self.type, (N, hi - lo), d.reshape(-1))

    def to_float(self) -> torch.Tensor:
        return tc.dequantize(self.data, self.type, self.shape)

    @staticmethod
    def interleave_rows(a: "RawTensor", b: "RawTensor") -> "RawTensor":
        """Rows a_0, b_0, a_1, b_1, ... of two equally shaped matrices (exact for every block format: a row is a
        whole number of blocks)."""
        if a.type != b.type or a.shape != b.shape:
            raise ValueError("row interleaving needs equal types and shapes")
        n = a.shape[0]
        d = torch.stack((a.data.reshape(n, -1), b.data.reshape(n, -1)), dim=1).reshape(-1)
        return RawTensor(a.type, (2 * n,) + tuple(a.shape[1:]), d)

    @staticmethod
    def cat_rows(parts: list["RawTensor"]) -> "RawTensor":
        t = parts[0].type
        if any(p.type != t or p.shape[1:] != parts[0].shape[1:] for p in parts):
            raise ValueError("row concatenation needs equal types and row lengths")
        return RawTensor(t, (sum(p.shape[0] for p in parts),) + tuple(parts[0].shape[1:]),
                         torch.cat([p.data for p in parts]))


class WeightSource:
    def get(self, name: str) -> RawTensor:
        raise NotImplementedError

    def has(self, name: str) -> bool:
        raise NotImplementedError


class GGUFSource(WeightSource):
    """Tensors of an open GGUF file, copied to ``device`` on demand."""

    def __init__(self, path: str, device):
        self.file = GGUFFile(path)
        self.device = device
        self.cfg = ModelConfig.from_gguf_metadata(self.file.metadata)

    def has(self, name):
        return name in self.file.tensors

    def get(self, name):
        t = self.file.tensors[name]
        return RawTensor(t.type, t.shape, torch.from_numpy(t.data.copy()).to(self.device))


class RandomSource(WeightSource):
    """Seeded N(0, 0.02) weights generated and quantized on ``device`` one tensor at a time."""

    def __init__(self, cfg: ModelConfig, plan: QuantPlan, seed: int, device):
        self.cfg, self.plan, self.seed, self.device = cfg, plan, seed, device
        self.specs = {s.name: s for s in tensor_specs(cfg)}

    def has(self, name):
        return name in self.specs

    def get(self, name):
        s = self.specs[name]
        t = self.plan.type_for(s)
        rows = s.shape[0]
        # Quantize in row chunks so a 128256 x 4096 table never needs several fp32 copies at once.
        if len(s.shape) >= 2 and s.kind not in ("norm", "bias", "sink"):
            x = init_tensor(s, self.seed, device=self.device)
            chunks = [tc.quantize(c, t) for c in x.split(max(1, (1 << 24) // max(1, x[0].numel())))]
            del x
            return RawTensor(t, s.shape, torch.cat(chunks))
        x = init_tensor(s, self.seed, device=self.device)
        return RawTensor(t, s.shape, tc.quantize(x, t))


class DictSource(WeightSource):
    """fp32 tensors from a dict, quantized per the plan (tests, trainer export)."""

    def __init__(self, cfg: ModelConfig, weights: dict, plan: QuantPlan, device):
        self.cfg, self.w, self.plan, self.device = cfg, weights, plan, device
        self.specs = {s.name: s for s in tensor_specs(cfg)}

    def has(self, name):
        return name in self.w

    def get(self, name):
        t = self.plan.type_for(self.specs[name])
        x = self.w[name].to(self.device, torch.float32)
        return RawTensor(t, tuple(x.shape), tc.quantize(x, t))


@dataclass
class QWeight:
    """A [N][K] matrix in an engine layout."""
    wt: int
    N: int
    K: int
    main: torch.Tensor
    plane2: torch.Tensor | None
    src_type: GgmlType

    @staticmethod
    def from_raw(r: RawTensor) -> "QWeight":
        N = r.shape[0]
        K = 1
        for s in r.shape[1:]:
            K *= s
        if r.type == GgmlType.Q4_K:
            return QWeight(ops.WT_Q4KR, N, K, tc.repack_q4_k(r.data), None, r.type)
        if r.type == GgmlType.Q6_K:
            main, d = tc.repack_q6_k(r.data)
            return QWeight(ops.WT_Q6KR, N, K, main, d, r.type)
        if r.type == GgmlType.Q8_0:
            q, d = tc.repack_q8_0(r.data)
            return QWeight(ops.WT_Q8R, N, K, q, d, r.type)
        if r.type == GgmlType.MXFP4:
            q, e = tc.repack_mxfp4(r.data)
            return QWeight(ops.WT_MXFP4R, N, K, q, e, r.type)
        x = tc.dequantize(r.data, r.type, (N, K)).to(torch.bfloat16).contiguous()
        return QWeight(ops.WT_BF16, N, K, x, None, r.type)

    @property
    def quantized(self) -> bool:
        return self.wt != ops.WT_BF16

    def to(self, device) -> "QWeight":
        """The same weight with its planes on ``device`` (a source on the host repacks there; the kernels need the GPU)."""
        if self.main.device == torch.device(device):
            return self
        return QWeight(self.wt, self.N, self.K, self.main.to(device), None if self.plane2 is None else self.plane2.to(device),
                       self.src_type)

    def nbytes(self) -> int:
        return self.main.numel() * self.main.element_size() + (0 if self.plane2 is None else self.plane2.numel() * self.plane2.element_size())

    def dequant_into(self, out: torch.Tensor) -> torch.Tensor:
        if self.wt == ops.WT_BF16:
            return self.main
        ops.dequant_bf16(self.wt, self.main, self.plane2, out, self.N, self.K)
        return out
