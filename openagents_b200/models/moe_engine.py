"""Expert-parallel serving engine for sparse mixture-of-experts decoders (gpt-oss shape).

Layout: attention is data-parallel (every rank holds the attention weights and serves its own
sequences with its own paged KV cache), the experts are sharded (``n_experts / world`` per rank).
A layer's feed-forward block is three kernels:

1. ``moe_route_dispatch`` - router, top-k, softmax and the dispatch in one kernel: each token's
   normalised hidden row is stored straight into the owning rank's receive buffer over NVLink peer
   memory (slot claimed by an atomic on the owner's counter); ends with the cross-rank barrier.
2. grouped tcgen05 GEMM, mode 1 - gate/up projection of every local expert over its received rows
   with SwiGLU in the epilogue.
3. grouped tcgen05 GEMM, mode 2 - down projection whose epilogue multiplies by the gate weight and
   adds the row into the residual stream of the rank the token came from (``red`` over peer memory);
   ends with the cross-rank barrier.  There is no separate combine or all-to-all launch.

Expert weights arrive as MXFP4 blocks (GGUF) and are expanded once, at load, to bf16 for the tensor
cores; the expansion is exact.

The reference names this topology without implementing it: ``sparse_expert`` placement with
"explicit expert ranges and a stable placement digest"
(docs/teardowns/2026-07-21-buzz-teardown.md:676-679).  ``placement_digest`` provides that digest.
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass

import torch

from ..ops import cuda_ops as ops
from ..parallel.tp import TPComm
from .config import ModelConfig
from .engine import LlamaEngine, _Layer
from .qweight import WeightSource
from ..utils.nvtx import nvtx_method


@dataclass
class _Experts:
    router_w: torch.Tensor            # fp32 [E][d]
    router_b: torch.Tensor | None     # fp32 [E]
    w13: torch.Tensor                 # bf16 [E_local * 2f][d], rows interleaved (gate_j, up_j)
    w2: torch.Tensor                  # bf16 [E_local * d][f]


class MoEEngine(LlamaEngine):
    ARCHS = ("gpt-oss", "llama")

    def __init__(self, cfg: ModelConfig, src: WeightSource, device="cuda", max_batch: int = 64, max_ctx: int = 4096,
                 n_pages: int | None = None, ep_rank: int = 0, ep_world: int = 1, max_tokens: int = 4096, comm: TPComm | None = None):
        if not cfg.n_experts:
            raise ValueError("MoEEngine needs a model with experts")
        if cfg.n_experts % ep_world:
            raise ValueError("the expert-parallel degree must divide the number of experts")
        self.ep_rank, self.ep_world = ep_rank, ep_world
        self.E, self.E_local, self.top_k = cfg.n_experts, cfg.n_experts // ep_world, cfg.top_k
        self.cap = (ep_world * max_tokens + 127) // 128 * 128      # rows an expert can receive in one forward
        need = (self.E_local * self.cap * (cfg.d_model * 2 + 8 + 4) + max_tokens * cfg.d_model * 4 + (1 << 20))
        self.ep = comm if comm is not None else TPComm(ep_rank, ep_world, device, heap_bytes=need)
        self.experts: list[_Experts] = []
        super().__init__(cfg, src, device=device, max_batch=max_batch, max_ctx=max_ctx, n_pages=n_pages, tp_rank=0,
                         tp_world=1, max_tokens=max_tokens, comm=None)
        self.small_path_tokens = 0                                   # every batch size takes the tensor-core path

    # ------------------------------------------------------------------ weights
    def _load_ffn(self, src: WeightSource, p: str, layer: int):
        e0, e1 = self.ep_rank * self.E_local, (self.ep_rank + 1) * self.E_local
        f, d = self.cfg.ffn, self.cfg.d_model
        g = src.get(p + "ffn_gate_exps.weight").rows(e0, e1).to_float().view(self.E_local, f, d)
        u = src.get(p + "ffn_up_exps.weight").rows(e0, e1).to_float().view(self.E_local, f, d)
        w13 = torch.stack((g, u), dim=2).reshape(self.E_local * 2 * f, d).to(torch.bfloat16).contiguous()
        del g, u
        w2 = src.get(p + "ffn_down_exps.weight").rows(e0, e1).to_float().view(self.E_local * d, f).to(torch.bfloat16).contiguous()
        rw = src.get(p + "ffn_gate_inp.weight").to_float().contiguous()
        rb = src.get(p + "ffn_gate_inp.bias").to_float().contiguous() if src.has(p + "ffn_gate_inp.bias") else None
        self.experts.append(_Experts(rw, rb, w13, w2))
        return None, None

    def weight_bytes(self) -> int:
        n = super().weight_bytes()
        for e in self.experts:
            n += (e.w13.numel() + e.w2.numel()) * 2 + e.router_w.numel() * 4
        return n

    def placement_digest(self) -> str:
        """Stable digest of which rank serves which experts."""
        body = {"experts": self.E, "world": self.ep_world,
                "ranges": [[r * self.E_local, (r + 1) * self.E_local] for r in range(self.ep_world)]}
        return "sha256:" + hashlib.sha256(json.dumps(body, sort_keys=True, separators=(",", ":")).encode()).hexdigest()

    # ------------------------------------------------------------------ workspaces
    def _alloc(self):
        super()._alloc()
        heap, dev = self.ep.heap, self.device
        T, d, f = self.max_tokens, self.d, self.cfg.ffn
        self.x, self.x_off = heap.alloc_tensor((T, d), torch.float32)               # peers add expert outputs into it
        self.recv_x, self.recv_x_off = heap.alloc_tensor((self.E_local * self.cap, d), torch.bfloat16)
        self.recv_meta, self.recv_meta_off = heap.alloc_tensor((self.E_local * self.cap, 2), torch.int32)
        self.recv_w, self.recv_w_off = heap.alloc_tensor((self.E_local * self.cap,), torch.float32)
        self.counts, self.counts_off = heap.alloc_tensor((2, self.E_local), torch.int32)
        self.counts.zero_()
        self.hf32 = self._ws("hf32", (T, d), torch.float32)                    # normalised hidden in fp32, for the router
        self.hmid = self._ws("hmid", (self.E_local * self.cap, f), torch.bfloat16)
        self.topk_ids = self._ws("topk_ids", (T, self.top_k), torch.int32, zero=True)
        self.topk_w = self._ws("topk_w", (T, self.top_k), torch.float32, zero=True)
        self.moe_status = self.status

    # ------------------------------------------------------------------ forward
    def _embed(self, T: int):
        ops.embedding(self.ids, self.x[:T], self.emb_type, self.emb.main, self.emb.plane2)
        # Counters of both parities are free here: every earlier forward of this rank has finished with
        # them (stream order) and no peer touches them before it has passed the barrier below.
        ops.moe_zero(self.counts)
        if self.ep_world > 1:
            self.ep.heap.barrier(ch=2)

    @nvtx_method("moe.dispatch+experts+combine")
    def _ffn_dense(self, li: int, L: _Layer, T: int, x, hb_d, hb_f, gu, fused: bool = False, slots: bool = False, table=None) -> int:
        ex, heap = self.experts[li], self.ep.heap
        par = li & 1
        d, f = self.d, self.cfg.ffn
        ops.moe_route_dispatch(hb_d, self.hf32[:T], ex.router_w, ex.router_b, self.top_k, self.E_local, self.cap, self.recv_x_off,
                               self.recv_meta_off, self.recv_w_off, self.counts_off + par * self.E_local * 4, heap.table,
                               topk_ids=self.topk_ids, topk_w=self.topk_w, status=self.status)
        n = 3
        if li + 1 < len(self.layers):
            # The other parity was last read by the previous layer's GEMMs (finished, stream order) and is
            # next written by peers only after they pass this layer's closing barrier.
            ops.moe_zero(self.counts[1 - par])
            n += 1
        ops.moe_gemm(self.recv_x, ex.w13, self.E_local, self.cap, 2 * f, d, self.counts[par], 1, out_bf16=self.hmid, ldc=f,
                     status=self.status)
        ops.moe_gemm(self.hmid, ex.w2, self.E_local, self.cap, d, f, self.counts[par], 2, ldc=d, meta=self.recv_meta,
                     gate_w=self.recv_w, sym=heap.table, sym_off=self.x_off, status=self.status)
        return n

    def _ffn_hf(self, T: int):
        return self.hf32[:T]

    def _layers_small(self, nb: int, max_ctx_pages: int):
        return self._layers_dense(nb, True, nb, 1, max_ctx_pages)
