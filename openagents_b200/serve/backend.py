"""Generation backends behind one interface: ``cuda`` (the sm_100a engine) and ``cpu`` (the fp32
oracle).  ``--backend`` accepts exactly these two, like the reference server's flag
(apps/pylon/docs/2026-06-09-pylon-qwen35-local-inference-roadmap.md:137-160 lists
``--backend cpu|cuda|metal``); there is no dispatch between them on a hot path: a server is built
with one backend and keeps it.
"""
from __future__ import annotations

import hashlib

import torch

from ..models.config import ModelConfig


class Backend:
    name = "abstract"
    cfg: ModelConfig

    def begin(self, seq_id: int, prompt: list[int]) -> int:
        """Open a sequence; returns how many prompt tokens are served from the prefix cache."""
        raise NotImplementedError

    def forward(self, seq_ids: list[int], new_tokens: list[list[int]]) -> torch.Tensor:
        """Append tokens to each sequence; logits [B, V] (float, CPU) of each last token."""
        raise NotImplementedError

    def publish(self, seq_id: int, tokens: list[int]):
        pass

    def end(self, seq_id: int):
        raise NotImplementedError

    def kv_stats(self) -> dict:
        return {}

    def topology(self) -> dict:
        return {"mode": "replicated", "stages": [{"nodeRef": "node.local", "layerStart": 0,
                                                   "layerEnd": self.cfg.n_layers, "role": "stage"}]}


class CpuBackend(Backend):
    """fp32 reference math on the host: the oracle, usable as a (slow) server backend."""
    name = "cpu"

    def __init__(self, cfg: ModelConfig, weights: dict[str, torch.Tensor]):
        from ..oracle.models import KVCacheRef
        self.cfg, self.W = cfg, weights
        self._mk = lambda: KVCacheRef(cfg.n_layers)
        self.caches: dict[int, object] = {}

    @classmethod
    def from_gguf(cls, path: str):
        from ..models.weights import load_gguf_float
        cfg, W = load_gguf_float(path)
        return cls(cfg, W)

    def begin(self, seq_id, prompt):
        if seq_id in self.caches:
            raise KeyError(f"sequence {seq_id} already exists")
        self.caches[seq_id] = self._mk()
        return 0

    @torch.no_grad()
    def forward(self, seq_ids, new_tokens):
        from ..oracle.models import llama_forward
        rows = [llama_forward(self.cfg, self.W, torch.tensor(t, dtype=torch.long), self.caches[s])[-1]
                for s, t in zip(seq_ids, new_tokens)]
        return torch.stack(rows).float()

    def end(self, seq_id):
        self.caches.pop(seq_id, None)

    def kv_stats(self):
        return {"sequences": len(self.caches), "tokens": sum(c.length for c in self.caches.values())}


class CudaBackend(Backend):
    name = "cuda"

    def __init__(self, engine):
        self.engine, self.cfg = engine, engine.cfg

    @classmethod
    def from_gguf(cls, path: str, device="cuda:0", max_num_seqs: int = 64, max_ctx: int = 4096, max_tokens: int = 4096,
                  tp_rank: int = 0, tp_world: int = 1, comm=None):
        from ..models.engine import LlamaEngine
        from ..models.qweight import GGUFSource
        src = GGUFSource(path, device)
        eng = LlamaEngine(src.cfg, src, device=device, max_batch=max_num_seqs, max_ctx=max_ctx, max_tokens=max_tokens,
                          tp_rank=tp_rank, tp_world=tp_world, comm=comm)
        return cls(eng)

    def begin(self, seq_id, prompt):
        return self.engine.begin(seq_id, prompt)

    def forward(self, seq_ids, new_tokens):
        if all(len(t) == 1 for t in new_tokens):
            logits, _ = self.engine.decode(seq_ids, [t[0] for t in new_tokens])
        else:
            logits, _ = self.engine.forward_tokens(seq_ids, new_tokens)
        return logits.float().cpu()

    def publish(self, seq_id, tokens):
        self.engine.pool.publish(seq_id, tokens)

    def end(self, seq_id):
        self.engine.end(seq_id)

    def kv_stats(self):
        p = self.engine.pool
        hits, lookups = p.prefix_stats
        return {"pages_total": p.n_pages, "pages_free": p.free_pages, "page_size": p.page_size,
                "prefix_hits": hits, "prefix_lookups": lookups}

    def topology(self):
        e = self.engine
        mode = "tensor_sharded" if e.world > 1 else "replicated"
        t = {"mode": mode, "tensorParallel": e.world,
             "stages": [{"nodeRef": "node.local", "layerStart": 0, "layerEnd": self.cfg.n_layers, "role": "stage"}]}
        t["placementDigest"] = "sha256:" + hashlib.sha256(repr(sorted(t.items(), key=lambda kv: kv[0])).encode()).hexdigest()
        return t
