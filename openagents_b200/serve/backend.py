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

    def step(self, seq_ids: list[int], new_tokens: list[list[int]], params: list, uniforms: list[float]) -> list[int]:
        """Append tokens to each sequence and sample one token per sequence (``params[i]`` are its sampling
        parameters, ``uniforms[i]`` the random number in [0, 1) its draw uses).  This is what the scheduler calls; the
        default samples on the host from ``forward``'s logits, the CUDA backend samples on the device and copies back
        four bytes per sequence."""
        logits = self.forward(seq_ids, new_tokens)
        self.last_d2h_bytes = logits.numel() * 4 if logits.is_cpu and self.name != "cpu" else 0
        return [sample_row(logits[i], params[i], uniforms[i]) for i in range(len(seq_ids))]

    last_d2h_bytes = 0

    # ---- speculative decoding support (optional): a backend that implements all three can verify drafted tokens
    supports_verify = False

    def verify(self, seq_id: int, tokens: list[int]) -> list[int]:
        """Append ``tokens`` and return the greedy prediction after EACH of them (``len(tokens)`` ids)."""
        raise NotImplementedError

    def truncate(self, seq_id: int, new_len: int):
        """Forget the sequence's positions from ``new_len`` on."""
        raise NotImplementedError

    def seq_len(self, seq_id: int) -> int:
        raise NotImplementedError

    # ---- scoring support (optional): log-probabilities of given continuations (evaluation packs, ``logprobs``)
    supports_score = False

    def score(self, seq_id: int, tokens: list[int], targets: list[int]) -> list[float]:
        """Append ``tokens``; natural-log probability of ``targets[i]`` as the token after ``tokens[i]`` (a negative target
        yields 0.0).  ``len(targets) == len(tokens)``."""
        raise NotImplementedError

    @property
    def max_context(self) -> int | None:
        """Longest sequence (prompt + generated) the backend can hold, or None when it does not know."""
        return None

    def publish(self, seq_id: int, tokens: list[int]):
        pass

    def end(self, seq_id: int):
        raise NotImplementedError

    def kv_stats(self) -> dict:
        return {}

    def topology(self) -> dict:
        return {"mode": "replicated", "stages": [{"nodeRef": "node.local", "layerStart": 0,
                                                   "layerEnd": self.cfg.n_layers, "role": "stage"}]}


def sample_row(logits: torch.Tensor, p, u: float) -> int:
    """One token from a [V] logits row, the way the device sampler does it: arg-max when greedy, else the ``top_k``
    (at most 64) largest logits, softmax at ``temperature``, the shortest prefix whose mass reaches ``top_p``, and the
    inverse CDF at ``u``."""
    if p.greedy:
        return int(torch.argmax(logits))
    k = min(p.top_k if p.top_k > 0 else 64, 64, logits.numel())
    vals, idx = torch.topk(logits.float(), k)
    probs = torch.exp((vals - vals[0]) / max(p.temperature, 1e-6))
    probs = probs / probs.sum()
    keep = k
    if p.top_p < 1.0:
        keep = min(k, int((torch.cumsum(probs, 0) < p.top_p).sum().item()) + 1)
    c = torch.cumsum(probs[:keep], 0)
    pick = int((c <= u * float(c[-1])).sum().item())
    return int(idx[min(pick, keep - 1)])


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

    supports_verify = True

    @torch.no_grad()
    def verify(self, seq_id, tokens):
        from ..oracle.models import llama_forward
        return llama_forward(self.cfg, self.W, torch.tensor(tokens, dtype=torch.long), self.caches[seq_id]).float().argmax(-1).tolist()

    supports_score = True

    @torch.no_grad()
    def score(self, seq_id, tokens, targets):
        from ..oracle.models import llama_forward
        lp = torch.log_softmax(llama_forward(self.cfg, self.W, torch.tensor(tokens, dtype=torch.long), self.caches[seq_id]).double(), -1)
        t = torch.tensor(targets, dtype=torch.long)
        out = lp.gather(1, t.clamp(min=0).unsqueeze(1)).squeeze(1)
        return torch.where(t >= 0, out, torch.zeros_like(out)).tolist()

    def truncate(self, seq_id, new_len):
        self.caches[seq_id].truncate(new_len)

    def seq_len(self, seq_id):
        return self.caches[seq_id].length

    @property
    def max_context(self):
        return self.cfg.context

    def kv_stats(self):
        return {"sequences": len(self.caches), "tokens": sum(c.length for c in self.caches.values())}


class CudaBackend(Backend):
    """The sm_100a engine (dense ``LlamaEngine``, tensor-parallel when given a communicator, or the expert-parallel
    ``MoEEngine`` for models with experts).  Sampling happens on the device: greedy rows take the engine's fused
    arg-max (merged across vocabulary shards under tensor parallelism), the others the top-k / top-p kernel; a step
    copies back four bytes per sequence."""
    name = "cuda"

    def __init__(self, engine):
        self.engine, self.cfg = engine, engine.cfg
        self._u = self._ids = self._scratch = None

    @classmethod
    def from_gguf(cls, path: str, device="cuda:0", max_num_seqs: int = 64, max_ctx: int = 4096, max_tokens: int = 4096,
                  tp_rank: int = 0, tp_world: int = 1, comm=None, ep_rank: int = 0, ep_world: int = 1):
        from ..models.qweight import GGUFSource
        src = GGUFSource(path, device)
        if src.cfg.n_experts:
            from ..models.moe_engine import MoEEngine
            eng = MoEEngine(src.cfg, src, device=device, max_batch=max_num_seqs, max_ctx=max_ctx, max_tokens=max_tokens,
                            ep_rank=ep_rank, ep_world=ep_world, comm=comm)
        else:
            from ..models.engine import LlamaEngine
            eng = LlamaEngine(src.cfg, src, device=device, max_batch=max_num_seqs, max_ctx=max_ctx, max_tokens=max_tokens,
                              tp_rank=tp_rank, tp_world=tp_world, comm=comm)
        b = cls(eng)
        b.tokenizer_metadata = {k: v for k, v in src.file.metadata.items() if k.startswith("tokenizer.")}
        return b

    def begin(self, seq_id, prompt):
        return self.engine.begin(seq_id, prompt)

    def _run(self, seq_ids, new_tokens):
        if all(len(t) == 1 for t in new_tokens):
            return self.engine.decode(seq_ids, [t[0] for t in new_tokens])
        return self.engine.forward_tokens(seq_ids, new_tokens)

    def forward(self, seq_ids, new_tokens):
        logits, _ = self._run(seq_ids, new_tokens)
        return self._full_rows(logits).float().cpu()

    def _full_rows(self, logits):
        """[B, V] rows from this rank's vocabulary shard (tensor parallel: an all-gather over the process group; every
        rank then holds the same rows)."""
        e = self.engine
        if not getattr(e, "vocab_sharded", False):
            return logits
        import torch.distributed as dist
        parts = [torch.empty_like(logits) for _ in range(e.world)]
        dist.all_gather(parts, logits.contiguous())
        return torch.cat(parts, dim=-1)

    def step(self, seq_ids, new_tokens, params, uniforms):
        from ..ops import cuda_ops as ops
        B = len(seq_ids)
        logits, ids = self._run(seq_ids, new_tokens)
        hot = [i for i, p in enumerate(params) if not p.greedy]
        if hot:
            dev = logits.device
            out = ids.clone()
            full = self._full_rows(logits) if getattr(self.engine, "vocab_sharded", False) else logits
            groups: dict[tuple, list[int]] = {}
            for i in hot:
                p = params[i]
                k = min(p.top_k if p.top_k > 0 else 64, 64, full.shape[1])
                groups.setdefault((float(p.temperature), k, float(p.top_p)), []).append(i)
            for (temp, k, top_p), rows in groups.items():
                idx = torch.tensor(rows, device=dev)
                sub = full.index_select(0, idx).float().contiguous()
                u = torch.tensor([uniforms[i] for i in rows], dtype=torch.float32).pin_memory().to(dev, non_blocking=True)
                picked = torch.empty(len(rows), dtype=torch.int32, device=dev)
                ops.sample_topk(sub, temp, k, top_p, u, picked, torch.empty_like(sub))
                out[idx] = picked
            ids = out
        self.last_d2h_bytes = 4 * B
        return ids[:B].tolist()

    def publish(self, seq_id, tokens):
        self.engine.pool.publish(seq_id, tokens)

    def end(self, seq_id):
        self.engine.end(seq_id)

    supports_verify = True

    def verify(self, seq_id, tokens):
        _, ids = self.engine.forward_tokens([seq_id], [list(tokens)], all_positions=True)
        self.last_d2h_bytes = 4 * len(tokens)
        return ids[: len(tokens)].tolist()

    supports_score = True

    def score(self, seq_id, tokens, targets):
        # logits of every position fit the workspace ``max_batch`` rows at a time
        out, step = [], self.engine.max_batch
        for lo in range(0, len(tokens), step):
            chunk = list(tokens[lo: lo + step])
            logits, _ = self.engine.forward_tokens([seq_id], [chunk], all_positions=True)
            full = self._full_rows(logits[: len(chunk)]).float()
            t = torch.tensor(targets[lo: lo + step], dtype=torch.long).pin_memory().to(full.device, non_blocking=True)
            lp = torch.log_softmax(full, -1).gather(1, t.clamp(min=0).unsqueeze(1)).squeeze(1)
            out.append(torch.where(t >= 0, lp, torch.zeros_like(lp)))
        self.last_d2h_bytes = 4 * len(tokens)
        return torch.cat(out).cpu().tolist() if out else []

    def truncate(self, seq_id, new_len):
        self.engine.truncate(seq_id, new_len)

    def seq_len(self, seq_id):
        return self.engine.pool.length(seq_id)

    @property
    def max_context(self):
        from ..models.engine import PAGE
        return self.engine.max_pages * PAGE

    def kv_stats(self):
        p = self.engine.pool
        hits, lookups = p.prefix_stats
        return {"pages_total": p.n_pages, "pages_free": p.free_pages, "pages_retained": p.retained_pages, "page_size": p.page_size,
                "prefix_hits": hits, "prefix_lookups": lookups}

    def topology(self):
        e = self.engine
        ep = getattr(e, "ep_world", 1)
        mode = "tensor_sharded" if e.world > 1 else "sparse_expert" if ep > 1 else "replicated"
        t = {"mode": mode, "tensorParallel": e.world, "expertParallel": ep,
             "stages": [{"nodeRef": "node.local", "layerStart": 0, "layerEnd": self.cfg.n_layers, "role": "stage"}]}
        t["placementDigest"] = (e.placement_digest() if hasattr(e, "placement_digest") else
                                "sha256:" + hashlib.sha256(repr(sorted(t.items(), key=lambda kv: kv[0])).encode()).hexdigest())
        return t


def open_backend(path: str, backend: str = "cuda", device="cuda:0", **engine_args) -> Backend:
    """The backend for a GGUF file by its architecture: the paged engine (or the fp32 oracle) for the llama and gpt-oss
    families, the recompute backends for GPT-2-shape checkpoints."""
    from ..gguf import GGUFFile
    with GGUFFile(path) as f:
        arch = f.metadata.get("general.architecture")
    if arch == "gpt2":
        from .gpt2_backend import Gpt2CpuBackend, Gpt2CudaBackend
        if backend == "cpu":
            return Gpt2CpuBackend.from_gguf(path)
        if max(engine_args.get("tp_world", 1), engine_args.get("ep_world", 1)) > 1:
            raise ValueError("GPT-2-shape checkpoints are served on one GPU")
        return Gpt2CudaBackend.from_gguf(path, device=device, rows=min(8, engine_args.get("max_num_seqs", 8)))
    if backend == "cpu":
        return CpuBackend.from_gguf(path)
    return CudaBackend.from_gguf(path, device=device, **engine_args)
