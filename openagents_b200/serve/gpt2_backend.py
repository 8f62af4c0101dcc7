"""Serving backends for GPT-2-shape checkpoints (what the trainer writes): learned positions, LayerNorm, GELU, biases.

The paged engine is built for the RMSNorm / RoPE / gated-FFN families.  A GPT-2-shape model is served by recomputing the
whole sequence on every call, on the trainer's own forward kernels (``Gpt2CudaBackend``; no KV cache, so a step costs one
forward over ``rows x seq_len`` positions) or on the fp32 oracle (``Gpt2CpuBackend``).  That is enough to chat with a
freshly tuned checkpoint, to run evaluation packs on it, and to sample roll-outs from the weights a trainer is updating
(``Gpt2CudaBackend.over_trainer`` shares the trainer's parameter buffer).
"""
from __future__ import annotations

import torch

from ..models.config import ModelConfig
from .backend import Backend


class _TokenListBackend(Backend):
    """Sequences are token lists; subclasses provide ``_logits(list of token lists) -> list of [len, V] float tensors``."""

    supports_verify = True
    supports_score = True

    def __init__(self, cfg: ModelConfig, context: int):
        self.cfg, self.context = cfg, context
        self.seqs: dict[int, list[int]] = {}

    def begin(self, seq_id, prompt):
        if seq_id in self.seqs:
            raise KeyError(f"sequence {seq_id} already exists")
        self.seqs[seq_id] = []
        return 0

    def _append(self, seq_ids, new_tokens):
        for s, t in zip(seq_ids, new_tokens):
            if len(self.seqs[s]) + len(t) > self.context:
                raise ValueError(f"sequence {s} would exceed the context of {self.context} tokens")
        for s, t in zip(seq_ids, new_tokens):
            self.seqs[s] += list(t)

    def forward(self, seq_ids, new_tokens):
        self._append(seq_ids, new_tokens)
        rows = self._logits([self.seqs[s] for s in seq_ids])
        return torch.stack([r[-1] for r in rows]).float().cpu()

    def score(self, seq_id, tokens, targets):
        old = len(self.seqs[seq_id])
        self._append([seq_id], [tokens])
        lp = torch.log_softmax(self._logits([self.seqs[seq_id]])[0][old:].double(), -1)
        t = torch.tensor(targets, dtype=torch.long, device=lp.device)
        out = lp.gather(1, t.clamp(min=0).unsqueeze(1)).squeeze(1)
        return torch.where(t >= 0, out, torch.zeros_like(out)).cpu().tolist()

    def verify(self, seq_id, tokens):
        old = len(self.seqs[seq_id])
        self._append([seq_id], [tokens])
        return self._logits([self.seqs[seq_id]])[0][old:].argmax(-1).cpu().tolist()

    def truncate(self, seq_id, new_len):
        del self.seqs[seq_id][new_len:]

    def seq_len(self, seq_id):
        return len(self.seqs[seq_id])

    def end(self, seq_id):
        self.seqs.pop(seq_id, None)

    @property
    def max_context(self):
        return self.context

    def kv_stats(self):
        return {"sequences": len(self.seqs), "tokens": sum(len(v) for v in self.seqs.values()), "kv_cache": "none (recompute)"}


class Gpt2CpuBackend(_TokenListBackend):
    name = "cpu"

    def __init__(self, cfg: ModelConfig, weights: dict[str, torch.Tensor]):
        super().__init__(cfg, cfg.context)
        self.W = {k: v.float() for k, v in weights.items()}
        self.W["token_embd.weight"] = self.W["token_embd.weight"][: cfg.vocab]

    @classmethod
    def from_gguf(cls, path: str):
        from ..models.weights import load_gguf_float
        return cls(*load_gguf_float(path))

    @torch.no_grad()
    def _logits(self, seqs):
        from ..oracle.models import gpt2_forward
        return [gpt2_forward(self.cfg, self.W, torch.tensor(s, dtype=torch.long)[None])[0] for s in seqs]


class Gpt2CudaBackend(_TokenListBackend):
    name = "cuda"

    def __init__(self, cfg: ModelConfig, model, rows: int, seq_len: int, sync=None):
        """``model``: a ``train.gpt2.GPT2Model`` (forward-only is enough).  ``sync``: called before every forward (a live
        trainer waits there for its parameter all-gather)."""
        super().__init__(cfg, min(seq_len, cfg.context))
        self.model, self.rows, self.T, self.sync = model, rows, seq_len, sync
        self.device = model.dev
        self._minus = torch.full((rows, seq_len), -1, dtype=torch.int64, device=self.device)

    @classmethod
    def from_weights(cls, cfg: ModelConfig, weights: dict[str, torch.Tensor], device="cuda:0", rows: int = 8, seq_len: int | None = None):
        from ..train.gpt2 import GPT2Model, param_layout
        seq_len = seq_len or cfg.context
        if seq_len % 64 or seq_len > cfg.context:
            raise ValueError("the window must be a multiple of 64 and fit the model's context")
        slots, total, _ = param_layout(cfg)
        flat = torch.zeros(total, dtype=torch.bfloat16, device=device)
        for s in slots:
            w = weights[s.name].to(device=device, dtype=torch.bfloat16)
            view = flat[s.offset: s.offset + s.numel].view(*s.shape)
            if s.name == "token_embd.weight":
                view[: w.shape[0]].copy_(w[: s.shape[0]])           # the padded vocabulary rows stay zero
            else:
                view.copy_(w.view(*s.shape))
        model = GPT2Model(cfg, flat, None, slots, rows, seq_len)
        model.refresh_param_views()
        return cls(cfg, model, rows, seq_len)

    @classmethod
    def from_gguf(cls, path: str, device="cuda:0", rows: int = 8, seq_len: int | None = None):
        from ..models.weights import load_gguf_float
        cfg, W = load_gguf_float(path)
        return cls.from_weights(cfg, W, device, rows, seq_len)

    @classmethod
    def over_trainer(cls, trainer):
        """Sample from the weights a ``train.trainer.Trainer`` is updating (same buffers, no copy)."""
        m = trainer.model
        return cls(trainer.cfg.model, m, m.B, m.T, sync=trainer._sync_params)

    @torch.no_grad()
    def _logits(self, seqs):
        out = []
        V = self.cfg.vocab
        for lo in range(0, len(seqs), self.rows):
            group = seqs[lo: lo + self.rows]
            tok = torch.zeros((self.rows, self.T), dtype=torch.int64)
            for r, s in enumerate(group):
                tok[r, : len(s)] = torch.tensor(s, dtype=torch.int64)
            if self.sync:
                self.sync()
            self.model.forward_backward(tok.pin_memory().to(self.device, non_blocking=True), self._minus, backward=False)
            logits = self.model.logits.view(self.rows, self.T, -1)
            out += [logits[r, : len(s), :V].float() for r, s in enumerate(group)]      # copies: the buffer is reused by the next group
        return out
