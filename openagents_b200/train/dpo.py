"""Direct preference optimisation on the trainer.

The reference's A5 workload fixes the pair loss (``softplus(-(r_chosen - r_rejected))`` with the implicit reward
``beta * (log pi(y|x) - log pi_ref(y|x))``; apps/openagents.com/workers/api/src/cs336-a5-dpo-preference-workload.ts:85-122,
restated in ``oracle.cs336.dpo_pair_loss``) and its post-training receipt lists preference work as the lane after
instruction tuning (training-post-training-instruct-sft.ts:24-27).  This module runs that loss on the GPU trainer without a
second forward pass:

* a micro-batch holds P pairs as 2P rows: rows 0..P-1 the chosen answers, rows P..2P-1 the rejected ones, each rendered
  with the instruction-tuning template, prompt and padding masked;
* the forward pass ends in the fused cross-entropy run in loss-only mode: per-token ``-log p`` with the logits left intact;
* ``dpo_row_scales`` (a few device-side tensor operations, no host round trip) sums them per sequence, forms the margins
  against the reference log-probabilities, and returns one signed factor per row: ``+beta * sigmoid(-margin) / pairs`` for
  chosen rows, the negative for rejected rows.  ``d loss / d logits = factor * (softmax - onehot)`` is exactly what the
  cross-entropy kernel writes when given per-row factors, so the ordinary backward pass follows;
* the reference log-probabilities come from one forward-only pass per batch with the frozen starting weights
  (``DpoTrainer.reference_logps``, before the first update, or from a stored table).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import sft


def build_preference_batch(pairs, tokenizer, seq_len: int, pad_id: int = 0):
    """``pairs``: ``{"messages": [...prompt turns...], "chosen": str, "rejected": str}``.  Returns int64 ``tokens`` /
    ``targets`` of shape ``[2P, seq_len]`` (chosen rows first; prompt and padding targets are -1) and the number of answer
    tokens per row."""
    rows = []
    for key in ("chosen", "rejected"):
        for p in pairs:
            ids, mask = sft.render_example(list(p["messages"]) + [{"role": "assistant", "content": p[key]}], tokenizer)
            # only the final answer is judged: earlier assistant turns belong to the prompt
            last = len(ids) - 1 - mask[::-1].index(1)
            first = last
            while first > 0 and mask[first - 1]:
                first -= 1
            mask = [1 if first <= i <= last else 0 for i in range(len(ids))]
            if len(ids) > seq_len + 1:
                raise ValueError(f"an example has {len(ids)} tokens, the window holds {seq_len + 1}")
            rows.append((ids, mask))
    tokens = torch.full((len(rows), seq_len), pad_id, dtype=torch.int64)
    targets = torch.full((len(rows), seq_len), -1, dtype=torch.int64)
    counts = []
    for r, (ids, mask) in enumerate(rows):
        n = len(ids) - 1
        tokens[r, :n] = torch.tensor(ids[:-1])
        t = torch.tensor(ids[1:])
        m = torch.tensor(mask[1:], dtype=torch.bool)
        targets[r, :n] = torch.where(m, t, torch.full_like(t, -1))
        counts.append(int(m.sum()))
    return tokens, targets, counts


def sequence_logps(loss_rows: torch.Tensor, n_rows: int) -> torch.Tensor:
    """Per-token losses ``-log p`` [n_rows * T] (0 where masked) -> log-probability of each row's answer [n_rows]."""
    return -loss_rows.view(n_rows, -1).sum(1)


def dpo_row_scales(loss_rows: torch.Tensor, ref_logps: torch.Tensor, beta: float, pairs_in_step: int, stats: dict | None = None):
    """``ref_logps`` [2P] in the same row order.  Returns (row factors [2P * T], this micro-batch's share of the mean pair
    loss).  ``stats`` (optional dict) receives the margins and the reward accuracy as device tensors."""
    B = ref_logps.numel()
    P = B // 2
    pol = sequence_logps(loss_rows, B)
    margin = beta * ((pol[:P] - ref_logps[:P]) - (pol[P:] - ref_logps[P:]))
    loss = F.softplus(-margin).sum() / pairs_in_step
    g = beta * torch.sigmoid(-margin) / pairs_in_step
    seq = torch.cat([g, -g])
    T = loss_rows.numel() // B
    if stats is not None:
        stats["margins"] = margin.detach()
        stats["rewardAccuracy"] = (margin > 0).float().mean()
    return seq.unsqueeze(1).expand(B, T).reshape(-1).float(), loss


class DpoTrainer:
    """Wraps a ``Trainer``: the same optimizer, sharding and overlap; only the objective differs."""

    def __init__(self, trainer, beta: float = 0.1):
        self.trainer, self.beta = trainer, beta
        self.last_stats: list[dict] = []

    def reference_logps(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """Log-probabilities of every row's answer under the CURRENT weights, ``[accum, 2P]``: call it before the first
        update (the starting weights are the reference policy) and keep the result with the batch."""
        tr = self.trainer
        tr._sync_params()
        out = []
        for a in range(tokens.shape[0]):
            rows = tr.model.forward_backward(tokens[a], targets[a], backward=False)
            out.append(sequence_logps(rows, tokens.shape[1]))
        return torch.stack(out)

    def train_step(self, tokens: torch.Tensor, targets: torch.Tensor, ref_logps: torch.Tensor) -> torch.Tensor:
        """``tokens`` / ``targets`` ``[accum, 2P, T]``, ``ref_logps`` ``[accum, 2P]`` (device).  Returns the mean pair loss of this
        rank's batch (device scalar); ``last_stats[a]`` holds each micro-batch's margins and reward accuracy."""
        accum, B = tokens.shape[0], tokens.shape[1]
        pairs = accum * (B // 2)
        self.last_stats = [{} for _ in range(accum)]
        fns = [(lambda rows, a=a: dpo_row_scales(rows, ref_logps[a], self.beta, pairs, self.last_stats[a])) for a in range(accum)]
        return self.trainer.train_step(tokens, targets, row_scale_fns=fns)

    def reward_accuracy(self) -> float:
        return float(torch.stack([s["rewardAccuracy"] for s in self.last_stats]).mean()) if self.last_stats else float("nan")
