"""Local-update training rounds (DiLoCo): several inner optimizer steps per replica, one outer step per round.

The coordination protocol the reference defines for training networks carries a ``diloco`` sync profile: a window is one
local-training round with a base checkpoint, a planned number of local steps, signed pointers to the local updates, an
aggregation rule and weight, participation thresholds and a staleness bound, and names the accepted aggregate as the next
round's base (docs/nips/TRN.md:440-470, 919-962; window tags in ``control.coordination.training_window``).  It leaves
the optimizer math to the runtime.  This module is that runtime part:

* ``run_local_round``: H inner steps on one replica (any trainer with ``train_step`` and a flat fp32 master vector), result =
  the pseudo-gradient ``base - local`` plus its weight (tokens consumed);
* ``admit_updates``: which local updates enter the aggregate: the round and base checkpoint must match; an update that is
  more than ``max_staleness_windows`` rounds old goes to ``sync_reentry`` (never a bare reject, as in
  ``control.lifecycle.decide_staleness``); the round is only sealed with ``min_participants`` and ``min_weight_fraction``;
* ``aggregate``: weighted or uniform mean of the admitted pseudo-gradients;
* ``OuterOptimizer``: SGD with Nesterov momentum on the aggregate (the published DiLoCo outer optimizer: learning rate 0.7,
  momentum 0.9);
* ``DilocoReplica``: one replica of a group of processes: inner rounds on its own trainer, the aggregate by an all-reduce
  of weight x pseudo-gradient over ``torch.distributed`` (NCCL between GPUs, gloo on the CPU), the same outer step on
  every replica, so all replicas start the next round from identical parameters.

Between two outer steps the replicas exchange nothing: the traffic of one round is one all-reduce of the parameter vector,
H times less than per-step data parallelism.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.distributed as dist


@dataclass
class DilocoConfig:
    inner_steps: int = 16                  # H: planned local steps per round
    outer_lr: float = 0.7
    outer_momentum: float = 0.9
    nesterov: bool = True
    aggregation_rule: str = "weighted_avg"  # weighted_avg | uniform_avg
    aggregation_weight: str = "tokens"      # tokens | examples | steps | uniform
    min_participants: int = 1
    min_weight_fraction: float = 0.8        # of the planned total weight
    max_staleness_windows: int = 1

    def window_tags(self, round_index: int, base_checkpoint: str) -> list[list]:
        """The profile's recommended tags for this round's window event."""
        return [["sync_profile", "diloco"], ["aggregation_rule", self.aggregation_rule], ["aggregation_weight", self.aggregation_weight],
                ["base_checkpoint", base_checkpoint], ["round", str(round_index)], ["planned_local_steps", str(self.inner_steps)],
                ["min_participants", str(self.min_participants)], ["min_weight_fraction", str(self.min_weight_fraction)],
                ["max_staleness_windows", str(self.max_staleness_windows)],
                ["inner_optimizer", "adamw"], ["outer_optimizer", "nesterov_sgd" if self.nesterov else "momentum_sgd"]]


@dataclass
class LocalUpdate:
    participant: str
    round_index: int
    base_checkpoint: str
    delta: torch.Tensor                     # base - local (pseudo-gradient), flat fp32
    local_steps: int
    tokens: int
    examples: int = 0
    losses: list = field(default_factory=list)

    def weight(self, kind: str) -> float:
        return {"tokens": float(self.tokens), "examples": float(self.examples), "steps": float(self.local_steps), "uniform": 1.0}[kind]


def run_local_round(trainer, batches, participant: str, round_index: int, base_checkpoint: str) -> LocalUpdate:
    """``batches``: iterable of ``(tokens, targets)`` for ``trainer.train_step`` (one inner step each).  The trainer's
    flat fp32 ``master`` vector is read before and after; the trainer keeps its inner optimizer state across rounds."""
    if hasattr(trainer, "_sync_params"):
        trainer._sync_params()
    base = trainer.master.detach().clone()
    losses, tokens, examples, steps = [], 0, 0, 0
    for tok, tgt in batches:
        losses.append(float(trainer.train_step(tok, tgt)))
        tokens += int(tok.numel())
        examples += int(tok.numel() // tok.shape[-1])
        steps += 1
    if hasattr(trainer, "_sync_params"):
        trainer._sync_params()
    return LocalUpdate(participant, round_index, base_checkpoint, base - trainer.master.detach(), steps, tokens, examples, losses)


def admit_updates(updates: list[LocalUpdate], cfg: DilocoConfig, round_index: int, base_checkpoint: str, planned_participants: int) -> dict:
    """Admission of one round's local updates.  Returns the admitted updates, one decision per update and whether the
    round may be sealed."""
    admitted, decisions = [], []
    for u in updates:
        behind = round_index - u.round_index
        if behind < 0:
            decisions.append({"participant": u.participant, "status": "rejected", "reason": "update_from_a_future_round"})
        elif behind > cfg.max_staleness_windows:
            decisions.append({"participant": u.participant, "status": "sync_reentry", "reason": "training.staleness.public.beyond_max_allowed_stale"})
        elif behind > 0 or u.base_checkpoint != base_checkpoint:
            # an older round within the bound, or the wrong base: the update cannot be averaged into this round's base
            decisions.append({"participant": u.participant, "status": "replay_required", "reason": "base_checkpoint_mismatch"})
        elif not bool(torch.isfinite(u.delta).all()):
            decisions.append({"participant": u.participant, "status": "rejected", "reason": "non_finite_update"})
        elif u.local_steps <= 0:
            decisions.append({"participant": u.participant, "status": "rejected", "reason": "no_local_work"})
        else:
            admitted.append(u)
            decisions.append({"participant": u.participant, "status": "accepted", "reason": None})
    kind = "uniform" if cfg.aggregation_rule == "uniform_avg" else cfg.aggregation_weight
    got = sum(u.weight(kind) for u in admitted)
    planned = sum(u.weight(kind) for u in updates if u.round_index == round_index)      # what was submitted for this round
    per = (planned / max(1, len([u for u in updates if u.round_index == round_index])))
    planned_total = per * planned_participants if planned_participants else planned
    frac = got / planned_total if planned_total > 0 else 0.0
    blockers = []
    if len(admitted) < cfg.min_participants:
        blockers.append("min_participants_not_met")
    if frac + 1e-12 < cfg.min_weight_fraction:
        blockers.append("min_weight_fraction_not_met")
    return {"admitted": admitted, "decisions": decisions, "weightFraction": frac, "sealable": not blockers, "blockers": blockers}


def aggregate(updates: list[LocalUpdate], cfg: DilocoConfig) -> torch.Tensor:
    if not updates:
        raise ValueError("nothing to aggregate")
    kind = "uniform" if cfg.aggregation_rule == "uniform_avg" else cfg.aggregation_weight
    ws = [u.weight(kind) for u in updates]
    total = sum(ws)
    if total <= 0:
        raise ValueError("aggregation weights sum to zero")
    out = torch.zeros_like(updates[0].delta)
    for u, w in zip(updates, ws):
        out.add_(u.delta, alpha=w / total)
    return out


class OuterOptimizer:
    """theta <- theta - lr * (mu * v' + g) with v' = mu * v + g (Nesterov), or theta - lr * v' (plain momentum);
    g is the aggregated pseudo-gradient."""

    def __init__(self, cfg: DilocoConfig):
        self.cfg, self.v, self.steps = cfg, None, 0

    def step(self, theta: torch.Tensor, g: torch.Tensor) -> torch.Tensor:
        c = self.cfg
        if self.v is None:
            self.v = torch.zeros_like(g)
        self.v.mul_(c.outer_momentum).add_(g)
        upd = self.v * c.outer_momentum + g if c.nesterov else self.v
        self.steps += 1
        return theta - c.outer_lr * upd

    def state_dict(self) -> dict:
        return {"v": None if self.v is None else self.v.clone(), "steps": self.steps}

    def load_state_dict(self, s: dict):
        self.v, self.steps = (None if s["v"] is None else s["v"].clone()), int(s["steps"])


class DilocoReplica:
    """One replica in a group of ``torch.distributed`` ranks.  ``trainer`` needs ``train_step``, ``master`` (flat fp32) and
    ``set_master(tensor)`` (install new parameters, refresh the working copy)."""

    def __init__(self, trainer, cfg: DilocoConfig, participant: str, group=None):
        self.trainer, self.cfg, self.participant, self.group = trainer, cfg, participant, group
        self.outer = OuterOptimizer(cfg)
        self.round_index = 0
        self.base_checkpoint = "checkpoint.round.0"
        self.history: list[dict] = []

    def _all_reduce(self, t: torch.Tensor):
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(t, group=self.group)

    def run_round(self, batches) -> dict:
        """H inner steps here, then the aggregate over all replicas and the same outer step everywhere.  A replica whose
        update is not finite contributes weight zero (the others still average theirs)."""
        c = self.cfg
        base = self.trainer.master.detach().clone()
        u = run_local_round(self.trainer, batches, self.participant, self.round_index, self.base_checkpoint)
        kind = "uniform" if c.aggregation_rule == "uniform_avg" else c.aggregation_weight
        ok = bool(torch.isfinite(u.delta).all()) and u.local_steps > 0
        w = u.weight(kind) if ok else 0.0
        num = u.delta * w if ok else torch.zeros_like(u.delta)
        stats = torch.tensor([w, 1.0 if ok else 0.0, float(u.tokens)], dtype=torch.float64, device=num.device)
        self._all_reduce(num)
        self._all_reduce(stats)
        total_w, participants = float(stats[0]), int(stats[1])
        sealed = participants >= c.min_participants and total_w > 0
        if sealed:
            g = num / total_w
            new = self.outer.step(base, g.to(base.dtype))
        else:
            new = base                            # the round is not sealed: everyone returns to the base
        self.trainer.set_master(new)
        rec = {"round": self.round_index, "baseCheckpoint": self.base_checkpoint, "participants": participants, "sealed": sealed,
               "localSteps": u.local_steps, "tokensAllReplicas": int(stats[2]), "meanLocalLoss": sum(u.losses) / max(1, len(u.losses)),
               "pseudoGradientNorm": float(num.norm() / total_w) if sealed else None}
        self.history.append(rec)
        self.round_index += 1
        if sealed:
            self.base_checkpoint = f"checkpoint.round.{self.round_index}"
        return rec
