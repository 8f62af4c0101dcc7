"""Evaluation packs: a frozen set of tasks with metric gates, run against one checkpoint, ending in a decision.

The reference cites one such pack by name (``benchmark://psion/actual_pretraining/checkpoint_eval@2026.04.02``) and publishes
the receipt of its decision: the pack ref, the checkpoint ref, the number of metric gates and how many passed, and a
decision state (apps/openagents.com/workers/api/src/training-ablation-derisking-ledger.ts:252-283); the pack's code is
upstream (``psionic-eval``).  The evidence contract files the outcome under the ``eval_run`` kind
(psionic-evidence-contract.ts:10-18).  Here the pack is data (tasks + gates), ``run_pack`` runs the tasks through the
scorers, ``decide`` applies the gates: every required gate passed -> ``continue``; a failed gate marked
``rollback_on_fail`` -> ``rollback``; any other failed required gate -> ``hold``.
"""
from __future__ import annotations

import hashlib
import json
import math
from dataclasses import dataclass, field

from . import scorers

DECISION_SCHEMA = "b200.eval.checkpoint_eval_decision.v1"
_CMP = {"<=": lambda v, t: v <= t, ">=": lambda v, t: v >= t, "<": lambda v, t: v < t, ">": lambda v, t: v > t}


@dataclass(frozen=True)
class MetricGate:
    metric: str                      # "<task>.<field>", e.g. "heldout.loss"
    comparator: str                  # <= | >= | < | >
    threshold: float
    required: bool = True
    rollback_on_fail: bool = False   # a regression so bad that the previous checkpoint should be restored

    def __post_init__(self):
        if self.comparator not in _CMP:
            raise ValueError(f"unknown comparator {self.comparator!r}")


@dataclass
class EvalPack:
    package_ref: str                              # e.g. "benchmark://b200/gpt2/checkpoint_eval@1"
    tasks: list[dict] = field(default_factory=list)   # {"name", "kind": perplexity|multiple_choice|exact_match, ...task arguments}
    gates: list[MetricGate] = field(default_factory=list)

    def digest(self) -> str:
        body = {"packageRef": self.package_ref, "tasks": [{k: (v if isinstance(v, (str, int, float, bool, list, dict, type(None))) else repr(type(v)))
                                                            for k, v in t.items() if k != "dataset"} for t in self.tasks],
                "gates": [[g.metric, g.comparator, g.threshold, g.required, g.rollback_on_fail] for g in self.gates]}
        return "sha256:" + hashlib.sha256(json.dumps(body, sort_keys=True, separators=(",", ":")).encode()).hexdigest()


def decide(metrics: dict[str, float], gates: list[MetricGate]) -> dict:
    rows, state = [], "continue"
    for g in gates:
        v = metrics.get(g.metric)
        ok = v is not None and not (isinstance(v, float) and math.isnan(v)) and _CMP[g.comparator](v, g.threshold)
        rows.append({"metric": g.metric, "comparator": g.comparator, "threshold": g.threshold, "value": v, "passed": ok, "required": g.required})
        if not ok and g.required:
            state = "rollback" if (g.rollback_on_fail or state == "rollback") else "hold"
    return {"decisionState": state, "gates": rows, "metricGateCount": len(rows), "passedMetricGateCount": sum(r["passed"] for r in rows)}


def run_pack(pack: EvalPack, backend, tokenizer, checkpoint_ref: str) -> dict:
    """Run every task, flatten the scalar results to ``<task>.<field>`` metrics and apply the gates."""
    metrics: dict[str, float] = {}
    details = {}
    for t in pack.tasks:
        kind, name = t["kind"], t["name"]
        if kind == "perplexity":
            r = scorers.perplexity(backend, t["dataset"], t.get("max_windows"), bytes_per_token=t.get("bytes_per_token"))
        elif kind == "multiple_choice":
            r = scorers.multiple_choice(backend, t["items"], tokenizer, t.get("length_normalised", True))
        elif kind == "exact_match":
            r = scorers.exact_match(backend, t["items"], tokenizer, t.get("max_new_tokens", 32), t.get("stop_ids", ()))
        else:
            raise ValueError(f"unknown task kind {kind!r}")
        details[name] = {k: v for k, v in r.items() if k not in ("picks", "rows")}
        for k, v in r.items():
            if isinstance(v, (int, float)) and not isinstance(v, bool):
                metrics[f"{name}.{k}"] = float(v)
    d = decide(metrics, pack.gates)
    out = {"schema": DECISION_SCHEMA, "benchmarkPackageRef": pack.package_ref, "packDigest": pack.digest(), "checkpointRef": checkpoint_ref,
           "backend": backend.name, "metrics": metrics, "tasks": details, **d}
    out["decisionDigest"] = "sha256:" + hashlib.sha256(json.dumps({k: out[k] for k in ("benchmarkPackageRef", "packDigest", "checkpointRef", "decisionState",
                                                                                           "metricGateCount", "passedMetricGateCount")},
                                                                   sort_keys=True).encode()).hexdigest()
    return out


def eval_run_evidence(decision: dict, created_at_iso: str) -> dict:
    """The decision as an evidence-only record of kind ``eval_run`` (it can inform a promotion, never make one)."""
    from ..gateway.evidence import evidence_record
    safe = decision["decisionDigest"].replace("sha256:", "")[:24]
    status = {"continue": "completed", "hold": "needs_review", "rollback": "retained_failure"}[decision["decisionState"]]
    return evidence_record(f"evidence.eval_run.{safe}", "eval_run", status, created_at_iso,
                           metricRefs=[f"metric.{m}" for m in sorted(decision["metrics"])][:32],
                           scorecardRefs=[f"scorecard.eval.{safe}"], modelRefs=[decision["checkpointRef"].replace("://", ":")])
