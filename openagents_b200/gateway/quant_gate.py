"""The quantization evaluation gate: a quantized lane is promoted only when it holds accepted outcomes.

Rule (inference/khala-quantization-eval-gate.ts:109-118 policy, :150-322 decision): run the same verified tasks on the original
and on the quantized model; pass when the accepted-outcome rate held or improved; pass when it dropped by at most
``max_accepted_rate_drop_abs`` (0.02) AND cost per accepted outcome improved by at least ``min_cost_improvement_frac``
(0.15); otherwise fail; aggressive scopes (KV cache, attention) additionally need an explicit acknowledgement; no samples or no
baseline accepted outcome fail closed.  The result is decision grade only with real-sweep evidence whose refs are all present
and whose precisions really differ (:27-106).

``compare_backends`` produces the samples for this package's own engines: the same items through the evaluation scorers on
the original checkpoint and on its re-quantized copy (``python -m openagents_b200.gguf quantize``), cost = tokens x a price per
token of each lane.
"""
from __future__ import annotations

from .metadata import is_aggressive_scope, is_quantized_precision

GATE_SCHEMA = "openagents.khala.quant-eval-gate.v1"
EVIDENCE_SCHEMA = "openagents.khala.real-quant-sweep-evidence.v1"
DEFAULT_POLICY = {"maxAcceptedRateDropAbs": 0.02, "minCostPerAcceptedImprovementFrac": 0.15, "requireAckForAggressiveScope": True}
_DETAIL = {
    "no_comparison_samples": "No quantized-versus-original samples were given; the gate cannot prove the quantized lane and fails closed.",
    "no_baseline_accepted_outcomes": "The original precision produced no accepted outcome, so there is no quality baseline to hold against.",
    "aggressive_scope_requires_ack": "The candidate quantizes the KV cache or attention; that needs an explicit acknowledgement before promotion.",
    "accepted_rate_held": "The quantized lane held or improved the accepted-outcome rate; quality is preserved.",
    "accepted_rate_dropped_beyond_bound": "The accepted-outcome rate dropped beyond the bound; a cost win cannot offset a quality loss this large.",
    "cost_per_accepted_improved_offsets_drop": "A drop within the bound, offset by a sufficient improvement of cost per accepted outcome.",
    "accepted_rate_dropped_without_cost_win": "The accepted-outcome rate dropped without a sufficient cost improvement to offset it.",
}


def decision_grade_blockers(evidence: dict | None, sample_count: int) -> list[str]:
    if evidence is None:
        return ["real_sweep_evidence_missing"]

    def blank(k):
        return not isinstance(evidence.get(k), str) or not evidence[k].strip()
    b = []
    for key, code in (("evidenceRef", "evidence_ref_missing"), ("ownerApprovalRef", "owner_approval_ref_missing"), ("workloadRef", "workload_ref_missing")):
        if blank(key):
            b.append(code)
    if blank("originalModelId") or blank("quantizedModelId"):
        b.append("model_context_missing")
    if evidence.get("originalPrecision") != "unquantized":
        b.append("original_precision_not_full")
    try:
        reduced = is_quantized_precision(evidence.get("quantizedPrecision"))
    except ValueError:
        reduced = False
    if not reduced:
        b.append("quantized_precision_not_reduced")
    if evidence.get("originalPrecision") == evidence.get("quantizedPrecision"):
        b.append("same_precision_compared")
    for key, code in (("acceptanceVerifierRef", "acceptance_verifier_ref_missing"), ("latencyEvidenceRef", "latency_evidence_ref_missing"),
                      ("costEvidenceRef", "cost_evidence_ref_missing")):
        if blank(key):
            b.append(code)
    refs = evidence.get("publicSafeEvidenceRefs") or []
    if not refs or any(not isinstance(r, str) or not r.strip() for r in refs):
        b.append("public_safe_evidence_refs_missing")
    if evidence.get("sampleCount") != sample_count or sample_count <= 0:
        b.append("sample_count_mismatch")
    return b


def run_quantization_eval_gate(samples: list[dict], scope: str, aggressive_scope_ack: bool = False, decision_grade: bool = False,
                               real_sweep_evidence: dict | None = None, policy: dict | None = None) -> dict:
    """``samples``: ``{taskId, originalVerified, quantizedVerified, originalCostBasisMsat, quantizedCostBasisMsat}``."""
    pol = {**DEFAULT_POLICY, **(policy or {})}
    blockers = decision_grade_blockers(real_sweep_evidence, len(samples)) if decision_grade else []
    dg = decision_grade and not blockers
    aggressive = is_aggressive_scope(scope)
    n = len(samples)
    oa = sum(bool(s["originalVerified"]) for s in samples)
    qa = sum(bool(s["quantizedVerified"]) for s in samples)
    oc = sum(s["originalCostBasisMsat"] for s in samples)
    qc = sum(s["quantizedCostBasisMsat"] for s in samples)
    o_rate, q_rate = (oa / n, qa / n) if n else (None, None)
    o_cpa, q_cpa = (oc / oa if oa else None), (qc / qa if qa else None)
    delta = None if o_rate is None else q_rate - o_rate
    improv = None if o_cpa in (None, 0) or q_cpa is None else (o_cpa - q_cpa) / o_cpa
    if n == 0:
        reason = "no_comparison_samples"
    elif oa == 0:
        reason = "no_baseline_accepted_outcomes"
    elif aggressive and pol["requireAckForAggressiveScope"] and not aggressive_scope_ack:
        reason = "aggressive_scope_requires_ack"
    elif delta >= 0:
        reason = "accepted_rate_held"
    elif -delta > pol["maxAcceptedRateDropAbs"]:
        reason = "accepted_rate_dropped_beyond_bound"
    elif improv is not None and improv >= pol["minCostPerAcceptedImprovementFrac"]:
        reason = "cost_per_accepted_improved_offsets_drop"
    else:
        reason = "accepted_rate_dropped_without_cost_win"
    return {"schemaVersion": GATE_SCHEMA, "passed": reason in ("accepted_rate_held", "cost_per_accepted_improved_offsets_drop"), "reason": reason,
            "detail": _DETAIL[reason], "sampleCount": n, "originalAcceptedRate": o_rate, "quantizedAcceptedRate": q_rate, "acceptedRateDeltaAbs": delta,
            "originalCostPerAcceptedMsat": o_cpa, "quantizedCostPerAcceptedMsat": q_cpa, "costPerAcceptedImprovementFrac": improv,
            "aggressiveScope": aggressive, "decisionGrade": dg, "realSweepEvidenceRef": real_sweep_evidence.get("evidenceRef") if dg else None,
            "decisionGradeBlockers": blockers}


def compare_backends(original, quantized, tokenizer, items: list[dict], max_new_tokens: int = 32, original_msat_per_token: float = 2.0,
                     quantized_msat_per_token: float = 1.0, stop_ids=()) -> list[dict]:
    """Gate samples from two serving backends of this package: every ``{"prompt", "answer"}`` item is answered greedily by both;
    verified = the answer matches; cost = (prompt + generated tokens) x the lane's price per token."""
    from ..eval.scorers import exact_match
    a = exact_match(original, items, tokenizer, max_new_tokens=max_new_tokens, stop_ids=stop_ids)
    b = exact_match(quantized, items, tokenizer, max_new_tokens=max_new_tokens, stop_ids=stop_ids)
    out = []
    for i, (it, ra, rb) in enumerate(zip(items, a["rows"], b["rows"])):
        p = len(tokenizer.encode(it["prompt"]))
        out.append({"taskId": it.get("id", f"task.{i}"), "originalVerified": ra["match"], "quantizedVerified": rb["match"],
                    "originalCostBasisMsat": (p + len(tokenizer.encode(ra["generated"]))) * original_msat_per_token,
                    "quantizedCostBasisMsat": (p + len(tokenizer.encode(rb["generated"]))) * quantized_msat_per_token})
    return out
