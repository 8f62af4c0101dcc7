"""Served-model metadata: quantization disclosure and speculation telemetry / policy.

Every field holds a measured value or the ``not_measured`` sentinel; nothing is guessed.

Quantization (inference/khala-quantization.ts:48 precision modes, :93 scopes, :124 backends,
descriptor and alias qualification in the same file): precision is a disclosed property of a
served model; ``unquantized`` and ``not_measured`` never count as quantized and never carry a
passed eval gate; KV-cache and attention scopes are the aggressive ones.

Speculation (inference/khala-speculation.ts:90 modes, :103 draft-free test, :385 policy):
n-gram and lookahead are draft-free; EAGLE is a learned mode that is not available; the policy
turns speculation off above a profitable batch size or compute pressure, and off when either
signal is unknown.
"""
from __future__ import annotations

import math

NOT_MEASURED = "not_measured"

PRECISION_MODES = ("unquantized", "fp8", "mxfp8", "nvfp4", "int8", "int4", "awq", "gptq", NOT_MEASURED)
QUANT_SCOPES = ("none", "weights_only", "weights_and_activations", "kv_cache", "attention", NOT_MEASURED)
QUANT_BACKENDS = ("provider-native", "vllm", "sglang", "tensorrt-llm", NOT_MEASURED)
QUANT_SCHEMA = "openagents.khala.quantization.v1"
SERVED_MODEL_SCHEMA = "openagents.khala.served-model.v1"


def is_quantized_precision(mode: str) -> bool:
    if mode not in PRECISION_MODES:
        raise ValueError(f"unknown precision mode {mode!r}")
    return mode not in ("unquantized", NOT_MEASURED)


def is_aggressive_scope(scope: str) -> bool:
    return scope in ("kv_cache", "attention")


def quantization_metadata(precision: str | None = None, backend: str | None = None, backend_version: str | None = None,
                          scope: str | None = None, eval_gate_passed: bool | None = None, eval_gate_ref: str | None = None) -> dict:
    precision = precision or NOT_MEASURED
    if precision not in PRECISION_MODES:
        raise ValueError(f"unknown precision mode {precision!r}")
    backend = backend or NOT_MEASURED
    if backend not in QUANT_BACKENDS:
        raise ValueError(f"unknown backend {backend!r}")
    if scope is not None and scope not in QUANT_SCOPES:
        raise ValueError(f"unknown scope {scope!r}")
    return {
        "schemaVersion": QUANT_SCHEMA,
        "precision": precision,
        "backend": backend,
        "backendVersion": backend_version if backend_version and backend_version.strip() else NOT_MEASURED,
        "scope": "none" if precision == "unquantized" else (scope if scope is not None else NOT_MEASURED),
        "evalGatePassed": bool(eval_gate_passed) if is_quantized_precision(precision) else False,
        "evalGateRef": eval_gate_ref,
    }


UNQUANTIZED = quantization_metadata("unquantized")
UNKNOWN_QUANTIZATION = quantization_metadata()


def alias_qualification(public_alias: str) -> str:
    """An alias is qualified when its last dash-separated part names a reduced precision."""
    tail = public_alias.lower().rsplit("-", 1)[-1]
    return "qualified" if tail in ("fp8", "mxfp8", "nvfp4", "int8", "int4", "awq", "gptq") else "unqualified"


def served_model_descriptor(public_alias: str, served_model_id: str, **quant) -> dict:
    return {"schemaVersion": SERVED_MODEL_SCHEMA, "publicAlias": public_alias, "servedModelId": served_model_id,
            "aliasQualification": alias_qualification(public_alias), "quantization": quantization_metadata(**quant)}


def engine_quantization(plan_name: str, kv_dtype: str = "fp16", version: str = "b200-serve") -> dict:
    """Disclosure for this engine's own weight plans: block-quantized GGUF weights are int8 / int4
    weights-only; a quantized KV cache would raise the scope to ``kv_cache``."""
    precision = {"Q8_0": "int8", "Q4_K": "int4", "MXFP4": "nvfp4", "BF16": "unquantized", "F32": "unquantized"}.get(plan_name, NOT_MEASURED)
    scope = "kv_cache" if kv_dtype not in ("fp16", "bf16", "fp32") else "weights_only"
    return quantization_metadata(precision, "provider-native", version, scope)


# ---------------------------------------------------------------- speculation
SPECULATION_MODES = ("none", "n_gram", "lookahead", "eagle", NOT_MEASURED)
SPEC_SCHEMA = "openagents.khala.speculation.v1"
SPEC_DECISION_SCHEMA = "openagents.khala.speculation-decision.v1"
DEFAULT_SPECULATION_POLICY = {"maxProfitableBatchSize": 4, "maxProfitableComputePressure": 0.6}


def is_draft_free_mode(mode: str) -> bool:
    return mode in ("n_gram", "lookahead")


def is_learned_mode(mode: str) -> bool:
    return mode == "eagle"


def _count(v):
    return v if isinstance(v, (int, float)) and not isinstance(v, bool) and math.isfinite(v) and v >= 0 else None


def _spec(mode, active, rate, proposed, accepted):
    return {"schemaVersion": SPEC_SCHEMA, "mode": mode, "active": active, "acceptanceRate": rate,
            "draftTokensProposed": proposed, "draftTokensAccepted": accepted}


NO_SPECULATION = _spec("none", False, NOT_MEASURED, NOT_MEASURED, NOT_MEASURED)
UNKNOWN_SPECULATION = _spec(NOT_MEASURED, False, NOT_MEASURED, NOT_MEASURED, NOT_MEASURED)


def speculation_metadata(mode: str | None = None, active: bool | None = None, proposed=None, accepted=None) -> dict:
    mode = mode or NOT_MEASURED
    if mode not in SPECULATION_MODES:
        raise ValueError(f"unknown speculation mode {mode!r}")
    if mode == "none":
        return dict(NO_SPECULATION)
    if mode == NOT_MEASURED:
        return dict(UNKNOWN_SPECULATION)
    p, a = _count(proposed), _count(accepted)
    rate = min(a, p) / p if p and a is not None else NOT_MEASURED
    if p is not None and a is not None:
        a = min(a, p)
    return _spec(mode, True if active is None else active, rate, NOT_MEASURED if p is None else p, NOT_MEASURED if a is None else a)


def decide_speculation(requested_mode: str, batch_size, compute_pressure, policy: dict | None = None) -> dict:
    policy = policy or DEFAULT_SPECULATION_POLICY

    def off(reason):
        return {"schemaVersion": SPEC_DECISION_SCHEMA, "enabled": False, "selectedMode": "none", "reason": reason}

    if requested_mode in ("none", NOT_MEASURED):
        return off("disabled_not_requested")
    if not is_draft_free_mode(requested_mode):
        return off("disabled_mode_unavailable")
    if batch_size == NOT_MEASURED or compute_pressure == NOT_MEASURED:
        return off("disabled_pressure_unknown")
    if batch_size > policy["maxProfitableBatchSize"]:
        return off("disabled_high_batch")
    if compute_pressure > policy["maxProfitableComputePressure"]:
        return off("disabled_high_pressure")
    return {"schemaVersion": SPEC_DECISION_SCHEMA, "enabled": True, "selectedMode": requested_mode, "reason": "enabled_low_batch"}


_EVIDENCE_TEXT_FIELDS = (("evidenceRef", "evidence_ref_missing"), ("ownerApprovalRef", "owner_approval_ref_missing"),
                         ("model", "model_context_missing"), ("route", "route_context_missing"),
                         ("engineRef", "engine_ref_missing"), ("acceptanceEvidenceRef", "acceptance_evidence_ref_missing"),
                         ("latencyEvidenceRef", "latency_evidence_ref_missing"))


def preflight_real_speculation_lane(owner_confirmed: bool, evidence: dict | None, policy: dict | None = None) -> dict:
    """Go/no-go for turning a real speculation lane on: every piece of evidence present and the
    policy enabled at the measured pressure (inference/khala-speculation.ts preflight)."""
    blockers = [] if owner_confirmed else ["owner_confirmation_missing"]
    if evidence is None:
        blockers.append("real_speculation_evidence_missing")
        decision = decide_speculation("n_gram", NOT_MEASURED, NOT_MEASURED, policy)
    else:
        text = lambda k: isinstance(evidence.get(k), str) and evidence[k].strip() != ""
        for k, b in _EVIDENCE_TEXT_FIELDS:
            if not text(k):
                blockers.append(b)
        if not (text("workloadRef") and text("workload")):
            blockers.append("workload_context_missing")
        t = evidence.get("temperature")
        if not (isinstance(t, (int, float)) and math.isfinite(t)):
            blockers.append("temperature_not_measured")
        if not is_draft_free_mode(evidence.get("mode", "")):
            blockers.append("mode_not_real_speculation")
        p, a = _count(evidence.get("draftTokensProposed")), _count(evidence.get("draftTokensAccepted"))
        if p is None or a is None or p <= 0:
            blockers.append("draft_counts_not_measured")
        elif a > p:
            blockers.append("accepted_exceeds_proposed")
        refs = evidence.get("publicSafeEvidenceRefs") or []
        if not refs or any(not (isinstance(r, str) and r.strip()) for r in refs):
            blockers.append("public_safe_evidence_refs_missing")
        sig = evidence.get("signal", {})
        decision = decide_speculation(evidence.get("mode", NOT_MEASURED), sig.get("batchSize", NOT_MEASURED),
                                      sig.get("computePressure", NOT_MEASURED), policy)
    if not decision["enabled"]:
        blockers.append("policy_disabled")
    eligible = not blockers and evidence is not None
    if eligible:
        meta = speculation_metadata(evidence["mode"], True, evidence["draftTokensProposed"], evidence["draftTokensAccepted"])
    elif decision["reason"] in ("disabled_high_batch", "disabled_high_pressure"):
        meta = dict(NO_SPECULATION)
    else:
        meta = dict(UNKNOWN_SPECULATION)
    return {"schemaVersion": "openagents.khala.real-speculation-preflight.v1", "eligible": eligible, "decision": decision,
            "metadata": meta, "blockers": blockers, "evidenceRef": evidence["evidenceRef"] if eligible else None,
            "publicSafeEvidenceRefs": list(evidence["publicSafeEvidenceRefs"]) if eligible else []}
