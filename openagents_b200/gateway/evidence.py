"""Evidence-only records for engine outputs, the quantized-model pilot gate, and the replica pool.

* Evidence contract - what the training/serving stack hands upward is evidence, never authority: a
  record may describe a training run, an eval, an optimizer run, a scorecard, a candidate module, a
  promotion proposal or a rollback, and carries five flags that forbid it from settling, promoting,
  paying, upgrading a public claim or changing routing.  Projections strip refs an audience may not see
  and refuse anything that looks like raw data, credentials or raw timestamps.
  (psionic-evidence-contract.ts:10-18 kinds, :40-49 and :117-125 authority, :250-365 projection.)
* Pilot gate - go/no-go for routing a lane to a newly quantized model: pure validation of owner
  approval, boot evidence, measured context length, a tool-calling loop, quality parity and measured
  tokens/s; it runs nothing itself.  (inference/glm-nvfp4-pilot.ts:6-20 model, baseline and launch
  flags, :77-84 serving-stack failure codes, and the result builder.)
* Replica pool - choose among replicas of one model by health, warmth, queue depth, in-flight count
  and observed latency, with a saturation policy (overflow at once, queue then overflow, queue then
  429).  (inference/hydralisk-adapter.ts:44-53 replica config, :64-79 routing state, :107-117 pool.)
"""
from __future__ import annotations

import math
import re

from .fabric import InferenceAdapterError

# ---------------------------------------------------------------- evidence contract
EVIDENCE_KINDS = ("candidate_module", "eval_run", "optimizer_run", "promotion_proposal", "rollback", "scorecard", "training_run")
EVIDENCE_STATUSES = ("archived", "completed", "draft", "failed", "needs_review", "retained_failure", "running")
EVIDENCE_ONLY_AUTHORITY = {"authorityBoundary": "evidence_only", "noAcceptedOutcomeSettlement": True, "noDirectModulePromotion": True,
                           "noPayoutMutation": True, "noPublicClaimUpgrade": True, "noRoutingMutation": True}
REF_FIELDS = ("candidateModuleRefs", "datasetRefs", "evidenceReceiptRefs", "failureRefs", "fixtureRefs", "metricRefs", "modelRefs",
              "optimizerRefs", "promotionProposalRefs", "providerRefs", "retainedFailureRefs", "reviewRefs", "rollbackRefs", "scorecardRefs",
              "sourceRefs", "trainingRunRefs")
_SAFE_REF = re.compile(r"^[A-Za-z0-9][A-Za-z0-9_.:/-]{0,260}$")
_UNSAFE = re.compile(r"(@|access[_-]?token|auth\.json|bearer|cookie|customer[_-]?(email|name|value)|dataset\.raw|mnemonic|password|"
                     r"private[_-]?key|secret|wallet)", re.I)
_RAW_TS = re.compile(r"\d{4}-\d{2}-\d{2}T\d{2}:\d{2}:\d{2}")
_AUDIENCE_HIDDEN = {
    "public": re.compile(r"(dataset\.private|failure\.operator|metric\.operator|provider\.private|review\.operator|source\.private)", re.I),
    "team": re.compile(r"(dataset\.private|provider\.private|source\.private)", re.I),
}
_AUDIENCE_HIDDEN["agent"] = _AUDIENCE_HIDDEN["customer"] = _AUDIENCE_HIDDEN["public"]


class EvidenceUnsafe(Exception):
    pass


def evidence_record(id: str, kind: str, status: str, created_at_iso: str, updated_at_iso: str | None = None, authority: dict | None = None, **refs) -> dict:
    if kind not in EVIDENCE_KINDS or status not in EVIDENCE_STATUSES:
        raise ValueError("unknown evidence kind or status")
    unknown = set(refs) - set(REF_FIELDS)
    if unknown:
        raise ValueError(f"unknown ref fields {sorted(unknown)}")
    rec = {"id": id, "evidenceKind": kind, "status": status, "createdAtIso": created_at_iso, "updatedAtIso": updated_at_iso or created_at_iso,
           "authority": dict(authority or EVIDENCE_ONLY_AUTHORITY)}
    rec.update({f: list(refs.get(f, ())) for f in REF_FIELDS})
    return rec


def authority_is_evidence_only(a: dict) -> bool:
    return a.get("authorityBoundary") == "evidence_only" and all(a.get(k) is True for k in EVIDENCE_ONLY_AUTHORITY if k != "authorityBoundary")


def evidence_needs_review(rec: dict) -> bool:
    return rec["status"] == "needs_review" or bool(rec["promotionProposalRefs"] or rec["rollbackRefs"] or rec["candidateModuleRefs"])


def _assert_safe(label, refs):
    for r in {x.strip() for x in refs if x.strip()}:
        if not _SAFE_REF.match(r) or _UNSAFE.search(r) or _RAW_TS.search(r):
            raise EvidenceUnsafe(f"{label} contains raw data, credentials, payment material or raw timestamps")


def _friendly_age(iso: str, now_iso: str) -> str:
    from datetime import datetime
    p = lambda s: datetime.fromisoformat(s.replace("Z", "+00:00"))
    sec = max(0, int((p(now_iso) - p(iso)).total_seconds()))
    for unit, n in (("day", 86400), ("hour", 3600), ("minute", 60)):
        if sec >= n:
            k = sec // n
            return f"{k} {unit}{'s' if k != 1 else ''} ago"
    return "just now"


def project_evidence(rec: dict, audience: str, now_iso: str) -> dict:
    """Audience-scoped view: refs the audience may not see are dropped, times become relative, and the three
    mutation permissions are derived from the authority flags (all false for evidence-only records)."""
    _assert_safe("evidence refs", [rec["id"]] + [r for f in REF_FIELDS for r in rec[f]])
    hidden = _AUDIENCE_HIDDEN.get(audience)
    keep = lambda refs: sorted({r.strip() for r in refs if r.strip() and not (hidden and hidden.search(r))})
    out = {f: keep(rec[f]) for f in REF_FIELDS}
    out.update({"audience": audience, "authority": rec["authority"], "evidenceKind": rec["evidenceKind"], "status": rec["status"],
                "id": (keep([rec["id"]]) or ["evidence_id.redacted"])[0], "evidenceOnly": authority_is_evidence_only(rec["authority"]),
                "promotionAllowed": not rec["authority"]["noDirectModulePromotion"], "routingMutationAllowed": not rec["authority"]["noRoutingMutation"],
                "settlementAllowed": not rec["authority"]["noAcceptedOutcomeSettlement"],
                "createdAtDisplay": _friendly_age(rec["createdAtIso"], now_iso), "updatedAtDisplay": _friendly_age(rec["updatedAtIso"], now_iso)})
    if _UNSAFE.search(repr(out)) or _RAW_TS.search(repr(out)):
        raise EvidenceUnsafe("evidence projection contains unsafe material")
    return out


def training_run_evidence(run_ref: str, receipts: list[str], metrics: list[str], created_at_iso: str, failed: bool = False) -> dict:
    """What ``b200-train`` publishes about a finished run."""
    return evidence_record(f"psionic_evidence.{run_ref}", "training_run", "failed" if failed else "completed", created_at_iso,
                           trainingRunRefs=[run_ref], evidenceReceiptRefs=receipts, metricRefs=metrics)


# ---------------------------------------------------------------- pilot gate
PILOT_SCHEMA = "openagents.khala.quantized_model_pilot_result.v1"
GLM_NVFP4_MODEL = "nvidia/GLM-5.2-NVFP4"
GLM_NVFP4_BASELINE_TPS = 47
MIN_TOOL_LOOP_SAMPLES = 20
GLM_NVFP4_VLLM_FLAGS = (("--tensor-parallel-size", "8"), ("--quantization", "modelopt_fp4"), ("--tool-call-parser", "glm47"),
                        ("--reasoning-parser", "glm45"), ("--trust-remote-code", None), ("--chunked-prefill-size", "131072"),
                        ("--mem-fraction-static", "0.80"))
SERVING_STACK_FAILURE_CODES = ("vllm_sparse_mla_backend_unavailable", "sglang_moe_w13_shape_mismatch", "sglang_trtllm_sm120_unsupported",
                               "sglang_flashmla_sparse_sm120_unsupported", "sglang_tilelang_sm120_compile_failure", "unknown")
_PILOT_REF_FIELDS = ("ownerApprovalRef", "endpointRef", "decisionRef", "bootLoadEvidenceRef", "measuredMaxModelLenEvidenceRef",
                     "qualityEvidenceRef")
_UNSAFE_FIELD_BLOCKER = {"ownerApprovalRef": "owner_approval_ref_unsafe", "endpointRef": "endpoint_ref_unsafe", "decisionRef": "decision_ref_unsafe",
                         "bootLoadEvidenceRef": "boot_load_evidence_ref_unsafe", "measuredMaxModelLenEvidenceRef": "measured_max_model_len_evidence_ref_unsafe",
                         "qualityEvidenceRef": "quality_evidence_ref_unsafe", "toolLoopEvidenceRef": "tool_loop_evidence_ref_unsafe",
                         "throughputEvidenceRef": "tps_evidence_ref_unsafe"}
_MISSING_FIELD_BLOCKER = {"ownerApprovalRef": "owner_approval_ref_missing", "endpointRef": "endpoint_ref_missing", "decisionRef": "decision_ref_missing",
                          "bootLoadEvidenceRef": "boot_load_evidence_ref_missing",
                          "measuredMaxModelLenEvidenceRef": "measured_max_model_len_evidence_ref_missing", "qualityEvidenceRef": "quality_evidence_ref_missing",
                          "toolLoopEvidenceRef": "tool_loop_evidence_missing"}


def _audit(field, raw):
    if raw is None or not str(raw).strip():
        return {"field": field, "status": "missing", "publicRef": None}
    r = str(raw).strip()
    ok = bool(_SAFE_REF.match(r)) and not _UNSAFE.search(r) and "://" not in r
    return {"field": field, "status": "accepted" if ok else "rejected_unsafe", "publicRef": r if ok else None}


def pilot_result(config: dict, tool_loop: dict | None = None, throughput: dict | None = None, model: str = GLM_NVFP4_MODEL,
                 baseline_tps: float = GLM_NVFP4_BASELINE_TPS, required_tool_loop_samples: int = MIN_TOOL_LOOP_SAMPLES) -> dict:
    """config: ownerArmed, the ref fields, endpointUrl, model, bootLoadStatus, measuredMaxModelLen, qualityParity,
    servingStackFindings.  tool_loop: sampleCount, providerErrorCount, toolCallsAttempted, toolCallsSucceeded,
    hallucinatedToolCallCount, evidenceRef.  throughput: measuredTps, outputTokens, evidenceRef."""
    tl = tool_loop or {"sampleCount": 0, "providerErrorCount": 0, "toolCallsAttempted": 0, "toolCallsSucceeded": 0, "hallucinatedToolCallCount": 0, "evidenceRef": None}
    tp = throughput or {"measuredTps": None, "outputTokens": 0, "evidenceRef": None}
    audits = [_audit(f, config.get(f)) for f in _PILOT_REF_FIELDS] + [_audit("toolLoopEvidenceRef", tl.get("evidenceRef")),
                                                                        _audit("throughputEvidenceRef", tp.get("evidenceRef"))]
    ref = {a["field"]: a["publicRef"] for a in audits}
    b = set()
    if config.get("ownerArmed") is not True:
        b.add("owner_arm_missing")
    for a in audits:
        if a["status"] == "rejected_unsafe":
            b.update(("unsafe_public_ref", _UNSAFE_FIELD_BLOCKER[a["field"]]))
        elif a["status"] == "missing" and a["field"] in _MISSING_FIELD_BLOCKER:
            b.add(_MISSING_FIELD_BLOCKER[a["field"]])
    if not (config.get("endpointUrl") or "").strip():
        b.add("endpoint_url_missing")
    if config.get("model", model) != model:
        b.add("model_mismatch")
    findings = config.get("servingStackFindings", [])
    failed_before = any(f.get("status") == "failed_before_endpoint" for f in findings)
    boot = ("failed" if config.get("bootLoadStatus") == "failed" or failed_before else
            "passed" if config.get("bootLoadStatus") == "passed" or (config.get("bootLoadStatus") != "not_attempted" and ref["bootLoadEvidenceRef"]) else "not_attempted")
    if boot == "failed":
        b.add("boot_load_failed")
    mlen = config.get("measuredMaxModelLen")
    mlen = mlen if isinstance(mlen, int) and mlen > 0 else None
    if mlen is None:
        b.add("measured_max_model_len_missing")
    if tl["sampleCount"] < required_tool_loop_samples:
        b.add("tool_loop_sample_count_too_low")
    if tl["providerErrorCount"] > 0:
        b.add("tool_loop_provider_error")
    if tl["toolCallsAttempted"] < required_tool_loop_samples or tl["toolCallsSucceeded"] < required_tool_loop_samples or tl["hallucinatedToolCallCount"] > 0:
        b.add("tool_loop_missing_tool_calls")
    if config.get("qualityParity", "not_measured") != "passed":
        b.add("quality_parity_missing")
    tps = tp.get("measuredTps")
    if tps is None or tp.get("outputTokens", 0) <= 0:
        b.add("tps_measurement_missing")
    elif not (isinstance(tps, (int, float)) and math.isfinite(tps) and tps >= 0):
        b.add("tps_not_finite")
    go = not b
    flags = [{"name": n, **({"value": v} if v is not None else {})} for n, v in GLM_NVFP4_VLLM_FLAGS]
    if mlen is not None:
        flags.append({"name": "--max-model-len", "value": str(mlen)})
    return {"schemaVersion": PILOT_SCHEMA, "publicSafe": True, "ownerArmed": config.get("ownerArmed") is True, "decision": "go" if go else "no_go",
            "canRouteCodingLane": go, "model": model, "bootLoadStatus": boot, "measuredMaxModelLen": mlen,
            "qualityParity": config.get("qualityParity", "not_measured"), "evidenceRefAudit": audits, "blockerRefs": sorted(b),
            "toolLoop": {**tl, "evidenceRef": ref["toolLoopEvidenceRef"]},
            "throughput": {**tp, "evidenceRef": ref["throughputEvidenceRef"], "baselineTps": baseline_tps,
                           "speedupVsBaseline": tps / baseline_tps if isinstance(tps, (int, float)) and math.isfinite(tps) and baseline_tps > 0 else None},
            "launchFlags": flags, "routingOutcome": "route_coding_tools_to_full_model_then_overflow" if go else "keep_live_lane"}


# ---------------------------------------------------------------- replica pool
SATURATION_POLICIES = ("overflow_immediately", "queue_then_overflow", "queue_then_429")
DEFAULT_QUEUE_WAIT_MS, MAX_QUEUE_WAIT_MS = 250, 1000
_HEALTH_SCORE = {"healthy": 2, "degraded": 1, "unhealthy": 0}
_WARM_RANK = {"warm": 2, "unknown": 1, "cold": 0}


def replica_state(replica_id: str, health="healthy", warm_state="unknown", inflight=0, max_inflight=1, queue_depth=0, observed_ttft_ms=None,
                  observed_tps=None, warm_at_ms=None, benchmark_reserved=False, draining=False, region=None) -> dict:
    return {"replicaId": replica_id, "health": health, "warmState": warm_state, "inflightCount": inflight, "maxInflight": max_inflight,
            "queueDepth": queue_depth, "observedTtftMs": observed_ttft_ms, "observedTps": observed_tps, "warmAtEpochMs": warm_at_ms,
            "benchmarkReserved": benchmark_reserved, "draining": draining, "region": region}


def busy_reason(s: dict) -> str | None:
    if s["benchmarkReserved"]:
        return "benchmark_reserved"
    if s["draining"]:
        return "draining"
    if s["health"] == "unhealthy":
        return "health_unhealthy"
    if s["inflightCount"] >= s["maxInflight"]:
        return "inflight_full"
    return None


def _rank_key(item):
    i, s = item
    return (-_HEALTH_SCORE[s["health"]], -_WARM_RANK[s["warmState"]], -(s["warmAtEpochMs"] if s["warmAtEpochMs"] is not None else -1),
            s["queueDepth"], s["inflightCount"], s["observedTtftMs"] if s["observedTtftMs"] is not None else math.inf,
            -(s["observedTps"] if s["observedTps"] is not None else -1), i)


def select_replica(states: list[dict], affinity_replica_id: str | None = None) -> dict:
    """Eligible replicas (not reserved, not draining, not unhealthy, with a free slot) ranked by health, warmth,
    most recently warmed, shortest queue, fewest in flight, lowest TTFT, highest tokens/s, then order.  A
    cache-affinity hint wins when that replica is eligible."""
    eligible = [(i, s) for i, s in enumerate(states) if busy_reason(s) is None]
    if not eligible:
        reasons = sorted({busy_reason(s) for s in states}) or ["no_replicas"]
        return {"replicaId": None, "busyReasons": reasons, "fallbackReason": "pool_saturated"}
    if affinity_replica_id is not None:
        for i, s in eligible:
            if s["replicaId"] == affinity_replica_id:
                return {"replicaId": s["replicaId"], "busyReasons": [], "fallbackReason": None, "affinityHit": True}
    i, s = min(eligible, key=_rank_key)
    return {"replicaId": s["replicaId"], "busyReasons": [], "affinityHit": False,
            "fallbackReason": "affinity_replica_busy" if affinity_replica_id is not None else None}


def default_saturation_policy(stream: bool) -> str:
    return "overflow_immediately" if stream else "queue_then_overflow"


def dispatch_to_pool(states_fn, run, policy: str = "queue_then_overflow", max_queue_wait_ms: float = DEFAULT_QUEUE_WAIT_MS, sleep=None,
                     affinity_replica_id: str | None = None, adapter_id: str = "hydralisk-vllm"):
    """``states_fn()`` returns the current replica states; ``run(replica_id)`` performs the request.  On a
    saturated pool the policy decides: fail retryably at once (the router overflows to the next lane), wait
    once (bounded) and retry, or wait and then answer 429 (not retryable: the caller should back off)."""
    if policy not in SATURATION_POLICIES:
        raise ValueError(f"unknown saturation policy {policy!r}")
    wait = min(max(0.0, max_queue_wait_ms), MAX_QUEUE_WAIT_MS)
    sel = select_replica(states_fn(), affinity_replica_id)
    waited = 0.0
    if sel["replicaId"] is None and policy != "overflow_immediately" and wait > 0:
        (sleep or (lambda ms: None))(wait)
        waited = wait
        sel = select_replica(states_fn(), affinity_replica_id)
    if sel["replicaId"] is None:
        final = policy == "queue_then_429"
        raise InferenceAdapterError(adapter_id, "glm_pool_saturated", f"pool saturated ({','.join(sel['busyReasons'])})", not final, 429 if final else 503)
    return run(sel["replicaId"]), {"replicaId": sel["replicaId"], "queueWaitMs": waited, "saturationPolicy": policy,
                                   "replicaFallbackReason": sel.get("fallbackReason"), "affinityHit": sel.get("affinityHit", False)}


def route_admission(states: list[dict], reserved_external_slots: int = 1) -> dict:
    """Internal stress traffic is admitted only while the external reserve stays free."""
    free = sum(max(0, s["maxInflight"] - s["inflightCount"]) for s in states if busy_reason(s) is None)
    return {"reservedExternalHeadroomAvailable": free >= 1, "internalStressHeadroomAvailable": free > reserved_external_slots,
            "reason": "headroom_available" if free > reserved_external_slots else "external_reserve_only" if free >= 1 else "pool_saturated"}
