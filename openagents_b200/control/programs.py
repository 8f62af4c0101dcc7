"""Training-program governance around the run/window authority: the model ladder, the device-capability
dataset, the gradient-window promotion gate and kernel-optimization campaigns.  All of it is pure
decision logic over receipts and digests; nothing here moves tensors.

Reference: apps/openagents.com/workers/api/src/training-model-ladder-rungs.ts:137-197 (rungs R0..R4, only
R0 closed); training-device-capability.ts:24-29 (measurements), :42-45 (host probes), :49 (thermal ratio
floor 0.8) and the same-class replication scopes; tassadar-gradient-window-regime.ts:3-11 (stage ladder),
:15-39 (candidate), and its projection (a window is promoted only with quarantine, an equal-digest
recompute, two equal replicas, a perfect canary and a promotion decision, and never when the update
touches the compiled core); kernel-optimization-campaign.ts:264-309 (fan-out, unique targets and slugs)
with packages/tassadar-executor/src/kernel-optimization-parity.ts (the per-job verdict: same target, same
op, a new kernel, parity traces bound to the same graph and validator, equal output digests, and a
strictly higher tok/s).
"""
from __future__ import annotations

import math
import re
import statistics

# ---------------------------------------------------------------- model ladder
R1_BLOCKER = "blocker.product_promises.r1_full_rehearsal_missing"
NETWORK_RUNG_BLOCKER = "blocker.product_promises.model_ladder_network_rungs_not_run"
LADDER = (
    {"rung": "R0", "modelClass": "tri-host bringup", "tokenScale": "approximately 4k tokens", "networkRung": False,
     "hardwareReality": "2 Macs plus 1 RTX 4080."},
    {"rung": "R1", "modelClass": "approximately 30-50M", "tokenScale": "1-5B tokens", "networkRung": False,
     "hardwareReality": "operator-owned devices over days."},
    {"rung": "R2", "modelClass": "approximately 125-200M", "tokenScale": "10-50B tokens", "networkRung": True,
     "hardwareReality": "operator plus early contributor nodes."},
    {"rung": "R3", "modelClass": "approximately 1B", "tokenScale": "100B+ tokens", "networkRung": True,
     "hardwareReality": "conditioned on R2 measured economics."},
    {"rung": "R4", "modelClass": "approximately 3B class", "tokenScale": "1T+ tokens", "networkRung": True,
     "hardwareReality": "only if R3 economics close."},
)
R1_CLOSEOUT_CRITERIA = ("data", "ablations", "marathon", "post_training", "evals", "economics_gate")
_UNSAFE_PUBLIC = re.compile(r"(deviceId|deviceRef|nodeId|nodeRef|ownerId|ownerRef|wallet|mnemonic|preimage|invoice|bolt11|bolt12|lno1|secret)", re.I)


class UnsafePublicMaterial(Exception):
    pass


def project_model_ladder(closeout_receipts: dict[str, list[str]] | None = None, r1_criteria_receipts: dict[str, str] | None = None) -> dict:
    """``closeout_receipts``: rung -> closeout receipt refs.  A rung is closed only with a receipt and with
    every lower rung closed; R1 additionally needs a receipt for each of its six closeout criteria."""
    closeout = closeout_receipts or {"R0": ["receipt.r0.bringup"]}
    crit = r1_criteria_receipts or {}
    if _UNSAFE_PUBLIC.search(repr(closeout)) or _UNSAFE_PUBLIC.search(repr(crit)):
        raise UnsafePublicMaterial("ladder receipts contain material that is not public-safe")
    rungs, closed_so_far, highest = [], True, None
    for r in LADDER:
        has = bool(closeout.get(r["rung"]))
        if r["rung"] == "R1":
            has = has and all(crit.get(c) for c in R1_CLOSEOUT_CRITERIA)
        closed = closed_so_far and has
        closed_so_far = closed
        if closed:
            highest = r["rung"]
        blockers = [] if closed else ([R1_BLOCKER] if r["rung"] == "R1" else [NETWORK_RUNG_BLOCKER] if r["rung"] == "R2" else [])
        rungs.append({**r, "status": "retained_rehearsal" if closed else "not_run", "closeoutReceiptAvailable": closed, "blockerRefs": blockers})
    names = [r["rung"] for r in LADDER]
    nxt = names[names.index(highest) + 1] if highest in names[:-1] else (names[0] if highest is None else None)
    return {"schemaVersion": "openagents.training.model_ladder.rungs.v1", "rungs": rungs,
            "r1CloseoutCriteria": [{"criterionId": c, "receiptAvailable": bool(crit.get(c)), "status": "receipt_available" if crit.get(c) else "missing_receipt"}
                                   for c in R1_CLOSEOUT_CRITERIA],
            "rungSummary": {"rungCount": len(LADDER), "closedRungCount": sum(r["closeoutReceiptAvailable"] for r in rungs),
                            "highestClosedRung": highest, "nextRequiredRung": nxt},
            "gate": {"greenGateSatisfied": highest not in (None, "R0"), "remainingBlockerRefs": sorted({b for r in rungs for b in r["blockerRefs"]})}}


# ---------------------------------------------------------------- device-capability dataset
BENCHMARK_MEASUREMENTS = ("attention_throughput", "memory_bandwidth", "tokens_per_second", "step_time_ms")
HOST_PROBE_MEASUREMENTS = ("host_ram_headroom_gb", "sustained_vs_burst_throughput_ratio")
THERMAL_RATIO_FLOOR = 0.8
THERMAL_METRIC = "sustained_vs_burst_throughput_ratio"
MIN_SAME_CLASS_SAMPLES = 2


def nearest_rank(values, q: float) -> float:
    s = sorted(values)
    return s[max(0, min(len(s) - 1, math.ceil(q * len(s)) - 1))]


def thermal_throttle_status(ratio, verified: bool) -> str:
    if ratio is None:
        return "missing"
    if not verified:
        return "needs_verified_thermal_probe"
    return "thermal_throttle_not_observed" if ratio >= THERMAL_RATIO_FLOOR else "thermal_throttle_observed"


def same_class_replication_status(scopes: list[str]) -> str:
    if not scopes:
        return "missing"
    if "cross_machine_same_class" in scopes:
        return "cross_machine_replicated"
    if "cross_process_same_host" in scopes:
        return "same_host_only"
    if all(s == "single_observation" for s in scopes):
        return "single_observation"
    return "unknown_scope"


def device_capability_distributions(samples: list[dict]) -> list[dict]:
    """``samples``: {deviceClassRef, machineRef, metric, value, unit, verified (bool), settled (bool), receiptRef}.
    One distribution per (device class, metric): nearest-rank p50/p90, whether enough same-class samples
    from different machines agree to count as cross-checked, and whether the numbers are settled."""
    groups: dict[tuple, list[dict]] = {}
    for s in samples:
        if s["metric"] not in BENCHMARK_MEASUREMENTS + HOST_PROBE_MEASUREMENTS:
            raise ValueError(f"unknown measurement {s['metric']!r}")
        if not (isinstance(s["value"], (int, float)) and math.isfinite(s["value"]) and s["value"] >= 0):
            raise ValueError("measurement values must be finite and non-negative")
        groups.setdefault((s["deviceClassRef"], s["metric"]), []).append(s)
    out = []
    for (cls, metric), g in sorted(groups.items()):
        vals = [s["value"] for s in g]
        machines = {s["machineRef"] for s in g}
        verified = all(s.get("verified") for s in g)
        if len(g) < MIN_SAME_CLASS_SAMPLES:
            state = "insufficient_same_class_samples"
        elif not verified:
            state = "measured_unverified"
        elif len(machines) < 2:
            state = "needs_replication"
        else:
            state = "cross_checked"
        med = statistics.median(vals)
        out.append({"deviceClassRef": cls, "metric": metric, "unit": g[0].get("unit", ""), "sampleCount": len(g), "min": min(vals), "max": max(vals),
                    "p50": nearest_rank(vals, 0.5), "p90": nearest_rank(vals, 0.9), "crossCheckState": state,
                    "agreement": (min(vals) / max(vals) if max(vals) > 0 else 0.0), "median": med,
                    "measurementProvenance": "settled_cross_checked" if state == "cross_checked" and all(s.get("settled") for s in g) else "measured_unsettled",
                    "replicationStatus": same_class_replication_status(
                        ["cross_machine_same_class" if len(machines) > 1 else "cross_process_same_host" if len(g) > 1 else "single_observation"]),
                    "receiptRefs": sorted({s["receiptRef"] for s in g if s.get("receiptRef")})})
    return out


def admit_device(distributions: list[dict], device_class: str) -> dict:
    """A device class is admitted for paid training work when every benchmark metric is cross-checked and no
    verified thermal probe shows throttling."""
    mine = {d["metric"]: d for d in distributions if d["deviceClassRef"] == device_class}
    blockers = [f"blocker.device_capability.{m}_not_cross_checked" for m in BENCHMARK_MEASUREMENTS
                if mine.get(m, {}).get("crossCheckState") != "cross_checked"]
    th = mine.get(THERMAL_METRIC)
    status = thermal_throttle_status(th["p50"] if th else None, bool(th and th["crossCheckState"] in ("cross_checked", "needs_replication")))
    if status == "thermal_throttle_observed":
        blockers.append("blocker.device_capability.thermal_throttle_observed")
    return {"deviceClassRef": device_class, "admitted": not blockers, "thermalThrottleStatus": status, "blockerRefs": blockers}


# ---------------------------------------------------------------- gradient-window promotion gate
GW_STAGES = ("submitted", "quarantined", "recomputed", "replicated", "canary_passed", "promoted", "blocked")
_GW = "blocker.public.tassadar_gradient_window."
_SAFE_REF = re.compile(r"^[A-Za-z0-9][A-Za-z0-9_.:/-]{0,260}$")
_DIGEST = re.compile(r"^(digest\.sha256\.|sha256:)?[a-f0-9]{32,128}$", re.I)
_UNSAFE_GW = re.compile(r"(@|/Users/|/home/|access[_-]?token|auth\.json|bearer|cookie|dataset\.(private|raw)|mnemonic|password|secret|wallet)", re.I)
_CORE_WORDS = ("compiled_exact_core", "compiled_core", "exact_core", "frozen_core", "analytic_executor", "tassadar_alm_numeric_executor",
               "tassadar_alm_numeric_execute")


class GradientWindowUnsafe(Exception):
    pass


def _safe_refs(label: str, refs) -> list[str]:
    out = sorted({r.strip() for r in refs if r is not None and r.strip()})
    for r in out:
        if not _SAFE_REF.match(r) or _UNSAFE_GW.search(r):
            raise GradientWindowUnsafe(f"{label} must be public-safe refs")
    return out


def project_gradient_window(candidate: dict, receipts: dict) -> dict:
    c, r = candidate, receipts
    _safe_refs("identity refs", [c["compiledCoreRef"], c["contributorRef"], c["modelFamilyRef"], c["randomSeedRef"], c["windowRef"],
                                 *c["frozenParameterScopes"], *c["trainableParameterScopes"]])
    construction = _safe_refs("construction receipt refs", c["constructionReceiptRefs"])
    verification = _safe_refs("verification receipt refs", c["verificationReceiptRefs"])
    curated = _safe_refs("curated data refs", c["curatedDataRefs"])
    quarantine = _safe_refs("quarantine receipt refs", r["quarantineReceiptRefs"])
    recompute_refs = _safe_refs("recompute receipt refs", r["recompute"]["receiptRefs"])
    replication_refs = _safe_refs("replication receipt refs", r["replication"]["receiptRefs"])
    canary_refs = _safe_refs("canary receipt refs", r["canary"]["receiptRefs"])
    decisions = _safe_refs("promotion decision refs", r["promotionDecisionRefs"])
    settlement = _safe_refs("settlement receipt refs", r.get("settlementReceiptRefs", []))
    for label in ("baseCheckpointDigest", "datasetShardDigest", "frozenCoreDigestAfter", "frozenCoreDigestBefore", "learnedInterfaceDigest",
                  "optimizerStateDigest", "quarantineCheckpointDigest", "trainingConfigDigest", "updateDigest"):
        if not _DIGEST.match(c[label]):
            raise GradientWindowUnsafe(f"{label} must be a sha256-style digest")
    for d in [r["recompute"]["expectedUpdateDigest"], r["recompute"]["recomputedUpdateDigest"], *r["replication"]["replicaUpdateDigests"]]:
        if not _DIGEST.match(d):
            raise GradientWindowUnsafe("receipt digests must be sha256-style digests")
    targets_core = lambda scope: any(w in scope.lower() for w in _CORE_WORDS)
    core_unchanged = c["frozenCoreDigestBefore"] == c["frozenCoreDigestAfter"]
    trainable_core = any(targets_core(s) for s in c["trainableParameterScopes"])
    frozen_core_present = any(targets_core(s) for s in c["frozenParameterScopes"])
    core_blocked = (not core_unchanged or c["compiledCoreGradientTargeted"] or trainable_core or not frozen_core_present
                    or not c["gradientsFlowThroughTrace"])
    quarantine_ok = bool(quarantine)
    recompute_ok = (bool(recompute_refs) and r["recompute"]["passed"] and r["recompute"]["expectedUpdateDigest"] == c["updateDigest"]
                    and r["recompute"]["recomputedUpdateDigest"] == c["updateDigest"])
    reps = r["replication"]["replicaUpdateDigests"]
    replication_ok = bool(replication_refs) and r["replication"]["passed"] and len(reps) >= 2 and all(d == c["updateDigest"] for d in reps)
    full = lambda v: isinstance(v, (int, float)) and math.isfinite(v) and v >= 1
    canary_ok = (bool(canary_refs) and r["canary"]["passed"] and full(r["canary"]["exactRolloutPassAt1"])
                 and full(r["canary"]["outputDigestMatchRate"]) and full(r["canary"]["replayAcceptanceRate"]))
    checks = ((not construction, "construction_substrate_missing"), (not verification, "verification_substrate_missing"),
              (not curated, "curated_data_refs_missing"), (not core_unchanged, "frozen_core_digest_changed"),
              (c["compiledCoreGradientTargeted"] or trainable_core, "compiled_core_gradient_targeted"),
              (not frozen_core_present, "frozen_core_scope_missing"), (not c["gradientsFlowThroughTrace"], "trace_not_forward_pass"),
              (not quarantine_ok, "quarantine_missing"), (not recompute_ok, "recompute_missing_or_failed"),
              (not replication_ok, "replication_missing_or_failed"), (not canary_ok, "canary_missing_or_failed"),
              (not decisions, "promotion_decision_missing"))
    blockers = sorted({_GW + name for bad, name in checks if bad})
    promoted = not blockers
    if promoted:
        stage = "promoted"
    elif core_blocked:
        stage = "blocked"
    else:
        stage = ("canary_passed" if quarantine_ok and recompute_ok and replication_ok and canary_ok else
                 "replicated" if quarantine_ok and recompute_ok and replication_ok else
                 "recomputed" if quarantine_ok and recompute_ok else "quarantined" if quarantine_ok else "submitted")
    return {"windowRef": c["windowRef"], "stage": stage, "promotionAllowed": promoted, "blockerRefs": blockers,
            "compiledCoreUnchanged": core_unchanged, "settlementEligible": promoted and bool(settlement),
            "authority": {"canonicalCheckpointMutationAllowed": promoted, "compiledCoreGradientMutationAllowed": False,
                          "directSubmissionMutationAllowed": False, "quarantineCheckpointMutationAllowed": quarantine_ok and not core_blocked,
                          "settlementMutationAllowed": False},
            "gateRef": "gate.public.tassadar_gradient_window." + re.sub(r"[^A-Za-z0-9_.:/-]", "_", c["windowRef"])[:120]}


# ---------------------------------------------------------------- kernel-optimization campaigns
PARITY_CLASS_ID = "kernel_optimization_throughput_parity.v1"
CAMPAIGN_CLASS_ID = "kernel_optimization_campaign.v1"
MAX_SATS = 21_000_000_000_000


class CampaignError(Exception):
    pass


def _slug(job: dict) -> str:
    return re.sub(r"[^a-z0-9]+", "-", "|".join(job[k].strip().lower() for k in ("kernelRef", "targetModel", "device", "hardwareRef"))).strip("-")


def build_campaign(campaign_ref: str, jobs: list[dict]) -> dict:
    """Fan a campaign out into one work request per (kernel, model, device, hardware) target."""
    if not campaign_ref.strip():
        raise CampaignError("campaignRef must be non-empty")
    if not jobs:
        raise CampaignError("campaign must contain at least one job")
    seen, requests, total = set(), [], 0
    for j in jobs:
        if not (isinstance(j["budgetSats"], int) and 0 < j["budgetSats"] <= MAX_SATS):
            raise CampaignError("budgetSats must be a positive whole number of sats")
        slug = _slug(j)
        if slug in seen:
            raise CampaignError(f"duplicate campaign target: {slug}")
        seen.add(slug)
        total += j["budgetSats"]
        requests.append({"requestedSlug": slug, "budgetSats": j["budgetSats"], "opRef": j["opRef"].strip(),
                         "target": {"targetModel": j["targetModel"], "device": j["device"], "hardwareRef": j["hardwareRef"]},
                         "kernelRef": j["kernelRef"], "verificationClass": PARITY_CLASS_ID})
    return {"classId": CAMPAIGN_CLASS_ID, "campaignRef": campaign_ref.strip(), "requests": requests, "totalBudgetSats": total}


def verify_kernel_parity(optimized_op_ref: str, baseline: dict, optimized: dict, parity: dict, baseline_parity: dict) -> dict:
    """``baseline`` / ``optimized``: throughput records {targetModel, device, hardwareRef, opRef, kernelRef,
    graphDigest, tokensPerSecond}; ``parity`` / ``baseline_parity``: replay verdicts of their outputs."""
    pos = lambda v: isinstance(v, (int, float)) and math.isfinite(v) and v > 0
    ok_tp = pos(baseline["tokensPerSecond"]) and pos(optimized["tokensPerSecond"])
    base = {"classId": PARITY_CLASS_ID, "optimizedOpRef": optimized_op_ref.strip(), "baselineTokensPerSecond": baseline["tokensPerSecond"],
            "optimizedTokensPerSecond": optimized["tokensPerSecond"], "parityOutcome": parity["outcome"],
            "speedupRatio": optimized["tokensPerSecond"] / baseline["tokensPerSecond"] if ok_tp else None,
            "target": {k: baseline[k] for k in ("targetModel", "device", "hardwareRef")}}
    rej = lambda reason, **kw: {**base, "outcome": "rejected", "rejection": {"reason": reason, **kw}}
    norm = lambda s: (s or "").strip().lower()
    if any(baseline[k] != optimized[k] for k in ("targetModel", "device", "hardwareRef")):
        return rej("target_mismatch")
    op = norm(optimized_op_ref)
    if not op or norm(baseline["opRef"]) != op or norm(optimized["opRef"]) != op:
        return rej("op_mismatch")
    if not norm(optimized["kernelRef"]) or norm(optimized["kernelRef"]) == norm(baseline["kernelRef"]):
        return rej("kernel_not_optimized")
    if not norm(optimized["graphDigest"]) or norm(optimized["graphDigest"]) != norm(parity["graphDigest"]):
        return rej("parity_trace_unbound")
    if not norm(baseline["graphDigest"]) or norm(baseline["graphDigest"]) != norm(baseline_parity["graphDigest"]):
        return rej("parity_trace_unbound")
    if not ok_tp:
        return rej("invalid_throughput")
    if parity["outcome"] != "verified":
        return rej("parity_rejected", parityRejection=parity.get("rejection"))
    if baseline_parity["outcome"] != "verified" or parity["validatorDeviceRef"].strip() != baseline_parity["validatorDeviceRef"].strip():
        return rej("output_parity_mismatch")
    a, b = norm(parity.get("replayedTraceDigest")), norm(baseline_parity.get("replayedTraceDigest"))
    if not a or not b or a != b:
        return rej("output_parity_mismatch")
    if optimized["tokensPerSecond"] <= baseline["tokensPerSecond"]:
        return rej("no_throughput_improvement", baselineTokensPerSecond=baseline["tokensPerSecond"], optimizedTokensPerSecond=optimized["tokensPerSecond"])
    return {**base, "outcome": "accepted", "rejection": None}


def settle_campaign(campaign: dict, settled: list[dict]) -> dict:
    """``settled``: {requestedSlug, budgetSats, verdict}.  Accepted jobs are owed their budget, rejected ones are
    refunded; the reconciliation checks job count, per-job budgets, targets and ops, and that escrow is conserved."""
    by_slug = {r["requestedSlug"]: r for r in campaign["requests"]}
    seen, dup, unexpected, budget_mismatch, target_mismatch, op_mismatch = set(), [], [], [], [], []
    owed = refunded = accepted = 0
    reasons: dict[str, int] = {}
    speedups = []
    for s in settled:
        slug = s["requestedSlug"]
        if slug in seen:
            dup.append(slug)
            continue
        seen.add(slug)
        req = by_slug.get(slug)
        if req is None:
            unexpected.append(slug)
            continue
        if s["budgetSats"] != req["budgetSats"]:
            budget_mismatch.append({"requestedSlug": slug, "dispatchedSats": req["budgetSats"], "settledSats": s["budgetSats"]})
        v = s["verdict"]
        if v["target"] != req["target"]:
            target_mismatch.append(slug)
        if v["optimizedOpRef"].strip().lower() != req["opRef"].lower():
            op_mismatch.append(slug)
        if v["outcome"] == "accepted":
            accepted += 1
            owed += s["budgetSats"]
            if v.get("speedupRatio"):
                speedups.append(v["speedupRatio"])
        else:
            refunded += s["budgetSats"]
            reason = (v.get("rejection") or {}).get("reason", "unknown")
            reasons[reason] = reasons.get(reason, 0) + 1
    unsettled = sorted(set(by_slug) - seen)
    discrepancies = ([f"duplicate:{s}" for s in dup] + [f"unexpected:{s}" for s in unexpected] + [f"unsettled:{s}" for s in unsettled]
                     + [f"budget:{m['requestedSlug']}" for m in budget_mismatch] + [f"target:{s}" for s in target_mismatch] + [f"op:{s}" for s in op_mismatch])
    conserved = owed + refunded == campaign["totalBudgetSats"]
    if not conserved:
        discrepancies.append("escrow_not_conserved")
    return {"classId": CAMPAIGN_CLASS_ID, "campaignRef": campaign["campaignRef"], "ok": not discrepancies, "totalJobs": len(campaign["requests"]),
            "settledJobs": len(seen), "acceptedCount": accepted, "rejectedCount": len(seen) - len(unexpected) - accepted, "payoutOwedSats": owed,
            "refundedSats": refunded, "escrowSats": campaign["totalBudgetSats"], "escrowConserved": conserved, "rejectionReasonCounts": reasons,
            "speedup": {"min": min(speedups), "max": max(speedups), "mean": sum(speedups) / len(speedups)} if speedups else None,
            "discrepancies": discrepancies}
