"""The gym's publishing layer: leaderboard, benchmark ladder, module-author split and the flywheel gate.

Everything here is a pure function of benchmark reports (``gateway.benchmark``): no network, no clock.

* ``leaderboard_projection``: one row per decision-grade report with accepted outcomes, ranked by cost per accepted
  outcome, then verification rate, then accepted outcomes, then ref; every other report is listed with the reason it was
  left out (inference/gym/leaderboard.ts:30-70 row and exclusion types, :118-214 row building, :219-262 ordering).
* ``ladder_leaderboard``: the recurring four-rung ladder (default free model, free / open field, paid frontier, public
  software-reproduction bucket).  A rung is ``published`` only when a decision-grade row of the protagonist and of at
  least one of its opponents exists; otherwise ``awaiting_owner`` with the blockers that explain why, never a number
  (inference/gym/ladder.ts:1-27 contract, :73-117 rung definitions, :228-301 reproduction rung, :303-333 blockers, :335-409).
* ``module_author_split``: how a contributor share would divide over the authors of the modules a run composed;
  modelled only, never a payout claim (leaderboard.ts:264-398).
* ``flywheel_evaluation``: whether a tuned candidate may shadow, or be promoted to, the live route: both reports
  decision grade, the candidate strictly cheaper per accepted outcome, a reward bundle, a training-frontier ref from the
  training stack and dog-food attribution present; runtime promotion additionally needs an approval ref
  (inference/gym/flywheel.ts:146-164 cost summary, :283-300 improvement, :302-434 evaluation).
"""
from __future__ import annotations

import re

from .benchmark import lane_availability

LEADERBOARD_SCHEMA = "openagents.gym.leaderboard_projection.v1"
LADDER_SCHEMA = "openagents.gym.ladder_leaderboard.v1"
SPLIT_SCHEMA = "openagents.gym.module_author_split_projection.v1"
FLYWHEEL_SCHEMA = "openagents.gym.flywheel_evaluation.v1"
PROTAGONIST = "khala"
_SAFE_REF = re.compile(r"^[A-Za-z0-9][A-Za-z0-9_.:/|@-]{0,200}$")
_UNSAFE = re.compile(r"(api[_-]?key|bearer|secret|password|mnemonic|/Users/|/home/|sk-[a-z0-9])", re.I)

RUNGS = (
    {"rung": "rung1", "title": "Rung 1: against the default free model", "family": "opencode_head_to_head", "opponentLanes": ("bigpickle",),
     "ownerGateRef": "gate.owner.gym.ladder.rung1.real_seam_with_bigpickle_model_id"},
    {"rung": "rung2", "title": "Rung 2: against free and open models", "family": "opencode_head_to_head",
     "opponentLanes": ("gemini-free", "gpt-oss-20b", "gpt-oss-120b", "glm-52"), "ownerGateRef": "gate.owner.gym.ladder.rung2.free_tier_real_seam"},
    {"rung": "rung3", "title": "Rung 3: against the paid frontier", "family": "opencode_head_to_head", "opponentLanes": ("claude", "openai-gpt", "vertex-gemini"),
     "ownerGateRef": "gate.owner.gym.ladder.rung3.paid_frontier_keys_and_spend_approval"},
    {"rung": "rung4", "title": "Rung 4: public software-reproduction bucket", "family": "mirrorcode_public_bucket", "opponentLanes": (),
     "ownerGateRef": "gate.owner.gym.ladder.rung4.mirrorcode_public_bucket_real_run"},
)


class GymUnsafe(ValueError):
    pass


def _unique(refs):
    out = []
    for r in refs:
        if r and r not in out:
            out.append(r)
    return out


def _assert_refs(label, refs):
    for r in refs:
        if not isinstance(r, str) or not _SAFE_REF.match(r) or _UNSAFE.search(r):
            raise GymUnsafe(f"{label}: {r!r} is not a public-safe ref")
    return _unique(refs)


def _segment(parts, fallback):
    s = re.sub(r"[^A-Za-z0-9_.-]+", "_", ".".join(parts)).strip("._")
    return s[:160] or fallback


def cost_per_accepted_outcome(report: dict) -> dict:
    accepted = sum(g.get("acceptedOutcomes", 0) for g in report["groups"])
    cost = sum(g.get("totalCostBasisMsat", 0) for g in report["groups"])
    return {"acceptedOutcomes": accepted, "totalCostBasisMsat": cost, "costPerAcceptedOutcomeMsat": None if accepted == 0 else cost / accepted}


def _row(inp: dict):
    _assert_refs("leaderboard report refs", [inp["reportRef"], inp["receiptRef"], inp["candidateRef"], inp["environmentRef"], inp["coordinatorRef"]])
    rep = inp["report"]
    if not rep.get("publicSafe", True):
        return {"reportRef": inp["reportRef"], "reason": "public_safety_violation"}
    if not rep.get("decisionGrade"):
        return {"reportRef": inp["reportRef"], "reason": "not_decision_grade"}
    c = cost_per_accepted_outcome(rep)
    if c["acceptedOutcomes"] <= 0:
        return {"reportRef": inp["reportRef"], "reason": "no_accepted_outcomes"}
    groups = rep["groups"]
    attempted = sum(g.get("attemptedVerifications", 0) for g in groups)
    wall_n = sum(g.get("wallClockSamples", 0) for g in groups)
    wall = sum((g.get("meanWallClockMs") or 0.0) * g.get("wallClockSamples", 0) for g in groups)
    return {"rank": 0, "reportRef": inp["reportRef"], "receiptRef": inp["receiptRef"], "configId": rep.get("configId", ""),
            "environmentRef": inp["environmentRef"], "candidateRef": inp["candidateRef"], "coordinatorRef": inp["coordinatorRef"],
            "acceptedOutcomes": c["acceptedOutcomes"], "attemptedVerifications": attempted,
            "verificationRateBps": None if attempted == 0 else round(c["acceptedOutcomes"] / attempted * 10_000),
            "inputTokens": sum(g.get("inputTokens", 0) for g in groups), "outputTokens": sum(g.get("outputTokens", 0) for g in groups),
            "totalTokens": sum(g.get("totalTokens", 0) for g in groups), "meanWallClockMs": None if wall_n == 0 else wall / wall_n,
            "costPerAcceptedOutcomeMsat": c["costPerAcceptedOutcomeMsat"], "totalCostBasisMsat": c["totalCostBasisMsat"],
            "cellsExecuted": rep.get("cellsExecuted", 0)}


def leaderboard_projection(inputs: list[dict]) -> dict:
    """``inputs``: ``{report, reportRef, receiptRef, candidateRef, environmentRef, coordinatorRef}``; a report has
    ``decisionGrade``, optional ``publicSafe`` and ``groups`` with the per-group counters."""
    cands = [_row(i) for i in inputs]
    rows = sorted((c for c in cands if "rank" in c),
                  key=lambda r: (r["costPerAcceptedOutcomeMsat"], -(r["verificationRateBps"] if r["verificationRateBps"] is not None else -1),
                                 -r["acceptedOutcomes"], r["reportRef"]))
    rows = [{**r, "rank": i + 1} for i, r in enumerate(rows)]
    return {"schemaVersion": LEADERBOARD_SCHEMA, "projectionRef": "projection.gym.leaderboard." + _segment([r["reportRef"] for r in rows], "empty"),
            "rowCount": len(rows), "rows": rows, "excludedReports": [c for c in cands if "rank" not in c],
            "caveatRefs": ["caveat.public.gym.leaderboard.decision_grade_only", "caveat.public.gym.leaderboard.public_safe_fields_only",
                           "caveat.public.gym.leaderboard.no_fixture_or_synthetic_ranking"]}


def _lane_of(candidate_ref: str):
    head = re.split(r"[./|]", candidate_ref)[0]
    try:
        lane_availability(head)
        return head
    except (KeyError, ValueError):
        return None


def _entry(row, family="opencode_head_to_head"):
    return {"rank": row["rank"], "lane": _lane_of(row["candidateRef"]), "benchmarkFamily": family, "reportRef": row["reportRef"],
            "candidateRef": row["candidateRef"], "acceptedOutcomes": row["acceptedOutcomes"], "verificationRateBps": row["verificationRateBps"],
            "costPerAcceptedOutcomeMsat": row["costPerAcceptedOutcomeMsat"], "passRateBps": None, "tokensTotal": 0, "exactTokenUsageEventRefs": []}


def _reproduction_rung(d, runs):
    good = [r for r in runs if r.get("decisionGrade") and r.get("passRate") is not None and r.get("exactTokenUsageEventRefs")]
    good.sort(key=lambda r: (-r["passRate"], r["tokensTotal"], r["runId"]))
    entries = [{"rank": i + 1, "lane": PROTAGONIST, "benchmarkFamily": d["family"], "reportRef": f"report.gym.mirrorcode.{r['runId']}",
                "candidateRef": f"{PROTAGONIST}.mirrorcode.{r['bucket']}.{r['taskId']}", "acceptedOutcomes": 1 if r.get("status") == "passed" else 0,
                "verificationRateBps": round(r["passRate"] * 10_000), "costPerAcceptedOutcomeMsat": 0, "passRateBps": round(r["passRate"] * 10_000),
                "tokensTotal": r["tokensTotal"], "exactTokenUsageEventRefs": list(r["exactTokenUsageEventRefs"])} for i, r in enumerate(good)]
    return {"rung": d["rung"], "title": d["title"], "benchmarkFamily": d["family"], "state": "published" if entries else "awaiting_owner",
            "opponentLanes": [], "entries": entries,
            "blockerRefs": [] if entries else ["blocker.gym.ladder.mirrorcode_no_decision_grade_public_bucket_run",
                                               "blocker.gym.ladder.mirrorcode_exact_token_rows_missing", d["ownerGateRef"]],
            "passRateBps": round(sum(e["passRateBps"] for e in entries) / len(entries)) if entries else None,
            "tokensTotal": sum(e["tokensTotal"] for e in entries),
            "exactTokenUsageEventRefs": _unique([x for e in entries for x in e["exactTokenUsageEventRefs"]])}


def ladder_leaderboard(inputs: list[dict], rungs=RUNGS, reproduction_runs=(), cadence: str = "weekly") -> dict:
    if cadence not in ("weekly", "per_model_release", "on_demand"):
        raise ValueError("unknown cadence")
    proj = leaderboard_projection(inputs)
    ours = [r for r in proj["rows"] if _lane_of(r["candidateRef"]) == PROTAGONIST or PROTAGONIST in r["candidateRef"]]
    best = ours[0] if ours else None
    out = []
    for d in rungs:
        if d["family"] == "mirrorcode_public_bucket":
            out.append(_reproduction_rung(d, list(reproduction_runs)))
            continue
        lanes = set(d["opponentLanes"])
        opp = [r for r in proj["rows"] if _lane_of(r["candidateRef"]) in lanes]
        measured = {_lane_of(r["candidateRef"]) for r in opp}
        published = best is not None and bool(opp)
        entries = []
        if published:
            entries = sorted([_entry(best)] + [_entry(r) for r in opp], key=lambda e: e["costPerAcceptedOutcomeMsat"])
            entries = [{**e, "rank": i + 1} for i, e in enumerate(entries)]
        blockers = []
        if not published:
            if best is None:
                blockers.append("blocker.gym.ladder.no_decision_grade_khala_row")
            for lane in d["opponentLanes"]:
                if lane in measured:
                    continue
                av = lane_availability(lane)
                blockers.append(f"blocker.gym.ladder.opponent_not_yet_measured.{lane}" if av == "available" else f"blocker.gym.ladder.opponent_lane_{av}.{lane}")
            if d["ownerGateRef"]:
                blockers.append(d["ownerGateRef"])
        out.append({"rung": d["rung"], "title": d["title"], "benchmarkFamily": d["family"], "state": "published" if published else "awaiting_owner",
                    "opponentLanes": list(d["opponentLanes"]), "entries": entries, "blockerRefs": _unique(blockers), "passRateBps": None,
                    "tokensTotal": 0, "exactTokenUsageEventRefs": []})
    return {"schemaVersion": LADDER_SCHEMA, "ladderRef": "ladder.gym.recurring.v1", "cadence": cadence, "demandKind": "internal", "demandSource": "gym_ladder",
            "projectionRef": proj["projectionRef"], "decisionGradeRowCount": proj["rowCount"], "rungs": out, "excludedReports": proj["excludedReports"],
            "caveatRefs": ["caveat.public.gym.ladder.decision_grade_rungs_only", "caveat.public.gym.ladder.fixture_or_synthetic_never_published",
                           "caveat.public.gym.ladder.awaiting_owner_rungs_show_gate_not_numbers",
                           "caveat.public.gym.ladder.no_beats_frontier_claim_from_single_run"]}


def module_author_split(report: dict, report_ref: str, owner_armed: bool, gross_revenue_msat: int, contributor_share_msat: int, contributions: list[dict]) -> dict:
    """``contributions``: ``{moduleRef, authorRef, programSignatureRef, evidenceRef, weightBps}``; weights must sum to 10 000."""
    _assert_refs("module author split refs", [report_ref] + [c[k] for c in contributions for k in ("moduleRef", "authorRef", "programSignatureRef", "evidenceRef")])
    for v in (gross_revenue_msat, contributor_share_msat):
        if not isinstance(v, int) or isinstance(v, bool) or v < 0:
            raise GymUnsafe("revenue amounts must be non-negative integer msat")
    b = []
    if not owner_armed:
        b.append("blocker.gym.author_split.owner_arming_missing")
    if not report.get("decisionGrade"):
        b.append("blocker.gym.author_split.report_not_decision_grade")
    if gross_revenue_msat <= 0:
        b.append("blocker.gym.author_split.gross_revenue_missing")
    if contributor_share_msat <= 0:
        b.append("blocker.gym.author_split.contributor_share_missing")
    if contributor_share_msat > gross_revenue_msat:
        b.append("blocker.gym.author_split.contributor_share_exceeds_gross")
    if not contributions:
        b.append("blocker.gym.author_split.composition_evidence_missing")
    if any(not isinstance(c["weightBps"], int) or c["weightBps"] <= 0 for c in contributions):
        b.append("blocker.gym.author_split.invalid_contribution_weight")
    if contributions and sum(c["weightBps"] for c in contributions) != 10_000:
        b.append("blocker.gym.author_split.contribution_weights_must_sum_to_10000")
    shares = [] if b else [{**c, "shareMsat": contributor_share_msat * c["weightBps"] // 10_000} for c in contributions]
    return {"schemaVersion": SPLIT_SCHEMA, "splitRef": "split.gym.module_author." + _segment([report_ref] + [c["moduleRef"] for c in contributions], "split"),
            "reportRef": report_ref, "ownerArmed": owner_armed, "state": "blocked" if b else "modeled", "grossRevenueMsat": gross_revenue_msat,
            "contributorShareMsat": contributor_share_msat, "shares": shares, "evidenceRefs": _unique([c["evidenceRef"] for c in contributions]),
            "blockerRefs": b, "authorPayoutClaimAllowed": False, "marketplaceListingAllowed": False, "settlementMutationAllowed": False}


def cost_improvement_bps(baseline: dict, candidate: dict):
    a, c = baseline["costPerAcceptedOutcomeMsat"], candidate["costPerAcceptedOutcomeMsat"]
    if a is None or c is None or a <= 0:
        return None
    return round((a - c) / a * 10_000)


def flywheel_evaluation(baseline_report: dict, candidate_report: dict, baseline_ref: str, candidate_report_ref: str, candidate_ref: str,
                        candidate_hash: str, environment_ref: str, reward_bundle_refs=(), training_frontier_refs=(), dogfood_event_refs=(),
                        requested_promotion: str = "shadow", runtime_promotion_approval_ref: str | None = None) -> dict:
    if requested_promotion not in ("shadow", "runtime_promotion"):
        raise ValueError("requested_promotion is shadow or runtime_promotion")
    _assert_refs("flywheel refs", [baseline_ref, candidate_report_ref, candidate_ref, candidate_hash, environment_ref]
                 + ([runtime_promotion_approval_ref] if runtime_promotion_approval_ref else []))
    rewards, frontier, dogfood = (_assert_refs(n, list(r)) for n, r in (("reward bundle refs", reward_bundle_refs),
                                                                        ("training frontier refs", training_frontier_refs), ("dog-food refs", dogfood_event_refs)))
    base, cand = cost_per_accepted_outcome(baseline_report), cost_per_accepted_outcome(candidate_report)
    imp = cost_improvement_bps(base, cand)
    core = []
    if not baseline_report.get("decisionGrade"):
        core.append("blocker.gym.flywheel.baseline_not_decision_grade")
    if not candidate_report.get("decisionGrade"):
        core.append("blocker.gym.flywheel.candidate_not_decision_grade")
    if cand["acceptedOutcomes"] <= 0:
        core.append("blocker.gym.flywheel.no_candidate_accepted_outcomes")
    if imp is None or imp <= 0:
        core.append("blocker.gym.flywheel.candidate_not_cheaper_than_heuristic")
    if not rewards:
        core.append("blocker.gym.flywheel.missing_reward_bundle")
    if not frontier:
        core.append("blocker.gym.flywheel.missing_psionic_frontier")
    if not dogfood:
        core.append("blocker.gym.flywheel.missing_khala_dogfood_attribution")
    shadow_ready = not core
    wants_runtime = requested_promotion == "runtime_promotion"
    blockers = core + (["blocker.gym.flywheel.runtime_promotion_requires_approval"] if wants_runtime and not runtime_promotion_approval_ref else [])
    runtime_ok = shadow_ready and wants_runtime and bool(runtime_promotion_approval_ref)
    return {"schemaVersion": FLYWHEEL_SCHEMA, "evaluationRef": "evaluation.gym.flywheel." + _segment([baseline_ref, candidate_report_ref, candidate_ref], "evaluation"),
            "candidateRef": candidate_ref, "candidateHash": candidate_hash, "environmentRef": environment_ref, "requestedPromotion": requested_promotion,
            "candidateState": "blocked" if not shadow_ready else ("runtime_promotion_ready" if runtime_ok else "shadow"),
            "shadowCandidateRef": "candidate.gym.shadow." + _segment([candidate_ref], "candidate") if shadow_ready else None,
            "runtimePromotionRef": "runtime_promotion.gym." + _segment([candidate_ref, runtime_promotion_approval_ref], "candidate") if runtime_ok else None,
            "runtimePromotionAllowed": runtime_ok, "blockers": _unique(blockers), "baseline": base, "candidate": cand, "costImprovementBps": imp,
            "rewardBundleRefs": rewards, "psionicFrontierRefs": frontier, "dogfoodEventRefs": dogfood}
