"""Leaderboard ordering and exclusions, ladder rungs, author split and the flywheel gate."""
import pytest

from openagents_b200.gateway import gym


def rep(accepted, cost, attempted=None, grade=True, safe=True, wall=(100.0, 4)):
    return {"decisionGrade": grade, "publicSafe": safe, "configId": "cfg.a", "cellsExecuted": 3,
            "groups": [{"acceptedOutcomes": accepted, "totalCostBasisMsat": cost, "attemptedVerifications": attempted if attempted is not None else accepted + 1,
                        "inputTokens": 10, "outputTokens": 5, "totalTokens": 15, "meanWallClockMs": wall[0], "wallClockSamples": wall[1]}]}


def inp(ref, cand, report):
    return {"report": report, "reportRef": ref, "receiptRef": "receipt." + ref, "candidateRef": cand, "environmentRef": "env.opencode", "coordinatorRef": "coord.a"}


def test_leaderboard_orders_by_cost_then_verification_and_lists_exclusions():
    inputs = [inp("r.slow", "gpt-oss-20b.v1", rep(4, 4000)), inp("r.khala", "khala.v3", rep(5, 2500, attempted=5)),
              inp("r.tie", "glm-52.v1", rep(5, 2500, attempted=10)), inp("r.fixture", "bigpickle.v1", rep(3, 30, grade=False)),
              inp("r.none", "claude.v1", rep(0, 100)), inp("r.leak", "fireworks.v1", rep(3, 30, safe=False))]
    p = gym.leaderboard_projection(inputs)
    assert [r["reportRef"] for r in p["rows"]] == ["r.khala", "r.tie", "r.slow"] and [r["rank"] for r in p["rows"]] == [1, 2, 3]
    assert p["rows"][0]["verificationRateBps"] == 10000 and p["rows"][1]["verificationRateBps"] == 5000 and p["rows"][0]["meanWallClockMs"] == 100.0
    assert {e["reportRef"]: e["reason"] for e in p["excludedReports"]} == {"r.fixture": "not_decision_grade", "r.none": "no_accepted_outcomes",
                                                                           "r.leak": "public_safety_violation"}
    with pytest.raises(gym.GymUnsafe):
        gym.leaderboard_projection([inp("r.x", "khala.sk-abc123", rep(1, 1))])


def test_ladder_publishes_only_measured_rungs():
    inputs = [inp("r.khala", "khala.v3", rep(5, 2500)), inp("r.oss", "gpt-oss-20b.v1", rep(4, 4000)), inp("r.fx", "bigpickle.v1", rep(3, 30, grade=False))]
    runs = [{"runId": "m1", "decisionGrade": True, "passRate": 0.5, "tokensTotal": 900, "exactTokenUsageEventRefs": ["usage.m1"], "bucket": "public", "taskId": "t1", "status": "passed"},
            {"runId": "m2", "decisionGrade": True, "passRate": 0.75, "tokensTotal": 1200, "exactTokenUsageEventRefs": ["usage.m2"], "bucket": "public", "taskId": "t2", "status": "failed"},
            {"runId": "m3", "decisionGrade": True, "passRate": 0.9, "tokensTotal": 10, "exactTokenUsageEventRefs": [], "bucket": "public", "taskId": "t3", "status": "passed"}]
    lad = gym.ladder_leaderboard(inputs, reproduction_runs=runs)
    r1, r2, r3, r4 = lad["rungs"]
    assert r1["state"] == "awaiting_owner" and r1["entries"] == [] and "blocker.gym.ladder.opponent_lane_fixture_only.bigpickle" in r1["blockerRefs"]
    assert r1["blockerRefs"][-1].startswith("gate.owner.gym.ladder.rung1")
    assert r2["state"] == "published" and [e["lane"] for e in r2["entries"]] == ["khala", "gpt-oss-20b"] and r2["blockerRefs"] == []
    assert r3["state"] == "awaiting_owner" and "blocker.gym.ladder.opponent_not_yet_measured.vertex-gemini" in r3["blockerRefs"]
    assert r4["state"] == "published" and [e["reportRef"] for e in r4["entries"]] == ["report.gym.mirrorcode.m2", "report.gym.mirrorcode.m1"]
    assert r4["passRateBps"] == 6250 and r4["tokensTotal"] == 2100 and r4["exactTokenUsageEventRefs"] == ["usage.m2", "usage.m1"]
    none = gym.ladder_leaderboard([inp("r.oss", "gpt-oss-20b.v1", rep(4, 4000))])
    assert none["rungs"][1]["state"] == "awaiting_owner" and "blocker.gym.ladder.no_decision_grade_khala_row" in none["rungs"][1]["blockerRefs"]
    assert none["rungs"][3]["state"] == "awaiting_owner" and none["decisionGradeRowCount"] == 1


def test_author_split_models_shares_or_blocks():
    cs = [{"moduleRef": "module.a", "authorRef": "author.1", "programSignatureRef": "sig.a", "evidenceRef": "ev.a", "weightBps": 7000},
          {"moduleRef": "module.b", "authorRef": "author.2", "programSignatureRef": "sig.b", "evidenceRef": "ev.b", "weightBps": 3000}]
    s = gym.module_author_split(rep(2, 10), "r.khala", True, 10_001, 1_001, cs)
    assert s["state"] == "modeled" and [x["shareMsat"] for x in s["shares"]] == [700, 300] and not s["authorPayoutClaimAllowed"]
    b = gym.module_author_split(rep(2, 10, grade=False), "r.khala", False, 100, 200, [{**cs[0], "weightBps": 5000}])
    assert b["state"] == "blocked" and b["shares"] == [] and set(b["blockerRefs"]) == {
        "blocker.gym.author_split.owner_arming_missing", "blocker.gym.author_split.report_not_decision_grade",
        "blocker.gym.author_split.contributor_share_exceeds_gross", "blocker.gym.author_split.contribution_weights_must_sum_to_10000"}
    with pytest.raises(gym.GymUnsafe):
        gym.module_author_split(rep(1, 1), "r", True, -1, 0, cs)


def test_flywheel_needs_cheaper_candidate_evidence_and_approval():
    kw = dict(baseline_ref="r.base", candidate_report_ref="r.cand", candidate_ref="khala.tuned.v4", candidate_hash="sha256.abc", environment_ref="env.opencode",
              reward_bundle_refs=["reward.bundle.1"], training_frontier_refs=["frontier.train.1"], dogfood_event_refs=["dogfood.1"])
    e = gym.flywheel_evaluation(rep(4, 4000), rep(5, 2500), **kw)
    assert e["candidateState"] == "shadow" and e["costImprovementBps"] == 5000 and e["blockers"] == [] and e["shadowCandidateRef"] and not e["runtimePromotionAllowed"]
    e = gym.flywheel_evaluation(rep(4, 4000), rep(5, 2500), **kw, requested_promotion="runtime_promotion")
    assert e["candidateState"] == "shadow" and e["blockers"] == ["blocker.gym.flywheel.runtime_promotion_requires_approval"]
    e = gym.flywheel_evaluation(rep(4, 4000), rep(5, 2500), **kw, requested_promotion="runtime_promotion", runtime_promotion_approval_ref="approval.owner.7")
    assert e["candidateState"] == "runtime_promotion_ready" and e["runtimePromotionRef"].startswith("runtime_promotion.gym.")
    e = gym.flywheel_evaluation(rep(4, 4000), rep(5, 6000, grade=False), **{**kw, "training_frontier_refs": []})
    assert e["candidateState"] == "blocked" and set(e["blockers"]) == {"blocker.gym.flywheel.candidate_not_decision_grade",
                                                                        "blocker.gym.flywheel.candidate_not_cheaper_than_heuristic",
                                                                        "blocker.gym.flywheel.missing_psionic_frontier"}
    assert gym.cost_improvement_bps({"costPerAcceptedOutcomeMsat": None}, {"costPerAcceptedOutcomeMsat": 1.0}) is None
