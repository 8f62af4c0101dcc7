"""Model ladder, device-capability dataset, gradient-window gate and kernel-optimization campaigns."""
import copy

import pytest

from openagents_b200.control import programs as pg
from openagents_b200.oracle import tassadar as ts

H = "a" * 64


def test_model_ladder():
    p = pg.project_model_ladder()
    assert p["rungSummary"] == {"rungCount": 5, "closedRungCount": 1, "highestClosedRung": "R0", "nextRequiredRung": "R1"}
    assert pg.R1_BLOCKER in p["gate"]["remainingBlockerRefs"] and not p["gate"]["greenGateSatisfied"]
    crit = {c: f"receipt.r1.{c}" for c in pg.R1_CLOSEOUT_CRITERIA}
    p = pg.project_model_ladder({"R0": ["r0"], "R1": ["r1"], "R3": ["r3"]}, crit)
    assert p["rungSummary"]["highestClosedRung"] == "R1" and p["rungSummary"]["nextRequiredRung"] == "R2"
    assert p["rungs"][3]["status"] == "not_run"                      # R3 cannot close over an open R2
    p = pg.project_model_ladder({"R0": ["r0"], "R1": ["r1"]}, dict(crit, evals=""))
    assert p["rungSummary"]["highestClosedRung"] == "R0"
    with pytest.raises(pg.UnsafePublicMaterial):
        pg.project_model_ladder({"R0": ["receipt with walletSeed"]})


def _samples(cls, metric, values, machines, verified=True, settled=True):
    return [{"deviceClassRef": cls, "machineRef": m, "metric": metric, "value": v, "unit": "u", "verified": verified, "settled": settled,
             "receiptRef": f"receipt.{cls}.{metric}.{i}"} for i, (v, m) in enumerate(zip(values, machines))]


def test_device_capability_dataset():
    s = []
    for metric in pg.BENCHMARK_MEASUREMENTS:
        s += _samples("b200", metric, [100, 93, 97], ["m1", "m2", "m1"])
    s += _samples("b200", pg.THERMAL_METRIC, [0.95, 0.9], ["m1", "m2"])
    s += _samples("laptop", "tokens_per_second", [10], ["l1"])
    s += _samples("mini", "tokens_per_second", [10, 11], ["x", "x"])
    d = pg.device_capability_distributions(s)
    by = {(x["deviceClassRef"], x["metric"]): x for x in d}
    a = by[("b200", "attention_throughput")]
    assert a["p50"] == 97 and a["p90"] == 100 and a["crossCheckState"] == "cross_checked" and a["agreement"] == pytest.approx(0.93)
    assert a["measurementProvenance"] == "settled_cross_checked" and a["replicationStatus"] == "cross_machine_replicated"
    assert by[("laptop", "tokens_per_second")]["crossCheckState"] == "insufficient_same_class_samples"
    assert by[("mini", "tokens_per_second")]["crossCheckState"] == "needs_replication"
    assert pg.admit_device(d, "b200") == {"deviceClassRef": "b200", "admitted": True, "thermalThrottleStatus": "thermal_throttle_not_observed", "blockerRefs": []}
    assert not pg.admit_device(d, "laptop")["admitted"]
    hot = pg.device_capability_distributions(s[:12] + _samples("b200", pg.THERMAL_METRIC, [0.7, 0.75], ["m1", "m2"]))
    assert "blocker.device_capability.thermal_throttle_observed" in pg.admit_device(hot, "b200")["blockerRefs"]
    assert pg.thermal_throttle_status(None, True) == "missing" and pg.thermal_throttle_status(0.5, False) == "needs_verified_thermal_probe"
    assert pg.same_class_replication_status([]) == "missing" and pg.same_class_replication_status(["unknown"]) == "unknown_scope"
    with pytest.raises(ValueError):
        pg.device_capability_distributions([dict(s[0], metric="vibes")])


def _window():
    cand = {"baseCheckpointDigest": H, "compiledCoreGradientTargeted": False, "compiledCoreRef": "core.v1", "constructionReceiptRefs": ["r.c"],
            "contributorRef": "contributor.1", "curatedDataRefs": ["data.curated.1"], "datasetShardDigest": H, "frozenCoreDigestAfter": H,
            "frozenCoreDigestBefore": H, "frozenParameterScopes": ["scope.compiled_core"], "gradientsFlowThroughTrace": True,
            "learnedInterfaceDigest": H, "modelFamilyRef": "family.1", "optimizerStateDigest": H, "psionicH1EvidenceRefs": [],
            "quarantineCheckpointDigest": H, "randomSeedRef": "seed.1", "sourceRefs": [], "trainableParameterScopes": ["scope.interface"],
            "trainingConfigDigest": H, "updateDigest": "b" * 64, "verificationReceiptRefs": ["r.v"], "windowRef": "window.7"}
    rec = {"quarantineReceiptRefs": ["r.q"], "recompute": {"expectedUpdateDigest": "b" * 64, "recomputedUpdateDigest": "b" * 64, "passed": True, "receiptRefs": ["r.r"]},
           "replication": {"passed": True, "receiptRefs": ["r.rep"], "replicaUpdateDigests": ["b" * 64, "b" * 64]},
           "canary": {"exactRolloutPassAt1": 1, "outputDigestMatchRate": 1, "replayAcceptanceRate": 1, "passed": True, "receiptRefs": ["r.can"]},
           "promotionDecisionRefs": ["decision.1"], "rollbackRefs": [], "settlementReceiptRefs": ["settle.1"]}
    return cand, rec


def test_gradient_window_gate():
    cand, rec = _window()
    p = pg.project_gradient_window(cand, rec)
    assert p["stage"] == "promoted" and p["promotionAllowed"] and p["settlementEligible"] and p["authority"]["canonicalCheckpointMutationAllowed"]
    assert not p["authority"]["compiledCoreGradientMutationAllowed"] and not p["authority"]["settlementMutationAllowed"]
    r2 = copy.deepcopy(rec); r2["canary"]["replayAcceptanceRate"] = 0.99
    assert pg.project_gradient_window(cand, r2)["stage"] == "replicated"
    r2 = copy.deepcopy(rec); r2["replication"]["replicaUpdateDigests"] = ["b" * 64]
    assert pg.project_gradient_window(cand, r2)["stage"] == "recomputed"
    r2 = copy.deepcopy(rec); r2["recompute"]["recomputedUpdateDigest"] = "c" * 64
    assert pg.project_gradient_window(cand, r2)["stage"] == "quarantined"
    r2 = copy.deepcopy(rec); r2["quarantineReceiptRefs"] = []
    assert pg.project_gradient_window(cand, r2)["stage"] == "submitted"
    r2 = copy.deepcopy(rec); r2["promotionDecisionRefs"] = []
    assert pg.project_gradient_window(cand, r2)["stage"] == "canary_passed"
    c2 = dict(cand, trainableParameterScopes=["scope.compiled_core.w"])
    p = pg.project_gradient_window(c2, rec)
    assert p["stage"] == "blocked" and "blocker.public.tassadar_gradient_window.compiled_core_gradient_targeted" in p["blockerRefs"]
    assert not p["authority"]["quarantineCheckpointMutationAllowed"]
    assert pg.project_gradient_window(dict(cand, frozenCoreDigestAfter="d" * 64), rec)["stage"] == "blocked"
    with pytest.raises(pg.GradientWindowUnsafe):
        pg.project_gradient_window(dict(cand, contributorRef="someone@example.com"), rec)
    with pytest.raises(pg.GradientWindowUnsafe):
        pg.project_gradient_window(dict(cand, updateDigest="not-a-digest"), rec)


def _job(kernel, budget=1000, op="rmsnorm"):
    return {"kernelRef": kernel, "targetModel": "llama-3-8b", "device": "cuda", "hardwareRef": "b200", "opRef": op, "budgetSats": budget}


def test_kernel_campaign_and_parity():
    camp = pg.build_campaign("campaign.1", [_job("rmsnorm.v2"), _job("attention.flash.v3", 2500, "attention.flash")])
    assert camp["totalBudgetSats"] == 3500 and len(camp["requests"]) == 2
    with pytest.raises(pg.CampaignError):
        pg.build_campaign("c", [_job("k"), _job("K ")])
    with pytest.raises(pg.CampaignError):
        pg.build_campaign("", [_job("k")])
    with pytest.raises(pg.CampaignError):
        pg.build_campaign("c", [_job("k", 0)])
    rec = lambda kernel, tps, g="g1": {"targetModel": "llama-3-8b", "device": "cuda", "hardwareRef": "b200", "opRef": "rmsnorm", "kernelRef": kernel,
                                      "graphDigest": g, "tokensPerSecond": tps}
    ver = lambda outcome="verified", digest="t1", dev="validator.1", g="g1": {"outcome": outcome, "graphDigest": g, "validatorDeviceRef": dev,
                                                                            "replayedTraceDigest": digest, "rejection": None}
    ok = pg.verify_kernel_parity("rmsnorm", rec("base", 100), rec("fast", 150), ver(), ver())
    assert ok["outcome"] == "accepted" and ok["speedupRatio"] == 1.5
    cases = [(("rmsnorm", rec("base", 100), dict(rec("fast", 150), device="rocm"), ver(), ver()), "target_mismatch"),
             (("swiglu", rec("base", 100), rec("fast", 150), ver(), ver()), "op_mismatch"),
             (("rmsnorm", rec("base", 100), rec("BASE ", 150), ver(), ver()), "kernel_not_optimized"),
             (("rmsnorm", rec("base", 100), rec("fast", 150, "g2"), ver(), ver()), "parity_trace_unbound"),
             (("rmsnorm", rec("base", 100), rec("fast", float("nan")), ver(), ver()), "invalid_throughput"),
             (("rmsnorm", rec("base", 100), rec("fast", 150), ver("rejected"), ver()), "parity_rejected"),
             (("rmsnorm", rec("base", 100), rec("fast", 150), ver(digest="t2"), ver()), "output_parity_mismatch"),
             (("rmsnorm", rec("base", 100), rec("fast", 150), ver(dev="validator.2"), ver()), "output_parity_mismatch"),
             (("rmsnorm", rec("base", 100), rec("fast", 100), ver(), ver()), "no_throughput_improvement")]
    for args, reason in cases:
        v = pg.verify_kernel_parity(*args)
        assert v["outcome"] == "rejected" and v["rejection"]["reason"] == reason, reason
    # replay verdicts of the numeric executor plug straight in
    import json
    from pathlib import Path
    gold = json.loads((Path(__file__).parent / "data" / "tassadar_loop_sum_golden.json").read_text())
    rv = ts.verify_full_replay(gold["model"], gold["steps"], gold["expectedTraceDigest"], "validator.1")
    g = gold["model"]["graph_digest"]
    assert pg.verify_kernel_parity("rmsnorm", rec("base", 100, g), rec("fast", 130, g), rv, rv)["outcome"] == "accepted"
    v2 = dict(ok, optimizedOpRef="attention.flash")
    bad = pg.verify_kernel_parity("attention.flash", dict(rec("base", 100), opRef="attention.flash"), dict(rec("slow", 90), opRef="attention.flash"), ver(), ver())
    slugs = [r["requestedSlug"] for r in camp["requests"]]
    s = pg.settle_campaign(camp, [{"requestedSlug": slugs[0], "budgetSats": 1000, "verdict": ok}, {"requestedSlug": slugs[1], "budgetSats": 2500, "verdict": bad}])
    assert s["ok"] and s["payoutOwedSats"] == 1000 and s["refundedSats"] == 2500 and s["escrowConserved"] and s["rejectionReasonCounts"] == {"no_throughput_improvement": 1}
    s = pg.settle_campaign(camp, [{"requestedSlug": slugs[0], "budgetSats": 900, "verdict": ok}, {"requestedSlug": "ghost", "budgetSats": 1, "verdict": ok},
                                  {"requestedSlug": slugs[0], "budgetSats": 900, "verdict": ok}])
    assert not s["ok"] and {"duplicate:" + slugs[0], "unexpected:ghost", "unsettled:" + slugs[1], "budget:" + slugs[0], "escrow_not_conserved"} <= set(s["discrepancies"])
    s = pg.settle_campaign(camp, [{"requestedSlug": slugs[0], "budgetSats": 1000, "verdict": v2}, {"requestedSlug": slugs[1], "budgetSats": 2500, "verdict": bad}])
    assert "op:" + slugs[0] in s["discrepancies"]
