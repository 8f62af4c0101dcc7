"""Prompt-cache layout, request telemetry, benchmark matrix, throughput report, evidence contract, pilot gate, replica pool."""
import pytest

from openagents_b200.gateway import benchmark as bm
from openagents_b200.gateway import evidence as ev
from openagents_b200.gateway import fabric as fb
from openagents_b200.gateway import prompt_cache as pc
from openagents_b200.gateway import request_telemetry as rt


def test_stable_prompt_layout_and_hashes():
    tagged = [({"role": "user", "content": "hi"}, None), ({"role": "system", "content": "tools"}, "toolSchemas"),
              ({"role": "system", "content": "misc"}, None), ({"role": "system", "content": "you are"}, "identity"),
              ({"role": "assistant", "content": "yo"}, None)]
    lay = pc.assemble_stable_prompt_layout(tagged)
    assert [m["content"] for m in lay["messages"]] == ["you are", "tools", "misc", "hi", "yo"]
    assert lay["stablePrefixText"] == "system:you aresystem:toolssystem:misc"
    assert lay["stablePrefixHash"] == pc.hash_stable_prefix(lay["stablePrefixText"]) and lay["stablePrefixHash"].startswith("prefix:fnv1a32:")
    # the volatile tail does not change the stable prefix hash
    lay2 = pc.assemble_stable_prompt_layout(tagged[1:4] + [({"role": "user", "content": "other"}, None)])
    assert lay2["stablePrefixHash"] == lay["stablePrefixHash"]
    assert pc.hash_cache_affinity_key("") == "cacheaff:fnv1a32:811c9dc5" and pc.hash_cache_affinity_key("a") == "cacheaff:fnv1a32:e40c292c"
    assert pc.canonical_json({"b": [1, {"z": 1, "a": None}], "a": "x"}) == '{"a":"x","b":[1,{"a":null,"z":1}]}'
    t = [{"type": "function", "function": {"name": "zeta", "parameters": {"b": 1, "a": 2}}}, {"name": "alpha"}]
    assert pc.serialize_tool_schemas(t) == pc.serialize_tool_schemas(list(reversed(t))) and pc.serialize_tool_schemas(t).startswith('{"name":"alpha"}')
    key = pc.derive_cache_affinity_key("acct1", session="s9")
    assert key == "acct=acct1sess=s9code="
    assert pc.session_affinity_params(pc.hash_cache_affinity_key(key)) == {"user": pc.hash_cache_affinity_key(key), "x-session-affinity": pc.hash_cache_affinity_key(key)}
    assert pc.reconcile_usage_tokens(10, 5, 18)["unaccountedTokens"] == 3 and not pc.reconcile_usage_tokens(10, 5, 15)["hasUnaccountedTokens"]


def test_request_telemetry_record():
    r = rt.build_record(request_id="r1", requested_model="khala", served_model="llama-8b-int4", route="openagents-network", provider="b200",
                        request_class="interactive_stream", prompt_tokens=100, completion_tokens=11, total_tokens=115, ttft_ms=40.0,
                        generation_wall_clock_ms=500.0, total_wall_clock_ms=540.0, provider_time_ms=530, cost_basis_msat=900, price_msat=1000,
                        quantization={"precision": "int4", "backend": "provider-native", "scope": "weights_only"},
                        speculation={"mode": "none"}, cache_affinity_key_raw="acct=1", fallback_reason=None, region="us")
    assert r["interTokenLatencyMs"] == 50.0 and r["perceivedTps"] == 22.0 and r["unaccountedTokens"] == 4
    assert r["marginBucket"] == "standard" and r["economicsState"] == "measured" and r["cacheAffinityKeyHash"].startswith("cacheaff:")
    assert r["gatewayOverheadMs"] == rt.NOT_MEASURED and "gateway_overhead_not_measured" in r["blockerRefs"]
    assert "fallback_reason_not_reported" not in r["blockerRefs"] and "region_not_measured" not in r["blockerRefs"]
    r2 = rt.build_record(request_id="r2", requested_model="m", served_model="m", route="x", provider="p", request_class="batch",
                         settlement_state="pending", completion_tokens=1, generation_wall_clock_ms=10)
    assert r2["interTokenLatencyMs"] == rt.NOT_MEASURED and r2["economicsState"] == "pending" and "economics_pending" in r2["blockerRefs"]
    assert r2["quantization"]["precision"] == rt.NOT_MEASURED and "fallback_reason_not_reported" in r2["blockerRefs"]
    assert [rt.margin_bucket(c, 100) for c in (120, 100, 95, 70, 10)] == ["negative", "zero", "thin", "standard", "rich"]
    assert rt.measured(-1) == rt.measured(float("nan")) == rt.measured(None) == rt.NOT_MEASURED and rt.measured(0) == 0
    blk = rt.block_from_record(r, "detail.1")
    assert blk["detailRef"] == "detail.1" and blk["ttftMs"] == 40.0 and "priceMsat" not in blk
    with pytest.raises(ValueError):
        rt.build_record(request_id="r", requested_model="m", served_model="m", route="x", provider="p", request_class="vip")


def test_benchmark_matrix():
    shapes = [bm.sequence_shape("chat-1k", 1024, 256, 512, 4), bm.sequence_shape("long-32k", 32768, 512)]
    cfg = {"targets": [{"lane": "pylon-whole-small", "engine": "b200-native", "profile": {"profileRef": "b200.tp1"}}, {"lane": "fireworks", "engine": "provider-native"}],
           "workloads": ["chat", "verifier-run", "long-context-codebase-question"], "shapes": shapes, "transports": ["streaming", "batch"],
           "sampling": [{"temperature": 0, "reasoningEffort": "off"}], "samplesPerCell": 5,
           "workloadShapePairs": [{"workload": "chat", "shapeId": "chat-1k"}, {"workload": "verifier-run", "shapeId": "chat-1k"},
                                  {"workload": "long-context-codebase-question", "shapeId": "long-32k"}]}
    cells = bm.expand_matrix(cfg)
    assert len(cells) == 2 * 3 * 2 and cells[0]["cellId"] == "pylon-whole-small|b200-native|profile:b200.tp1|chat|chat-1k|streaming|t0|roff"
    assert cells[0]["laneAvailability"] == "not_yet_available" and cells[-1]["laneAvailability"] == "available"
    assert bm.expand_matrix(cfg, served={"pylon-whole-small"})[0]["laneAvailability"] == "available"
    assert {c["verificationExpectation"] for c in cells} == {"none", "test_passed", "seeded"} and cells[-1]["candidateRef"] == "fireworks/provider-native"
    assert len(bm.expand_matrix({**cfg, "workloadShapePairs": None})) == 24
    with pytest.raises(ValueError):
        bm.sequence_shape("bad", 10, 1, 20)
    with pytest.raises(ValueError):
        bm.lane_availability("nope")


def test_throughput_report_and_rollout():
    def s(c, itl, tps, status="ok"):
        return {"concurrency": c, "status": status, "ttftMs": 50.0 * c, "totalWallClockMs": 1000.0, "perceivedTps": tps, "interTokenLatencyMs": itl, "completionTokens": 100}
    samples = [s(1, 10, 100), s(1, 11, 95), s(4, 14, 80), s(4, 15, 75), s(16, 40, 30), s(16, 45, 25), s(16, "not_measured", "not_measured", "failed")]
    pts = bm.concurrency_points(samples)
    assert [p["concurrency"] for p in pts] == [1, 4, 16] and pts[0]["aggregateTps"] == 97.5 and pts[2]["aggregateTps"] == 27.5 * 16
    assert pts[2]["failedSamples"] == 1 and pts[2]["okSamples"] == 2 and pts[1]["interTokenLatencyMs"]["p90"] == 15
    assert bm.degradation_point(pts) == {"concurrency": 16, "reason": "latency_degraded"}
    assert bm.degradation_point(pts[:2]) == {"concurrency": None, "reason": "not_detected"}
    assert bm.degradation_point(bm.concurrency_points(samples + [s(4, 1, 1, "quota_limited")]))["reason"] == "quota_limited"
    lev = bm.lever_expectation
    m = lambda n, tps, itl: {"lever": lev(n, "nvfp4"), "concurrency": n, "aggregateTps": tps, "interTokenLatencyP90Ms": itl, "ttftP90Ms": 200}
    sweep = {"sweepRef": "sweep.1"}
    rec = bm.rollout_recommendation([m(2, 100, 20), m(8, 300, 60), m(16, 420, 150)], sweep)
    assert rec["decisionGrade"] and rec["selection"]["maxNumSeqs"] == 8 and rec["selection"]["aggregateTpsLiftPercent"] == pytest.approx(200)
    assert {"name": "--max-num-seqs", "value": "8"} in rec["selection"]["engineFlags"]
    assert bm.rollout_recommendation([m(2, 100, 20), m(8, 90, 60)], sweep)["blockers"] == ["no_measured_throughput_lift"]
    assert bm.rollout_recommendation([m(2, 100, 20), m(8, 300, 160)], sweep)["blockers"] == ["interactive_itl_slo_exceeded"]
    assert set(bm.rollout_recommendation([m(8, 300, 60)], None)["blockers"]) == {"missing_optimization_sweep", "missing_baseline_max_num_seqs_2_measurement"}
    assert bm.rollout_recommendation([m(2, 100, 20), m(8, "not_measured", 60)], sweep)["blockers"] == ["missing_measured_aggregate_tps"]
    run = bm.owner_armed_rollout(rec, "owner.arm.1")
    assert run["status"] == "ready_to_apply" and run["canApplyLiveFlags"] and run["applicationPlan"]["applyMode"] == "owner_armed_manual"
    assert bm.owner_armed_rollout(rec, " ")["blockers"] == ["missing_owner_arm_ref"]
    assert "recommendation_not_decision_grade" in bm.owner_armed_rollout(bm.rollout_recommendation([], sweep), "x")["blockers"]
    assert lev(16)["lowBatchSpeculativeDecoding"]["maxBatchSize"] == 4 and lev(2, speculation_below_batch=None)["lowBatchSpeculativeDecoding"]["policy"] == "disabled"


def test_evidence_contract():
    rec = ev.evidence_record("psionic_evidence.optimizer_1", "optimizer_run", "needs_review", "2026-06-07T02:30:00.000Z", "2026-06-07T02:45:00.000Z",
                             candidateModuleRefs=["candidate_module.v2"], datasetRefs=["dataset.public_eval", "dataset.private_eval_refs"],
                             reviewRefs=["review.operator_required"], promotionProposalRefs=["promotion_proposal.1"])
    assert ev.authority_is_evidence_only(rec["authority"]) and ev.evidence_needs_review(rec)
    pub = ev.project_evidence(rec, "public", "2026-06-07T04:45:00.000Z")
    assert pub["datasetRefs"] == ["dataset.public_eval"] and pub["reviewRefs"] == [] and pub["updatedAtDisplay"] == "2 hours ago"
    assert not pub["promotionAllowed"] and not pub["settlementAllowed"] and not pub["routingMutationAllowed"] and pub["evidenceOnly"]
    team = ev.project_evidence(rec, "team", "2026-06-07T02:45:30.000Z")
    assert team["reviewRefs"] == ["review.operator_required"] and team["datasetRefs"] == ["dataset.public_eval"] and team["updatedAtDisplay"] == "just now"
    assert ev.project_evidence(rec, "operator", "2026-06-09T02:45:00.000Z")["datasetRefs"] == ["dataset.private_eval_refs", "dataset.public_eval"]
    loose = dict(rec, authority=dict(rec["authority"], noRoutingMutation=False))
    assert not ev.authority_is_evidence_only(loose["authority"]) and ev.project_evidence(loose, "public", "2026-06-08T00:00:00Z")["routingMutationAllowed"]
    for bad in ("someone@example.com", "dataset.raw.dump", "run at 2026-06-07T02:30:00", "has space"):
        with pytest.raises(ev.EvidenceUnsafe):
            ev.project_evidence(dict(rec, sourceRefs=[bad]), "public", "2026-06-08T00:00:00Z")
    tr = ev.training_run_evidence("training_run.gpt2_small.1", ["receipt.1"], ["metric.loss"], "2026-06-07T00:00:00Z")
    assert tr["evidenceKind"] == "training_run" and tr["status"] == "completed" and not ev.evidence_needs_review(tr)
    with pytest.raises(ValueError):
        ev.evidence_record("x", "vibes", "draft", "2026-01-01T00:00:00Z")


def _pilot_cfg(**over):
    c = {"ownerArmed": True, "ownerApprovalRef": "approval.owner.1", "endpointRef": "endpoint.pilot.1", "decisionRef": "decision.1",
         "bootLoadEvidenceRef": "evidence.boot.1", "measuredMaxModelLenEvidenceRef": "evidence.len.1", "qualityEvidenceRef": "evidence.quality.1",
         "endpointUrl": "http://127.0.0.1:8000", "bootLoadStatus": "passed", "measuredMaxModelLen": 131072, "qualityParity": "passed"}
    c.update(over)
    return c


def test_pilot_gate():
    tl = {"sampleCount": 20, "providerErrorCount": 0, "toolCallsAttempted": 20, "toolCallsSucceeded": 20, "hallucinatedToolCallCount": 0, "evidenceRef": "evidence.tools.1"}
    tp = {"measuredTps": 61.0, "outputTokens": 4096, "evidenceRef": "evidence.tps.1"}
    go = ev.pilot_result(_pilot_cfg(), tl, tp)
    assert go["decision"] == "go" and go["canRouteCodingLane"] and go["blockerRefs"] == [] and go["throughput"]["speedupVsBaseline"] == pytest.approx(61 / 47)
    assert {"name": "--quantization", "value": "modelopt_fp4"} in go["launchFlags"] and {"name": "--max-model-len", "value": "131072"} in go["launchFlags"]
    no = ev.pilot_result(_pilot_cfg(ownerArmed=False, qualityParity="failed", endpointRef="https://host/secret", model="other/model"),
                         dict(tl, sampleCount=5, toolCallsSucceeded=19), None)
    assert no["decision"] == "no_go" and no["routingOutcome"] == "keep_live_lane"
    assert {"owner_arm_missing", "quality_parity_missing", "endpoint_ref_unsafe", "unsafe_public_ref", "model_mismatch", "tool_loop_sample_count_too_low",
            "tool_loop_missing_tool_calls", "tps_measurement_missing"} <= set(no["blockerRefs"])
    assert "endpoint_ref_missing" not in no["blockerRefs"]
    boot = ev.pilot_result(_pilot_cfg(servingStackFindings=[{"engine": "sglang", "status": "failed_before_endpoint", "failureCode": "sglang_moe_w13_shape_mismatch"}]), tl, tp)
    assert boot["bootLoadStatus"] == "failed" and "boot_load_failed" in boot["blockerRefs"]
    assert "tps_not_finite" in ev.pilot_result(_pilot_cfg(), tl, dict(tp, measuredTps=float("inf")))["blockerRefs"]
    assert "tool_loop_provider_error" in ev.pilot_result(_pilot_cfg(), dict(tl, providerErrorCount=1), tp)["blockerRefs"]


def test_replica_pool():
    S = ev.replica_state
    states = [S("a", warm_state="cold"), S("b", warm_state="warm", inflight=1, max_inflight=4), S("c", health="degraded", warm_state="warm"),
              S("d", warm_state="warm", draining=True), S("e", warm_state="warm", inflight=2, max_inflight=2)]
    assert ev.busy_reason(states[3]) == "draining" and ev.busy_reason(states[4]) == "inflight_full" and ev.busy_reason(S("x", benchmark_reserved=True)) == "benchmark_reserved"
    assert ev.select_replica(states)["replicaId"] == "b"
    assert ev.select_replica(states, "a") == {"replicaId": "a", "busyReasons": [], "fallbackReason": None, "affinityHit": True}
    assert ev.select_replica(states, "e")["fallbackReason"] == "affinity_replica_busy"
    assert ev.select_replica([S("q", queue_depth=3), S("r", queue_depth=1)])["replicaId"] == "r"
    assert ev.select_replica([S("q", observed_ttft_ms=90), S("r", observed_ttft_ms=50)])["replicaId"] == "r"
    full = [S("a", inflight=1), S("b", health="unhealthy")]
    assert ev.select_replica(full)["replicaId"] is None and ev.select_replica(full)["busyReasons"] == ["health_unhealthy", "inflight_full"]
    with pytest.raises(fb.InferenceAdapterError) as e:
        ev.dispatch_to_pool(lambda: full, lambda r: r, policy="overflow_immediately")
    assert e.value.kind == "glm_pool_saturated" and e.value.retryable and e.value.http_status == 503
    slept = []
    with pytest.raises(fb.InferenceAdapterError) as e:
        ev.dispatch_to_pool(lambda: full, lambda r: r, policy="queue_then_429", max_queue_wait_ms=5000, sleep=slept.append)
    assert not e.value.retryable and e.value.http_status == 429 and slept == [1000]
    seq = iter([full, [S("a")]])
    out, meta = ev.dispatch_to_pool(lambda: next(seq), lambda r: f"ran:{r}", policy="queue_then_overflow", sleep=slept.append)
    assert out == "ran:a" and meta["queueWaitMs"] == 250 and meta["saturationPolicy"] == "queue_then_overflow"
    assert ev.default_saturation_policy(True) == "overflow_immediately" and ev.default_saturation_policy(False) == "queue_then_overflow"
    assert ev.route_admission([S("a", max_inflight=2)])["internalStressHeadroomAvailable"] and not ev.route_admission([S("a")])["internalStressHeadroomAvailable"]
    assert ev.route_admission(full)["reason"] == "pool_saturated"
