"""The gym throughput report measured on this package's own server: live concurrency sweep, lever check, report."""
import threading

from openagents_b200.gateway import benchmark as bm
from openagents_b200.models.config import TINY_LLAMA
from openagents_b200.models.weights import PLAN_Q8_0, random_weights, save_gguf
from openagents_b200.receipts import manifests as mf
from openagents_b200.serve.backend import CpuBackend
from openagents_b200.serve.server import ServedModel, ServerState, serve


def test_live_sweep_report_and_lever_check(tmp_path):
    cfg = TINY_LLAMA.with_(vocab=512, d_model=64, n_heads=2, n_kv_heads=1, head_dim=32, ffn=128)
    p = str(tmp_path / "tiny.gguf")
    save_gguf(p, cfg, random_weights(cfg, 0), PLAN_Q8_0)
    model = ServedModel("tiny", CpuBackend.from_gguf(p), mf.artifact_digest(p), max_num_seqs=4)
    state = ServerState([model])
    httpd = serve(state, "127.0.0.1", 0)
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    base = f"http://127.0.0.1:{httpd.server_address[1]}/v1"
    exp = bm.lever_expectation(4, speculation_below_batch=None)
    status_model = state.status()["models"][0]
    assert status_model["levers"]["max_num_seqs"] == 4
    actual = bm.lever_actual_from_status(status_model, exp)
    assert actual["maxNumSeqs"] == 4 and actual["kvHeadroomGate"]["gateStatus"] == "not_checked"      # the CPU backend reports no pages
    assert bm.lever_mismatches(exp, actual) == []
    assert bm.lever_mismatches(bm.lever_expectation(16), actual) == ["maxNumSeqs", "lowBatchSpeculativeDecoding"]
    gpu_like = dict(status_model, kv={"pages_total": 100, "pages_free": 5})
    tight = bm.lever_actual_from_status(gpu_like, exp)
    assert tight["kvHeadroomGate"]["observedFreeKvCachePercent"] == 5.0 and bm.lever_mismatches(exp, tight) == ["kvHeadroomGate"]
    samples = bm.run_throughput_sweep(base, "tiny", concurrency_ramp=(1, 3), samples_per_concurrency=2, max_tokens=6, actual_levers=actual)
    assert len(samples) == 2 * 1 + 2 * 3 and all(s["status"] == "ok" and s["completionTokens"] == 6 for s in samples)
    assert all(isinstance(s["perceivedTps"], float) and s["totalWallClockMs"] > 0 for s in samples)
    rep = bm.throughput_report({"lane": "psionic", "engine": "openagents_b200", "modelRef": "tiny"}, samples, (1, 3), 2, exp, actual)
    assert rep["okSampleCount"] == 8 and [pt["concurrency"] for pt in rep["points"]] == [1, 3] and rep["levers"]["mismatches"] == []
    assert rep["bestAggregate"]["aggregateTps"] > 0 and rep["degradation"]["reason"] in ("not_detected", "latency_degraded")
    # the three simultaneous requests of a round shared decode batches
    assert model.sched.stats["batch_size_sum"] / model.sched.stats["steps"] > 1.2
    # a model the server does not have: every sample fails, nothing is invented
    bad = bm.run_throughput_sweep(base, "absent", concurrency_ramp=(2,), samples_per_concurrency=1, max_tokens=2)
    assert [s["status"] for s in bad] == ["failed", "failed"] and bad[0]["errorClass"] == "http_404" and bad[0]["perceivedTps"] == bm.NOT_MEASURED
    assert bm.throughput_report({}, bad, (2,), 1)["bestAggregate"] is None
    httpd.shutdown()
    model.close()


def test_matrix_runner_report_and_leaderboard_on_the_fixture_and_a_live_server(tmp_path):
    """Matrix -> samples through a lane seam -> telemetry records -> report -> leaderboard.  The fixture seam is illustrative only
    (never decision grade, so the leaderboard leaves it out); the HTTP seam measures a live server of this package."""
    import threading
    from openagents_b200.gateway import benchmark as bm
    from openagents_b200.gateway import gym
    from openagents_b200.models.config import TINY_LLAMA
    from openagents_b200.models.weights import PLAN_Q8_0, random_weights, save_gguf
    from openagents_b200.serve.backend import CpuBackend
    from openagents_b200.serve.server import ServedModel, ServerState, serve
    shapes = [bm.sequence_shape("short", 24, 6, cacheable_prefix_tokens=8), bm.sequence_shape("real-ish", 40, 4, provenance="recorded")]
    config = {"id": "cfg.test", "targets": [{"lane": "khala", "engine": "b200-native"}, {"lane": "bigpickle", "engine": "provider-native"},
                                           {"lane": "psionic-shard-wan", "engine": "b200-native"}],
              "workloads": ["chat", "opencode-coding-task"], "shapes": shapes, "transports": ["streaming"],
              "sampling": [{"temperature": 0, "reasoningEffort": "low"}], "samplesPerCell": 2}
    rs = bm.run_benchmark(config, bm.FixtureLaneSeam())
    assert rs["cellsExpanded"] == 12 and rs["cellsSkipped"] == 4 and rs["cellsExecuted"] == 8               # the not-yet-available lane is skipped
    assert {r["skippedReason"] for r in rs["runs"] if r["record"] is None} == {"lane_not_yet_available:psionic-shard-wan"}
    rep = bm.build_benchmark_report(rs)
    assert rep["decisionGrade"] is False and rep["illustrativeNotice"].startswith("ILLUSTRATIVE ONLY") and rep["publicSafe"]
    g = {(x["lane"], x["workload"]): x for x in rep["groups"]}
    assert g[("khala", "chat")]["attemptedVerifications"] == 0 and g[("khala", "opencode-coding-task")]["attemptedVerifications"] == 4
    assert g[("khala", "opencode-coding-task")]["toolCallsAttempted"] == 8 and g[("khala", "chat")]["ttftMs"]["sampleCount"] == 4
    assert g[("psionic-shard-wan", "chat")]["executedSamples"] == 0 and g[("psionic-shard-wan", "chat")]["skippedSamples"] == 2
    inp = {"report": rep, "reportRef": "report.fixture", "receiptRef": "receipt.fixture", "candidateRef": "khala.fixture", "environmentRef": "env.test", "coordinatorRef": "coord.a"}
    assert gym.leaderboard_projection([inp])["excludedReports"] == [{"reportRef": "report.fixture", "reason": "not_decision_grade"}]
    assert bm.check_report_public_safety({**rep, "groups": [{"apiKey": "x"}]})["violations"] == ["apikey"]

    cfg = TINY_LLAMA.with_(vocab=512, d_model=64, n_heads=2, n_kv_heads=1, head_dim=32, ffn=128)
    path = str(tmp_path / "m.gguf")
    save_gguf(path, cfg, random_weights(cfg, 0), PLAN_Q8_0)
    httpd = serve(ServerState([ServedModel("tiny", CpuBackend.from_gguf(path), None, max_num_seqs=4)]), "127.0.0.1", 0)
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    try:
        seam = bm.HttpLaneSeam(f"http://127.0.0.1:{httpd.server_address[1]}", "tiny", lanes=("khala",), verify=lambda cell, text: True,
                               cost_msat=lambda p, c: p + 3 * c)
        live_cfg = {**config, "targets": config["targets"][:2], "shapes": shapes[1:], "workloads": ["opencode-coding-task"], "samplesPerCell": 1}
        rs2 = bm.run_benchmark(live_cfg, seam)
        assert rs2["cellsExecuted"] == 1 and rs2["cellsSkipped"] == 1                                          # the fixture-only lane cannot be bought here
        assert [r["skippedReason"] for r in rs2["runs"]] == [None, "lane_fixture_only:bigpickle"]
        rep2 = bm.build_benchmark_report(rs2)
        k = rep2["groups"][0]
        assert rep2["decisionGrade"] is True and k["acceptedOutcomes"] == 1 and k["inputTokens"] > 40 and 1 <= k["outputTokens"] <= 4
        assert k["ttftMs"]["p50"] > 0 and k["totalWallClockMs"]["mean"] >= k["ttftMs"]["p50"] and k["costPerAcceptedOutcomeMsat"] == k["inputTokens"] + 3 * k["outputTokens"]
        board = gym.leaderboard_projection([{**inp, "report": rep2, "reportRef": "report.live", "candidateRef": "khala.b200"}])
        assert board["rowCount"] == 1 and board["rows"][0]["verificationRateBps"] == 10000 and board["rows"][0]["meanWallClockMs"] > 0
    finally:
        httpd.shutdown()
