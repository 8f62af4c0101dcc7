"""The quantization evaluation gate, and its samples from two real backends (a checkpoint and its re-quantized copy)."""
import json

from openagents_b200.gateway.quant_gate import compare_backends, decision_grade_blockers, run_quantization_eval_gate


def samples(orig, quant, oc=100, qc=50):
    return [{"taskId": f"t{i}", "originalVerified": o, "quantizedVerified": q, "originalCostBasisMsat": oc, "quantizedCostBasisMsat": qc}
            for i, (o, q) in enumerate(zip(orig, quant))]


def test_gate_decisions():
    held = run_quantization_eval_gate(samples([1] * 8 + [0] * 2, [1] * 8 + [0] * 2), "weights_only")
    assert held["passed"] and held["reason"] == "accepted_rate_held" and held["costPerAcceptedImprovementFrac"] == 0.5 and not held["decisionGrade"]
    hundred = [1] * 100
    small_drop = run_quantization_eval_gate(samples(hundred, [1] * 99 + [0]), "weights_only")
    assert small_drop["passed"] and small_drop["reason"] == "cost_per_accepted_improved_offsets_drop" and abs(small_drop["acceptedRateDeltaAbs"] + 0.01) < 1e-12
    no_win = run_quantization_eval_gate(samples(hundred, [1] * 99 + [0], oc=100, qc=95), "weights_only")
    assert not no_win["passed"] and no_win["reason"] == "accepted_rate_dropped_without_cost_win"
    big = run_quantization_eval_gate(samples(hundred, [1] * 90 + [0] * 10, qc=1), "weights_only")
    assert not big["passed"] and big["reason"] == "accepted_rate_dropped_beyond_bound"         # no cost win offsets a drop this large
    assert run_quantization_eval_gate([], "weights_only")["reason"] == "no_comparison_samples"
    assert run_quantization_eval_gate(samples([0, 0], [1, 1]), "weights_only")["reason"] == "no_baseline_accepted_outcomes"
    kv = run_quantization_eval_gate(samples([1, 1], [1, 1]), "kv_cache")
    assert not kv["passed"] and kv["reason"] == "aggressive_scope_requires_ack" and kv["aggressiveScope"]
    assert run_quantization_eval_gate(samples([1, 1], [1, 1]), "kv_cache", aggressive_scope_ack=True)["passed"]
    loose = run_quantization_eval_gate(samples(hundred, [1] * 95 + [0] * 5), "weights_only", policy={"maxAcceptedRateDropAbs": 0.1})
    assert loose["passed"]


def test_decision_grade_needs_complete_evidence():
    ev = {"schemaVersion": "openagents.khala.real-quant-sweep-evidence.v1", "evidenceRef": "evidence.q.1", "ownerApprovalRef": "approval.1", "workloadRef": "workload.1",
          "originalModelId": "m.bf16", "quantizedModelId": "m.q4k", "originalPrecision": "unquantized", "quantizedPrecision": "int4", "quantizationBackend": "provider-native",
          "quantizationBackendVersion": "1", "sampleCount": 2, "acceptanceVerifierRef": "verifier.1", "latencyEvidenceRef": "latency.1", "costEvidenceRef": "cost.1",
          "publicSafeEvidenceRefs": ["public.1"]}
    ok = run_quantization_eval_gate(samples([1, 1], [1, 1]), "weights_only", decision_grade=True, real_sweep_evidence=ev)
    assert ok["decisionGrade"] and ok["realSweepEvidenceRef"] == "evidence.q.1" and ok["decisionGradeBlockers"] == []
    assert decision_grade_blockers(None, 2) == ["real_sweep_evidence_missing"]
    bad = {**ev, "ownerApprovalRef": " ", "quantizedPrecision": "unquantized", "sampleCount": 3, "publicSafeEvidenceRefs": []}
    assert decision_grade_blockers(bad, 2) == ["owner_approval_ref_missing", "quantized_precision_not_reduced", "same_precision_compared",
                                               "public_safe_evidence_refs_missing", "sample_count_mismatch"]
    r = run_quantization_eval_gate(samples([1, 1], [1, 1]), "weights_only", decision_grade=True, real_sweep_evidence=bad)
    assert r["passed"] and not r["decisionGrade"] and r["realSweepEvidenceRef"] is None


def test_samples_from_a_checkpoint_and_its_requantized_copy(tmp_path, capsys):
    """bf16 checkpoint -> ``gguf quantize --plan q4_k`` -> both served by the CPU backend -> gate samples."""
    from openagents_b200.gguf.__main__ import main as gguf_main
    from openagents_b200.models.config import TINY_LLAMA
    from openagents_b200.models.weights import PLAN_BF16, random_weights, save_gguf
    from openagents_b200.serve.backend import open_backend
    from openagents_b200.serve.generation import ByteTokenizer
    cfg = TINY_LLAMA.with_(vocab=512, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512)
    src, dst = str(tmp_path / "a.gguf"), str(tmp_path / "q.gguf")
    save_gguf(src, cfg, random_weights(cfg, 0), PLAN_BF16)
    assert gguf_main(["quantize", src, dst, "--plan", "q4_k", "--quiet"]) == 0
    assert json.loads(capsys.readouterr().out)["worstRelativeRmsError"] < 0.12
    orig, quant = open_backend(src, "cpu"), open_backend(dst, "cpu")
    tok = ByteTokenizer(cfg.vocab)
    # the answers the original gives are the reference: the original is then right by construction, the copy where it agrees
    prompts = ["hello", "abc", "the cat", "12345"]
    items = []
    for p in prompts:
        orig.begin(1, tok.encode(p))
        out, feed = [], tok.encode(p)
        for _ in range(3):
            nxt = int(orig.forward([1], [feed])[0].argmax())
            out.append(nxt)
            feed = [nxt]
        orig.end(1)
        items.append({"prompt": p, "answer": tok.decode(out)})
    s = compare_backends(orig, quant, tok, items, max_new_tokens=3)
    assert len(s) == 4 and all(x["originalVerified"] for x in s) and all(x["quantizedCostBasisMsat"] <= x["originalCostBasisMsat"] for x in s)
    g = run_quantization_eval_gate(s, "weights_only")
    assert g["originalAcceptedRate"] == 1.0 and g["sampleCount"] == 4 and g["reason"] in ("accepted_rate_held", "accepted_rate_dropped_beyond_bound")
