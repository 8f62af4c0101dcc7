"""Tassadar numeric executor: the golden trace digest, replay verdicts, dense lowering, linked composition.
Cases follow packages/tassadar-executor/src/numeric-executor.test.ts and dense-weight-module.test.ts."""
import copy
import json
from pathlib import Path

import pytest

from openagents_b200.oracle import tassadar as ts

GOLD = json.loads((Path(__file__).parent / "data" / "tassadar_loop_sum_golden.json").read_text())


def test_golden_trace_digest_and_outputs():
    t = ts.execute_numeric_model(GOLD["model"], GOLD["steps"])
    assert t["traceDigest"] == GOLD["expectedTraceDigest"]
    assert t["stepCount"] == len(GOLD["steps"]) == 80
    out = ts.collect_interpreter_outputs(t["stepOutputs"])
    assert out["halted"] and out["outputs"] == GOLD["expectedOutputs"] == [15]
    if GOLD.get("expectedFinalRow"):
        assert t["stepOutputs"][-1] == GOLD["expectedFinalRow"]


def test_full_replay_and_window_verdicts():
    m, steps = GOLD["model"], GOLD["steps"]
    ok = ts.verify_full_replay(m, steps, GOLD["expectedTraceDigest"], "device.test")
    assert ok["outcome"] == "verified" and ok["replayedSteps"] == 80
    bad = ts.verify_full_replay(m, steps, "forged", "device.test")
    assert bad["outcome"] == "rejected" and bad["rejection"]["reason"] == "trace_digest_mismatch"
    rows = ts.execute_numeric_model(m, steps)["stepOutputs"][10:13]
    assert ts.verify_window(m, steps, 10, rows, "device.test")["outcome"] == "verified"
    tampered = [list(r) for r in rows]
    tampered[1][1] += 1
    v = ts.verify_window(m, steps, 10, tampered, "device.test")
    assert v["outcome"] == "rejected" and v["rejection"] == {"reason": "row_mismatch", "step": 11}


def test_refusals():
    m = GOLD["model"]
    with pytest.raises(ts.NumericExecutionError) as e:
        ts.execute_numeric_model(m, [[0, 1]])
    assert e.value.kind == "input_arity_mismatch"
    assert ts.verify_full_replay(m, [[0, 1]], "x", "d")["rejection"]["reason"] == "execution_refused"
    big = {"schema_version": 1, "model_id": "m", "graph_digest": "g", "bundle_digest": "", "input_field_count": 1, "slot_count": 2,
           "layer_count": 1, "seed_writes": [], "attention": [], "ffn": [{"value_slot": 0, "gate_slot": 0, "out_slot": 1, "phase": 1}],
           "wiring": [{"out_slot": 0, "bias": 0, "terms": [], "input_field": 0, "phase": 0}], "writes": [], "output_slots": [1]}
    assert ts.execute_numeric_model(big, [[3]])["stepOutputs"] == [[9]]
    assert ts.execute_numeric_model(big, [[-3]])["stepOutputs"] == [[0]]          # gate is max(x, 0)
    with pytest.raises(ts.NumericExecutionError) as e:
        ts.execute_numeric_model(big, [[2 ** 27]])
    assert e.value.kind == "exactness_window_exceeded"
    miss = dict(big, ffn=[], attention=[{"keyed_read": {"channel": 0, "query_slot": 0, "out_slot": 1, "phase": 1}}],
                seed_writes=[[0, 5, 50], [0, 7, 70], [0, 5, 51]])
    assert ts.execute_numeric_model(miss, [[5], [7]])["stepOutputs"] == [[51], [70]]   # latest write wins a tie
    with pytest.raises(ts.NumericExecutionError) as e:
        ts.execute_numeric_model(miss, [[6]])
    assert e.value.kind == "missing_key"


def test_dense_lowering_round_trip_and_validation():
    m = GOLD["model"]
    dense = ts.numeric_model_to_dense_module(m)
    assert dense["dModel"] == m["slot_count"]
    t = ts.execute_dense_module(dense, GOLD["steps"])
    assert t["traceDigest"] == GOLD["expectedTraceDigest"]
    broken = copy.deepcopy(dense)
    broken["ffnBlocks"][0]["wGate"][0][3] = 2
    with pytest.raises(ts.DenseModuleError):
        ts.dense_module_to_numeric_model(broken)
    broken = copy.deepcopy(dense)
    broken["attentionBlocks"][0]["wK"][0][0] = 1
    with pytest.raises(ts.DenseModuleError):
        ts.dense_module_to_numeric_model(broken)
    with pytest.raises(ts.DenseModuleError):
        ts.dense_module_to_numeric_model(dict(dense, moduleKind="other"))


def test_linked_composition():
    m = GOLD["model"]
    composed, place = ts.compose_numeric_models([m, m], "graph.composed")
    assert composed["slot_count"] == 2 * m["slot_count"] and place[1]["projectedOutputStart"] == len(m["output_slots"])
    banks = [{"bankId": f"bank{i}", "model": m, "expectedTraceDigest": GOLD["expectedTraceDigest"], **place[i]} for i in range(2)]
    v = ts.verify_linked_composition(composed, banks, GOLD["steps"])
    assert v["replayVerificationCleared"] and all(c["projectedRowsMatchSource"] for c in v["constituentVerifications"])
    assert v["constituentVerifications"][0]["projectedTraceDigest"] == GOLD["expectedTraceDigest"]
    banks[1]["expectedTraceDigest"] = "wrong"
    v = ts.verify_linked_composition(composed, banks, GOLD["steps"], expected_composed_digest="also wrong")
    assert not v["replayVerificationCleared"]
    assert set(v["blockerRefs"]) == {"blocker.public.tassadar_compiled_module.composed_trace_mismatch",
                                     "blocker.public.tassadar_compiled_module.source_trace_mismatch"}


def test_capability_envelope_needs_a_verified_self_test():
    wl = {"fixtureId": "fixture.loop_sum", "expectedModelDigest": "ab" * 32, "expectedTraceDigest": GOLD["expectedTraceDigest"],
          "model": GOLD["model"], "steps": GOLD["steps"]}
    r = ts.run_self_test(wl)
    assert r["outcome"] == "verified" and r["receiptRef"] == "receipt.tassadar_executor.self_test.v1." + GOLD["expectedTraceDigest"][:16]
    assert "stepOutputs" not in r and "model" not in r
    d = ts.build_capability_declaration(r)
    assert d["declared"] and d["capabilityRefs"] == [ts.CAPABILITY_REF, r["receiptRef"]]
    row = ts.decode_capability_matrix_row(json.loads(json.dumps(d["matrixRow"])))
    assert row["compileReceiptRef"] == "receipt.tassadar_compile.model_digest." + "ab" * 8 and row["posture"] == "execute_exact_or_refuse"
    for k, v in (("posture", "best_effort"), ("compileReceiptRef", "free form"), ("legRefs", ["leg.unknown"]), ("replayReceiptRef", "receipt.x")):
        with pytest.raises(ts.CapabilityShapeError):
            ts.decode_capability_matrix_row({**row, k: v})
    bad = ts.run_self_test({**wl, "expectedTraceDigest": "00" * 32})
    assert bad["outcome"] == "failed" and bad["receiptRef"] is None and bad["refusalDetail"] == "trace_digest_mismatch"
    ref = ts.build_capability_declaration(bad)
    assert not ref["declared"] and ref["refusal"]["kind"] == "self_test_failed"
    refs = [ts.CAPABILITY_REF, "capability.other"]
    assert ts.strip_unreceipted_capability(refs) == ["capability.other"]
    assert ts.strip_unreceipted_capability(["capability.other", r["receiptRef"]]) == ["capability.other"]
    assert ts.strip_unreceipted_capability(refs + [r["receiptRef"]]) == refs + [r["receiptRef"]]


def _reference_fixtures():
    """The reference's own fixture files, when its tree sits beside this repository (or where ``OPENAGENTS_REFERENCE_TREE`` points)."""
    import os
    root = Path(os.environ.get("OPENAGENTS_REFERENCE_TREE") or Path(__file__).resolve().parents[2] / "reference")
    d = root / "packages" / "tassadar-executor" / "fixtures"
    return d if (d / "tassadar-compiled-program-corpus-v1.json").exists() else None


@pytest.mark.skipif(_reference_fixtures() is None, reason="the reference tree is not beside this repository")
def test_every_reference_fixture_replays_digest_for_digest():
    """The compiled-program corpus (backward-branch sum, multiply-add, load/store round trip, factorial countdown, stack comparison
    ladder), the loop-sum fixture and the dense-weight module: trace digest, final row, emitted outputs and halt flag all equal what
    the reference's fixture generator recorded."""
    d = _reference_fixtures()
    corpus = json.loads((d / "tassadar-compiled-program-corpus-v1.json").read_text())
    assert corpus["programCount"] == len(corpus["fixtures"]) >= 5
    for fx in corpus["fixtures"] + [json.loads((d / "tassadar-poc-loop-sum-v1.json").read_text())]:
        tr = ts.execute_numeric_model(fx["model"], fx["steps"])
        out = ts.collect_interpreter_outputs(tr["stepOutputs"])
        assert tr["traceDigest"] == fx["expectedTraceDigest"], fx["fixtureId"]
        assert list(tr["stepOutputs"][-1]) == fx["expectedFinalRow"] and out["outputs"] == fx["expectedOutputs"], fx["fixtureId"]
        if "halted" in fx:
            assert out["halted"] == fx["halted"]
        verdict = ts.verify_full_replay(fx["model"], fx["steps"], fx["expectedTraceDigest"], "validator.local")
        assert verdict["outcome"] == "verified" and verdict["rejection"] is None
    dense = json.loads((d / "tassadar-dense-weight-module-v1.json").read_text())
    tr = ts.execute_dense_module(dense["denseModule"], dense["steps"])
    assert tr["traceDigest"] == dense["expectedTraceDigest"] and list(tr["stepOutputs"][-1]) == dense["expectedFinalRow"]
