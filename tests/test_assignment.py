"""The local-inference assignment loop against this package's CPU model server."""
import pytest

from openagents_b200.control import assignment as asg
from openagents_b200.control import node_bridge as nb
from openagents_b200.models.config import TINY_LLAMA
from openagents_b200.models.weights import PLAN_Q8_0, random_weights, save_gguf
from openagents_b200.serve.backend import CpuBackend
from openagents_b200.serve.server import ServedModel, ServerState

NOW = 1_780_000_000.0


def _lease(**kw):
    base = {"schema": asg.LEASE_SCHEMA, "assignmentRef": "assignment.demo.1", "leaseRef": "lease.demo.1", "goal": "say hello",
            "paymentMode": "no-spend", "capabilityRefs": ["capability.psionic.local_inference"], "expiresAt": asg._iso(NOW + 600),
            "psionicQwenRequirements": {"workClass": "local_inference", "mode": "coding_agent", "receiptRefs": ["receipt.preflight.1"]}}
    base.update(kw)
    return base


ROWS = [{"modelRef": nb.MODEL_REFS["small"], "ready": True}]


def test_lease_validation_and_admission():
    assert asg.decode_lease(_lease())["capabilityRefs"] == ["capability.psionic.local_inference"]
    for bad in (dict(_lease(), schema="x"), dict(_lease(), assignmentRef="has space"), dict(_lease(), paymentMode="free"),
                dict(_lease(), expiresAt="soon"), dict(_lease(), psionicQwenRequirements={"workClass": "training", "mode": "coding_agent"})):
        with pytest.raises(asg.LeaseError):
            asg.decode_lease(bad)
    caps = ("capability.psionic.local_inference",)
    ok = asg.compute_admission(asg.decode_lease(_lease()), ROWS, NOW, caps)
    assert ok == {"admitted": True, "blockerRefs": [], "selectedModelRef": nb.MODEL_REFS["small"], "missingCapabilityRefs": []}
    late = asg.compute_admission(asg.decode_lease(_lease(expiresAt=asg._iso(NOW - 1))), ROWS, NOW, caps)
    assert late["blockerRefs"] == ["blocker.assignment.lease_expired"]
    need2b = asg.decode_lease(_lease(psionicQwenRequirements={"workClass": "local_inference", "mode": "requires_2b"}))
    assert asg.compute_admission(need2b, ROWS, NOW, caps)["blockerRefs"] == ["blocker.psionic_qwen35.model_2b_missing"]
    assert asg.compute_admission(asg.decode_lease(_lease()), ROWS, NOW, ())["blockerRefs"] == ["blocker.assignment.capability_not_advertised"]
    assert "blocker.assignment.delegation_invalid" in asg.compute_admission(asg.decode_lease(_lease(delegationInvalid=True)), ROWS, NOW, caps)["blockerRefs"]
    assert asg.bounded_progress_message("  a \n b  ") == "a b" and asg.bounded_progress_message("") == "Assignment progress updated."
    long = asg.bounded_progress_message("x" * 500)
    assert len(long) == asg.PROGRESS_MESSAGE_MAX and long.endswith("...")


def test_full_loop_on_the_local_model_server(tmp_path):
    cfg = TINY_LLAMA.with_(vocab=512, d_model=64, n_heads=2, n_kv_heads=1, head_dim=32, ffn=128)
    p = str(tmp_path / "tiny.gguf")
    save_gguf(p, cfg, random_weights(cfg, 0), PLAN_Q8_0)
    model = ServedModel(nb.MODEL_REFS["small"], CpuBackend.from_gguf(p), None, max_num_seqs=2)
    state = ServerState([model])

    def complete(model_ref, goal, max_tokens):
        r, usage = state.complete(state.model(model_ref), [{"role": "user", "content": goal}], {"max_tokens": max_tokens})
        return model.tok.decode(r.output), usage

    sent = []
    out = asg.run_local_inference_assignment(_lease(), ROWS, complete, lambda k, b: sent.append((k, b)), now=lambda: NOW,
                                             node_capability_refs=("capability.psionic.local_inference",), max_tokens=5)
    kinds = [k for k, _ in sent]
    assert kinds == ["acceptance", "progress", "progress", "progress", "progress", "closeout"]
    seqs = [b["sequence"] for k, b in sent if k == "progress"]
    assert seqs == [1, 2, 3, 4] and [b["status"] for k, b in sent if k == "progress"] == ["accepted", "running", "artifact-ready", "closeout-submitted"]
    c = out["closeout"]
    assert c["status"] == "accepted" and c["settlementState"] == "not_applicable" and c["payoutClaimAllowed"] is False and c["redacted"] is True
    assert c["receiptRefs"][:2] == [nb.BACKEND_REF, "receipt.preflight.1"] and nb.MODEL_REFS["small"] in c["receiptRefs"]
    assert c["resultRefs"][0].startswith("result.sha256.") and c["summaryRefs"] == [f"summary.tokens.exact.{out['usage']['total_tokens']}"]
    last = [b for k, b in sent if k == "progress"][-1]
    assert last["tokensSoFar"] == out["usage"]["total_tokens"] and last["tokenCountKind"] == "exact"
    assert "say hello" not in str(sent[1:])                              # the goal and the answer stay on the node
    # paid lease: a clean run may claim; a progress post the coordinator refuses blocks settlement but not the work
    sent.clear()
    paid = asg.run_local_inference_assignment(_lease(paymentMode="paid"), ROWS, complete, lambda k, b: sent.append((k, b)), now=lambda: NOW,
                                              node_capability_refs=("capability.psionic.local_inference",), max_tokens=3)["closeout"]
    assert paid["settlementState"] == "pending" and paid["payoutClaimAllowed"] is True

    def flaky(kind, body):
        if kind == "progress" and body["status"] == "running":
            raise RuntimeError("progress rejected (409)")
        sent.append((kind, body))
    blocked = asg.run_local_inference_assignment(_lease(paymentMode="paid"), ROWS, complete, flaky, now=lambda: NOW,
                                                 node_capability_refs=("capability.psionic.local_inference",), max_tokens=3)["closeout"]
    assert blocked["status"] == "accepted" and blocked["settlementState"] == "blocked" and blocked["payoutClaimAllowed"] is False
    assert blocked["blockerRefs"] == ["blocker.assignment.progress_or_artifact_rejected", "blocker.assignment.progress_or_artifact_http_409"]
    # rejection, operator cancel, engine failure, lease that ran out during the run
    rej = asg.run_local_inference_assignment(_lease(), [], complete, lambda k, b: None, now=lambda: NOW,
                                             node_capability_refs=("capability.psionic.local_inference",))
    assert rej["accepted"] is False and rej["acceptance"]["denialRef"] == "blocker.psionic_qwen35.qwen35_model_missing"
    kw = dict(now=lambda: NOW, node_capability_refs=("capability.psionic.local_inference",))
    assert asg.run_local_inference_assignment(_lease(), ROWS, complete, lambda k, b: None, should_cancel=lambda: True, **kw)["closeout"]["status"] == "cancelled"

    def boom(*a):
        raise MemoryError("KV cache is out of pages")
    failed = asg.run_local_inference_assignment(_lease(), ROWS, boom, lambda k, b: None, **kw)["closeout"]
    assert failed["status"] == "rejected" and "blocker.assignment.error.MemoryError" in failed["blockerRefs"]
    clock = iter([NOW, NOW, NOW, NOW, NOW, NOW + 700] + [NOW + 700] * 20)
    slow = asg.run_local_inference_assignment(_lease(), ROWS, complete, lambda k, b: None, now=lambda: next(clock),
                                              node_capability_refs=("capability.psionic.local_inference",), max_tokens=2)["closeout"]
    assert slow["status"] == "timed-out"
    run = asg.AssignmentRun(asg.decode_lease(_lease()), lambda k, b: sent.append((k, b)), now=lambda: NOW)
    first = run.closeout("stale")
    n = len(sent)
    assert run.closeout("accepted") is first and len(sent) == n          # idempotent
    model.close()


def test_executor_trace_assignment_runs_the_pinned_workload():
    import json
    import os
    from openagents_b200.control import assignment as asg
    from openagents_b200.oracle import tassadar as tz
    g = json.load(open(os.path.join(os.path.dirname(__file__), "data", "tassadar_loop_sum_golden.json")))
    model = dict(g["model"])
    transit = {k: v for k, v in model.items() if k != "seed_writes"}
    transit["initialChannelWrites"] = model["seed_writes"]
    receipt = tz.run_self_test({"fixtureId": "loop_sum", "model": g["model"], "steps": g["steps"], "expectedTraceDigest": g["expectedTraceDigest"],
                                "expectedModelDigest": "0" * 64})
    caps = [tz.CAPABILITY_REF, receipt["receiptRef"]]

    def lease(expected, kind="tassadar_executor_trace", m=transit):
        return {"schema": asg.LEASE_SCHEMA, "assignmentRef": "assignment.tz.1", "leaseRef": "lease.tz.1", "goal": "replay the pinned workload",
                "paymentMode": "no-spend", "capabilityRefs": [tz.CAPABILITY_REF], "expiresAt": "2099-01-01T00:00:00Z",
                "codingAssignment": {"kind": kind, "tassadar": {"fixtureId": "loop_sum", "model": m, "steps": g["steps"], **({"expectedTraceDigest": expected} if expected else {})}}}
    posts = []
    out = asg.run_tassadar_assignment(lease(g["expectedTraceDigest"]), lambda k, b: posts.append((k, b)), node_capability_refs=caps)
    assert out["accepted"] and out["closeout"]["status"] == "accepted" and out["closeout"]["blockerRefs"] == []
    assert f"result.tassadar_poc.trace_digest.{g['expectedTraceDigest']}" in out["closeout"]["resultRefs"]
    assert out["execution"]["summaryRefs"] == ["summary.tassadar_poc.trace_digest_match"] and [k for k, _ in posts] == ["acceptance", "progress", "progress", "closeout"]
    bad = asg.run_tassadar_assignment(lease("0" * 64), lambda k, b: None, node_capability_refs=caps)
    assert bad["closeout"]["status"] == "rejected" and bad["closeout"]["blockerRefs"] == ["blocker.assignment.tassadar_trace_digest_mismatch"]
    assert bad["closeout"]["payoutClaimAllowed"] is False
    # the capability without its self-test receipt is not admitted; another kind of lease is not this runner's
    unreceipted = asg.run_tassadar_assignment(lease(None), lambda k, b: None, node_capability_refs=[tz.CAPABILITY_REF])
    assert not unreceipted["accepted"] and "blocker.assignment.tassadar_capability_unreceipted" in unreceipted["acceptance"]["blockerRefs"]
    assert asg.tassadar_payload_from({"kind": "coding", "tassadar": {}}) is None
    assert asg.tassadar_payload_from(lease(None)["codingAssignment"])["model"]["seed_writes"] == model["seed_writes"]
    broken = dict(transit)
    broken.pop(next(k for k in broken if k not in ("initialChannelWrites", "graph_digest")))
    refused = asg.execute_tassadar_assignment(asg.decode_lease(lease(None, m=broken)))
    assert refused["status"] == "rejected" and refused["blockerRefs"] == ["blocker.assignment.tassadar_execution_refused"]
