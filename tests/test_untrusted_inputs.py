"""Records that arrive from outside (a coordinator, a relay, a model server's listing, a client) are decoded by functions that either
answer (a verdict, blocker refs, a list of problems) or raise their own declared error type.  Here each such function is fed a
few hundred seeded mutations of a valid record (fields replaced by values of other types, dropped, nested ones mutated in turn)
and must never leak a TypeError / KeyError / AttributeError from its own bookkeeping."""
import copy
import random

import pytest

from openagents_b200.control import assignment as asg
from openagents_b200.control import coordination as co
from openagents_b200.control import node_bridge as nb
from openagents_b200.control import nostr, seal
from openagents_b200.control import verification as v
from openagents_b200.gateway import fabric as fb
from openagents_b200.receipts import manifests as mf
from openagents_b200.serve import request_schema as schema
from openagents_b200.serve import tools as tl
from openagents_b200.train import assignment_manifest as am

VALUES = [None, True, False, 0, -1, 2 ** 40, 3.5, float("nan"), "", "x", [], [1, 2], {}, {"a": 1}, [[]], [[1, "x"]], [[1, 2], [3]], "sha256:" + "0" * 64]


def mutate(obj, rnd):
    o = copy.deepcopy(obj)
    if isinstance(o, dict) and o:
        for _ in range(rnd.randint(1, 3)):
            k = rnd.choice(list(o) + ["zzz"])
            r = rnd.random()
            if r < 0.6:
                o[k] = rnd.choice(VALUES)
            elif r < 0.8 and k in o:
                del o[k]
            elif k in o and isinstance(o[k], (dict, list)):
                o[k] = mutate(o[k], rnd)
    elif isinstance(o, list) and o:
        i = rnd.randrange(len(o))
        o[i] = rnd.choice(VALUES) if rnd.random() < 0.7 else mutate(o[i], rnd)
    return o


def hammer(fn, seed_obj, allowed=(), n=250, seed=11):
    rnd = random.Random(seed)
    fn(copy.deepcopy(seed_obj))                       # the unmutated record is accepted (or refused) without an internal error
    for _ in range(n):
        m = mutate(seed_obj, rnd)
        try:
            fn(m)
        except allowed:
            pass


def test_verification_classes_answer_on_any_payload():
    fre = {"leftMatrix": [[1, 2], [3, 4]], "rightMatrix": [[5, 6], [7, 8]], "claimedProductMatrix": [[19, 22], [43, 50]], "challengeVector": [1, 2],
           "rowOpenings": [{"row": 0}], "fieldModulus": 2147483647, "expectExactProduct": True}
    assert v.run_verification_class("freivalds_merkle", fre).outcome == "Verified"
    hammer(lambda p: v.run_verification_class("freivalds_merkle", p), fre)
    hammer(lambda p: v.run_verification_class("deterministic_recompute", p), {"expectedDigestRef": "a", "recomputedDigestRef": "a"})
    hammer(lambda p: v.run_verification_class("exact_trace_replay", p),
           {"traceCommitmentDigestRef": "a", "replayDigestRef": "a", "sampledWindow": {"startStep": 0, "endStep": 4}})
    hammer(lambda p: v.run_verification_class("seeded_replication", p), {"observedScore": 0.9, "minimumScore": 0.5})
    # a threshold that is not a number can never be met; a row-opening field that is not a list counts as no openings
    assert v.run_verification_class("seeded_replication", {"observedScore": 0.9, "minimumScore": [1]}).outcome == "Rejected"
    assert v.run_verification_class("statistical_cross_check", {"observedScore": True, "minimumScore": 0}).outcome == "Rejected"
    assert "RowOpeningMissing" in v.run_verification_class("freivalds_merkle", {**fre, "rowOpenings": 7}).failure_codes


def test_signed_events_and_coordination_records():
    ev = nostr.finalize_event({"kind": 1, "tags": [["a", "b"]], "content": "hi"}, bytes(range(1, 33)), 1)
    assert nostr.verify_event(ev) == []
    hammer(nostr.verify_event, ev, n=40)
    w = co.training_window("net.1", "window.1", 0, "sha256:" + "a" * 64, 10, {"minReceipts": 1})
    rc = co.training_receipt(w, "ab" * 32, 10, 1000, "artifact.1", "sha256:" + "b" * 64)
    assert co.check_event(rc) == [] and co.check_event(7) == ["not_an_event"] and co.check_event({"kind": True}) == ["unknown_kind:True"]
    hammer(co.check_event, rc)
    verdict = co.validator_verdict(w, "e" * 64, "ab" * 32, "accepted")
    hammer(lambda m: co.aggregate_window(w, [m], [verdict]), rc, allowed=(co.TrnError,))
    hammer(lambda m: co.aggregate_window(w, [{**rc, "id": "e" * 64}], [m]), verdict, allowed=(co.TrnError,))
    hammer(lambda m: co.aggregate_window(m, [rc], [verdict]), w, allowed=(co.TrnError,))
    # a receipt whose weight tag is garbled contributes nothing instead of stopping the aggregation
    garbled = {**rc, "id": "e" * 64, "tags": [t if t[0] != "weight" else ["weight", "lots"] for t in rc["tags"]]}
    out = co.aggregate_window(w, [garbled], [verdict])
    assert out["admitted"] == [] and out["quorum_met"] is False
    hammer(seal.evaluate_untrusted, {"checkpointRef": "checkpoint.1", "contentDigest": "sha256:" + "a" * 64, "storageClass": "durable",
                                     "replicationCount": 2, "sealedAt": "2026-01-01T00:00:00Z"})


def test_leases_model_rows_candidate_manifests_and_host_listings():
    now = 1_780_000_000.0
    lease = {"schema": asg.LEASE_SCHEMA, "assignmentRef": "assignment.demo.1", "leaseRef": "lease.demo.1", "goal": "say hello", "paymentMode": "no-spend",
             "capabilityRefs": ["capability.psionic.local_inference"], "expiresAt": asg._iso(now + 600),
             "psionicQwenRequirements": {"workClass": "local_inference", "mode": "coding_agent", "receiptRefs": ["receipt.preflight.1"]}}
    rows = [{"modelRef": nb.MODEL_REFS["small"], "ready": True}, {"modelRef": "x", "ready": False}]
    caps = ("capability.psionic.local_inference",)
    assert asg.compute_admission(asg.decode_lease(lease), rows, now, caps)["admitted"] is True
    hammer(lambda m: asg.compute_admission(asg.decode_lease(m), rows, now, caps), lease, allowed=(asg.LeaseError,))
    hammer(lambda r: asg.compute_admission(asg.decode_lease(lease), r, now, caps), rows)
    assert nb.admission_from_model_rows([5, {"modelRef": 7}, {"modelRef": "m", "ready": "yes"}])["admittedModelRefs"] == []
    import test_node_bridge as tn
    hammer(nb.decode_gepa_candidate_manifest, tn._manifest(), allowed=(nb.CandidateManifestError,))
    for text in ("", "NVIDIA B200, 183359, 580.159", "a,b", ",,,,", "NVIDIA B200, lots, x\n\n, ,", "\x00\xff"):
        nb.parse_nvidia_smi(text)
    hammer(fb.normalize_serve_response, {"content": "x", "finishReason": "stop", "usage": {"promptTokens": 1, "completionTokens": 1, "totalTokens": 2},
                                         "servedModel": "m", "servingRunRef": "r", "stages": [{"a": 1}], "parityMode": "exact_greedy_parity",
                                         "parityVerified": True})


def test_training_assignment_manifest_is_refused_not_crashed_on(tmp_path):
    f = tmp_path / "records.jsonl"
    f.write_bytes(b"x" * 64)
    man = am.make_manifest("assignment.1", "sft", [{"role": "records", "path": str(f)}, {"role": "tokenizer", "path": str(f)}], steps=2)
    assert am.validate(man) == []

    def through(m):
        if isinstance(m, dict):          # re-seal, so that the field checks (not the digest) are what stands between a mutation and the lowering
            try:
                m["manifestDigest"] = mf.canonical_digest({k: x for k, x in m.items() if k != "manifestDigest"})
            except (TypeError, ValueError):
                pass
        if not am.validate(m):
            am.launcher_argv(m, str(tmp_path))
            am.verify_inputs(m)
    hammer(through, man, n=600)
    for patch, blocker in (({"nproc": "two"}, "nproc"), ({"optimizer": {"lr": "fast"}}, "optimizer"), ({"model": 5}, "model"), ({"seed": -1}, "seed"),
                           ({"inputs": 7}, "inputs"), ({"budget": [1]}, "budget"), ({"expectedOutputs": None}, "expected_outputs")):
        bad = {**man, **patch}
        bad["manifestDigest"] = mf.canonical_digest({k: x for k, x in bad.items() if k != "manifestDigest"})
        assert f"blocker.training_assignment.{blocker}" in am.validate(bad), (patch, am.validate(bad))


def test_tool_declarations_and_tool_call_text():
    tools = [{"type": "function", "function": {"name": "f", "parameters": {"type": "object", "properties": {"x": {"type": "integer"}}, "required": ["x"]}}}]
    assert schema.tools({"tools": tools}) == tools
    for bad in ([{"type": "function"}], [{"type": "function", "function": {"name": 5}}], [{"type": "retrieval", "function": {"name": "f"}}],
                [{"function": {"name": "f", "parameters": [1]}}], [{"function": "f"}]):
        with pytest.raises(schema.BadRequest, match=r"tools\[0\]"):
            schema.tools({"tools": bad})
    hammer(lambda m: tl.normalize_tool_choice(m.get("c"), m.get("t")), {"c": {"type": "function", "function": {"name": "f"}}, "t": tools}, allowed=(tl.ToolCallError,))
    hammer(lambda m: tl.finish_with_tools('<tool_call>{"name": "f", "arguments": {"x": 1}}</tool_call>', m, "auto", None), tools, allowed=(tl.ToolCallError,))
    for text in ('<tool_call>{"name": 5}</tool_call>', '<tool_call>[1,2]</tool_call>', '<tool_call>{"name": "f", "arguments": "notjson"}</tool_call>', '<tool_call>{',
                 '<tool_call>null</tool_call>', '<tool_call>{"name":"f","arguments":[1]}</tool_call>'):
        msg, finish = tl.finish_with_tools(text, tools, "auto", None)
        assert finish == "stop" and "tool_calls" not in msg           # a malformed block stays text
        with pytest.raises(tl.ToolCallError):
            tl.finish_with_tools(text, tools, "required", None)
