"""Control-plane predicates and state machines (CPU).  One case per rejection reason, in the
style of the reference's own tests (training-durable-checkpoint-seal / standby / curtailment)."""
import dataclasses

import numpy as np
import pytest

from openagents_b200.control import lifecycle as lc
from openagents_b200.control import run_window as rw
from openagents_b200.control import seal
from openagents_b200.control import verification as ver

GOOD = seal.DurableCheckpointSeal("sha256:" + "a" * 64, 2, True, 1024, "content_addressed_object_store", "run.w0",
                                  remote_checkpoint_store_ref="store.r2", remote_checkpoint_object_ref="objects/aa",
                                  readback_rehash_receipt_ref="receipt.readback.aa")


def test_seal_passes_and_each_reason_holds():
    assert seal.evaluate(GOOD).decision == seal.SEAL
    cases = {"checkpoint_digest_not_content_addressed": dict(checkpoint_digest_ref="md5:abc"),
             "storage_class_not_durable_content_addressed": dict(storage_class="single_host_disk"),
             "replication_factor_below_durable_minimum": dict(replication_factor=1),
             "checkpoint_retrieval_not_verified": dict(retrieval_verified=False),
             "remote_checkpoint_store_missing": dict(remote_checkpoint_store_ref=None),
             "remote_checkpoint_object_ref_missing": dict(remote_checkpoint_object_ref=None),
             "readback_rehash_receipt_missing": dict(readback_rehash_receipt_ref=None)}
    for reason, kw in cases.items():
        g = seal.evaluate(dataclasses.replace(GOOD, **kw))
        assert g.decision == seal.HOLD and reason in g.reasons
    assert seal.evaluate_untrusted({"storageClass": "tape"}).decision == seal.HOLD
    ok = seal.evaluate_untrusted({"checkpointDigestRef": "sha256:" + "b" * 64, "replicationFactor": 3,
                                  "retrievalVerified": True, "sizeBytes": 10, "storageClass": "content_addressed_replicated_blob",
                                  "windowRef": "run.w1", "remoteCheckpointStoreRef": "store.x",
                                  "remoteCheckpointObjectRef": "objects/bb", "readbackRehashReceiptRef": "receipt.bb"})
    assert ok.durable


def test_join_ladder_closed_set():
    s = "registered"
    seen = [s]
    for _ in range(4):
        t, r = lc.join_next(s)
        s = lc.join_transition(s, t, r)
        seen.append(s)
    assert seen == ["registered", "qualified", "state_synced", "warmup", "active"]
    s = lc.join_transition("active", "lagged", "join_lifecycle.public.beyond_max_allowed_stale")
    s = lc.join_transition(s, "sync_reentry", "join_lifecycle.public.sync_reentry_started")
    s = lc.join_transition(s, "state_synced", "join_lifecycle.public.reentry_seal_digest_synced")
    assert s == "state_synced"
    with pytest.raises(lc.JoinTransitionError):
        lc.join_transition("registered", "active", "join_lifecycle.public.shadow_work_verified")


def test_staleness_routes_to_reentry_never_rejects():
    assert lc.decide_staleness(5).outcome == "accept"
    d = lc.decide_staleness(6)
    assert d.outcome == "sync_reentry" and d.reason_code and d.effective_max_steps_behind == 5
    d = lc.decide_staleness(3, 5, class_override=2)
    assert d.outcome == "sync_reentry" and d.threshold_source == "verification_class_override"
    with pytest.raises(ValueError):
        lc.decide_staleness(-1)


def test_standby_and_curtailment():
    d = lc.StandbyDispatch("standby.a", "run.x", True, False, True, "run.x.w3", "run.x.w3", 1, 1000)
    assert lc.decide_standby(d) == ("promote_standby", ())
    for kw, reason in ((dict(qualified=False), "standby_not_qualified"), (dict(banned_for_round=True), "standby_banned_for_round"),
                       (dict(bootstrap_seal_verified=False), "bootstrap_seal_not_verified"),
                       (dict(bootstrap_seal_window_ref="run.x.w2"), "bootstrap_seal_window_mismatch"),
                       (dict(live_vacancy_count=0), "no_live_vacancy"), (dict(last_heartbeat_age_ms=120_001), "standby_heartbeat_stale")):
        dec, reasons = lc.decide_standby(dataclasses.replace(d, **kw))
        assert dec == "hold_standby" and reason in reasons
    c = lc.CurtailmentDrill("drill.1", "run.x", True, True, 30_000, True, 300_000, True, True)
    assert lc.decide_curtailment(c)[0] == "drill_passed"
    assert "ack_latency_exceeds_sla" in lc.decide_curtailment(dataclasses.replace(c, ack_latency_ms=30_001))[1]
    assert "halt_latency_exceeds_sla" in lc.decide_curtailment(dataclasses.replace(c, halt_latency_ms=300_001))[1]
    assert "durable_checkpoint_not_sealed_before_halt" in lc.decide_curtailment(dataclasses.replace(c, durable_checkpoint_sealed=False))[1]


def test_run_window_state_machine():
    t = [0.0]
    a = rw.Authority(now=lambda: t[0], lease_ttl_s=10)
    run = a.plan_run("promise.demo", max_allowed_stale=7)
    assert run.max_allowed_stale == 7 and run.seal_publication_cadence_windows == 1
    w = a.plan_window(run.run_ref, 0, 10)
    with pytest.raises(rw.TransitionError):
        a.claim_lease(w.window_ref, "worker.a")          # not active yet
    a.activate_window(w.window_ref)
    l1 = a.claim_lease(w.window_ref, "worker.a")
    assert a.claim_lease(w.window_ref, "worker.a") is l1  # idempotent
    t[0] = 11.0
    assert a.live_leases(w.window_ref) == []              # expired
    # sealing without a durable checkpoint HOLDs (cadence 1 publishes every window)
    _, gate = a.seal_window(w.window_ref, rw.SealMetadata())
    assert gate.decision == seal.HOLD and a._window(w.window_ref).state == "active"
    _, gate = a.seal_window(w.window_ref, rw.SealMetadata(checkpoint_digest_ref=GOOD.checkpoint_digest_ref,
                                                         durable_checkpoint_seal=GOOD))
    assert gate.durable and a._window(w.window_ref).state == "sealed"
    a.reconcile_window(w.window_ref)
    assert a.run_blockers(run.run_ref) == [rw.PLANNED_WITH_RECONCILED_WINDOWS_BLOCKER]
    a.advance_run(run.run_ref, "active")
    assert a.run_blockers(run.run_ref) == []
    with pytest.raises(rw.TransitionError):
        a.advance_run(run.run_ref, "reconciled")
    assert a.last_durable_seal(run.run_ref).window_ref == w.window_ref
    assert a.change_commit_authority(run.run_ref, 0) == 0 and a.change_commit_authority(run.run_ref, 3) == 1
    assert a.projection(run.run_ref)["term"] == 1


def _freivalds_payload(tamper=False):
    rng = np.random.default_rng(0)
    p = ver.DEFAULT_MODULUS
    A, B = rng.integers(0, p, (8, 16)), rng.integers(0, p, (16, 8))
    C = ver.matmul_mod(A, B, p)
    if tamper:
        C = C.copy()
        C[3, 2] = (C[3, 2] + 1) % p
    return {"fieldModulus": p, "leftMatrix": A.tolist(), "rightMatrix": B.tolist(), "claimedProductMatrix": C.tolist(),
            "challengeVector": rng.integers(0, p, 8).tolist(), "rowOpenings": [{"rowRef": "row.0"}], "merkleProofValid": True}


def test_verification_classes():
    assert ver.run_verification_class("freivalds_merkle", _freivalds_payload()).outcome == "Verified"
    v = ver.run_verification_class("freivalds_merkle", _freivalds_payload(tamper=True))
    assert v.outcome == "Rejected" and "FreivaldsMismatch" in v.failure_codes
    bad = _freivalds_payload()
    bad["rowOpenings"] = []
    assert "RowOpeningMissing" in ver.run_verification_class("freivalds_merkle", bad).failure_codes
    bad = _freivalds_payload()
    bad["leftMatrix"][0][0] = -1
    assert "FieldMismatch" in ver.run_verification_class("freivalds_merkle", bad).failure_codes
    bad = _freivalds_payload()
    bad["challengeVector"] = bad["challengeVector"][:-1]
    assert "DimensionMismatch" in ver.run_verification_class("freivalds_merkle", bad).failure_codes
    assert ver.run_verification_class("deterministic_recompute", {"expectedDigestRef": "d.1", "recomputedDigestRef": "d.1"}).outcome == "Verified"
    assert "DigestMismatch" in ver.run_verification_class("deterministic_recompute", {"expectedDigestRef": "d.1", "recomputedDigestRef": "d.2"}).failure_codes
    assert "OutputDigestMissing" in ver.run_verification_class("deterministic_recompute", {}).failure_codes
    tr = {"traceCommitmentDigestRef": "trace.tassadar.commitment.abc", "replayDigestRef": "trace.tassadar.replay.abc",
          "sampledWindow": {"startStep": 0, "endStep": 4}}
    assert ver.run_verification_class("exact_trace_replay", tr).outcome == "Verified"
    tr["replayDigestRef"] = "trace.tassadar.replay.abd"
    assert "ExecutorTraceMismatch" in ver.run_verification_class("exact_trace_replay", tr).failure_codes
    assert ver.run_verification_class("seeded_replication", {"observedScore": 0.99, "minimumScore": 0.95}).outcome == "Verified"
    assert ver.run_verification_class("statistical_cross_check", {"observedScore": 0.5}).outcome == "Rejected"
    assert ver.run_verification_class("nope", {}).failure_codes == ("VerificationClassUnknown",)
    assert ver.REGISTRY["statistical_cross_check"].max_steps_behind_override == 2


def test_challenge_queue_lease_retry_timeout():
    t = [0.0]
    q = ver.ChallengeQueue(now=lambda: t[0], lease_ttl_s=5, retry_budget=2)
    q.enqueue("c.1", "deterministic_recompute", {"expectedDigestRef": "d", "recomputedDigestRef": "d"})
    c = q.claim("validator.a")
    assert c.state == "Leased"
    t[0] = 6
    with pytest.raises(ValueError):
        q.finalize("c.1")
    assert q.items["c.1"].state == "Retrying"
    c = q.claim("validator.b")
    assert q.finalize("c.1").outcome == "Verified" and q.items["c.1"].state == "Verified"
    with pytest.raises(ValueError):
        q.finalize("c.1")
    q.enqueue("c.2", "deterministic_recompute", {})
    q.claim("v")
    t[0] = 20
    q.claim("v")
    t[0] = 40
    q.expire()
    assert q.items["c.2"].state == "TimedOut" and q.items["c.2"].failure_code == "RetryBudgetExhausted"
