"""One distributed training run through the control plane, end to end on the CPU: run and window planning, join ladder and
leases for two contributor nodes, per-step shard gradients with digest commitments (the ordered A1 workload), operator-side
aggregation and validation, cross-node ``deterministic_recompute`` and ``freivalds_merkle`` verification through the challenge
queue, signed coordination records, the durable-seal gate (HOLD on a single local copy, SEAL on a replicated one) and
reconciliation.  The run is the reference's published two-device run, so its digests are known in advance."""
import ctypes

import numpy as np

from openagents_b200.control import coordination as co
from openagents_b200.control import lifecycle as lc
from openagents_b200.control import nostr
from openagents_b200.control import run_window as rw
from openagents_b200.control import seal
from openagents_b200.control import verification as ver
from openagents_b200.oracle import cs336 as c

SEED = c.PUBLISHED_SEED_DIGEST_HEX


class Node:
    """A contributor: computes the gradient of its shard at a given parameter state and commits to it."""

    def __init__(self, name: str, shard: int, cfg: c.A1Config, key: bytes):
        self.name, self.shard, self.cfg, self.key = name, shard, cfg, key
        self.lib = c._ordered_lib()
        self.seqs = np.ascontiguousarray(c.reference_sequences(cfg, SEED, f"train:{shard}", cfg.train_sequences_per_shard), dtype=np.int32)
        self.join_state = "registered"

    def join(self):
        while self.join_state != "active":
            nxt = lc.join_next(self.join_state)
            self.join_state = lc.join_transition(self.join_state, nxt[0], nxt[1])

    def gradient(self, params: np.ndarray, step: int, shard: int | None = None):
        dp, ip = ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_int32)
        seqs = self.seqs if shard in (None, self.shard) else np.ascontiguousarray(
            c.reference_sequences(self.cfg, SEED, f"train:{shard}", self.cfg.train_sequences_per_shard), dtype=np.int32)
        g = np.zeros_like(params)
        cf = self.cfg
        self.lib.b200_a1_shard_gradient(cf.d_model, cf.d_ff, cf.vocabulary_size, cf.sequence_length, params.ctypes.data_as(dp),
                                        seqs.ctypes.data_as(ip), len(seqs), g.ctypes.data_as(dp))
        return g, c.reference_shard_gradient_digest(SEED, step, self.shard if shard is None else shard, g)


def test_one_run_through_the_control_plane():
    cfg = c.A1Config()
    t = [1_780_000_000.0]
    auth = rw.Authority(now=lambda: t[0], lease_ttl_s=600)
    run = auth.plan_run("promise.cs336.a1.real_gradient", max_allowed_stale=5)
    auth.advance_run(run.run_ref, "active")
    nodes = [Node("node.mac", 0, cfg, bytes.fromhex("00" * 31 + "03")), Node("node.linux", 1, cfg, bytes.fromhex("B7E151628AED2A6ABF7158809CF4F3C762E7160F38B4DA56A784D9045190CFEF"))]
    for n in nodes:
        n.join()
        assert n.join_state == "active"
    params = np.ascontiguousarray(c.reference_initial_parameters(cfg, SEED))
    assert c.reference_state_digest(SEED, 0, params) == c.PUBLISHED_INITIAL_STATE_DIGEST_HEX        # both nodes start from the same committed state
    queue = ver.ChallengeQueue(now=lambda: t[0], lease_ttl_s=60, retry_budget=2)
    dp = ctypes.POINTER(ctypes.c_double)
    lib = c._ordered_lib()
    losses, signed = [], []
    windows = [(0, 3), (3, 6)]                                   # two windows of three optimizer steps
    for w_i, (lo, hi) in enumerate(windows):
        w = auth.plan_window(run.run_ref, lo, hi)
        auth.activate_window(w.window_ref)
        for n in nodes:
            auth.claim_lease(w.window_ref, n.name)
        assert len(auth.live_leases(w.window_ref)) == 2
        wrec = co.training_window("net.cs336", w.window_ref, w_i, c.reference_state_digest(SEED, lo, params), hi - lo, "policy.a1", sync_profile="diloco")
        for step in range(lo, hi):
            commits = [n.gradient(params, step) for n in nodes]              # (gradient, digest commitment) per contributor
            # staleness: both contributions are for the current step
            assert all(lc.decide_staleness(0, run.max_allowed_stale).outcome == "accept" for _ in commits)
            nxt = np.zeros_like(params)
            arr = (dp * 2)(*[g.ctypes.data_as(dp) for g, _ in commits])
            lib.b200_a1_sgd_step(params.size, params.ctypes.data_as(dp), arr, 2, cfg.learning_rate, nxt.ctypes.data_as(dp))
            # verification: at the first and last step the OTHER node recomputes each shard's gradient digest
            if step in (0, 5):
                for n, (_, digest) in zip(nodes, commits):
                    other = nodes[1 - n.shard]
                    _, again = other.gradient(params, step, shard=n.shard)
                    queue.enqueue(f"challenge.recompute.s{step}.shard{n.shard}", "deterministic_recompute", {"expectedDigestRef": digest, "recomputedDigestRef": again})
            params = nxt
        val = np.ascontiguousarray(c.reference_sequences(cfg, SEED, "val", cfg.validation_sequence_count), dtype=np.int32)
        losses.append(float(lib.b200_a1_mean_loss(cfg.d_model, cfg.d_ff, cfg.vocabulary_size, cfg.sequence_length, params.ctypes.data_as(dp),
                                                  val.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), len(val))))
        # signed receipts for the window, one per contributor, and the validator's verdicts pointing at them
        for n in nodes:
            rec = nostr.finalize_event(co.training_receipt(wrec, nostr.public_key(n.key).hex(), hi - lo, (hi - lo) * 768, f"artifact.gradients.{w.window_ref}.{n.name}",
                                                           "sha256:" + c.reference_state_digest(SEED, hi, params)), n.key, created_at=int(t[0]))
            assert nostr.verify_event(rec) == [] and co.check_event(rec) == []
            signed.append(rec)
        # seal: a single local copy is HOLD (training may continue), a replicated read-back-verified copy seals
        digest_ref = "sha256:" + c.reference_state_digest(SEED, hi, params)
        _, gate = auth.seal_window(w.window_ref, rw.SealMetadata(checkpoint_digest_ref=digest_ref))
        assert gate.decision == seal.HOLD and auth._window(w.window_ref).state == "active"
        good = seal.DurableCheckpointSeal(checkpoint_digest_ref=digest_ref, replication_factor=2, retrieval_verified=True, size_bytes=params.nbytes,
                                          storage_class="content_addressed_replicated_blob", window_ref=w.window_ref, remote_checkpoint_store_ref="store.a",
                                          remote_checkpoint_object_ref=f"objects/{digest_ref[7:23]}", readback_rehash_receipt_ref=f"receipt.readback.{w_i}")
        _, gate = auth.seal_window(w.window_ref, rw.SealMetadata(checkpoint_digest_ref=digest_ref, durable_checkpoint_seal=good,
                                                                 verification_overhead={"verificationSeconds": 0.4, "trainingSeconds": 2.0}))
        assert gate.durable and auth._window(w.window_ref).state == "sealed"
        auth.reconcile_window(w.window_ref)
        t[0] += 30
    # the commitment of the homework step goes through the Freivalds class as well
    queue.enqueue("challenge.freivalds.final", "freivalds_merkle", {**c.training_step_matrix(SEED), "expectExactProduct": True})
    verdicts = []
    while True:
        ch = queue.claim("validator.recheck")
        if ch is None:
            break
        verdicts.append(queue.finalize(ch.challenge_ref))
    assert len(verdicts) == 5 and all(v.outcome == "Verified" and v.failure_codes == () for v in verdicts)
    # what the run produced is what the reference published for it
    assert losses == [c.PUBLISHED_VALIDATION_LOSSES[3], c.PUBLISHED_VALIDATION_LOSSES[6]]
    assert c.reference_state_digest(SEED, 6, params) == c.PUBLISHED_FINAL_STATE_DIGEST_HEX
    assert auth.run_blockers(run.run_ref) == [] and auth.last_durable_seal(run.run_ref) is not None
    assert len(signed) == 4 and len({e["pubkey"] for e in signed}) == 2
