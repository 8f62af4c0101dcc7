"""Failure detection and recovery without a GPU fault: gloo ranks on the CPU where a rank leaves between steps or never
joins a collective, the round ledger's ban / preserve / standby-gated abort, the discard-and-reload flow, and the
exhaustive protocol models with their must-fail mutations."""
import os
import socket
import time
from datetime import timedelta

import pytest
import torch

from openagents_b200.control.lifecycle import StandbyDispatch
from openagents_b200.parallel import protocol_model as pm
from openagents_b200.parallel.failure import (CollectiveFailure, HeartbeatBoard, PeerLeft, RoundLedger, check_collectives,
                                              latest_sealed_checkpoint)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


# ---------------------------------------------------------------- protocol models
@pytest.mark.parametrize("world", [2, 3])
def test_protocol_models_pass_and_every_mutation_is_caught(world):
    res = pm.run_all(world=world)
    for name, r in res.items():
        assert r["pass"], (name, r["violation"])
        assert r["mutations"], name
        for mut, m in r["mutations"].items():
            assert m["caught"], f"{name}: mutation {mut} was not caught"


def test_slot_allreduce_model_more_rounds():
    assert pm.slot_allreduce(world=2, rounds=5)
    assert not pm.slot_allreduce(world=2, rounds=5, mutation="single_buffer")


# ---------------------------------------------------------------- round ledger
def _standby(**kw):
    base = dict(standby_contributor_ref="pylon.standby.1", run_ref="run.x", qualified=True, banned_for_round=False,
                bootstrap_seal_verified=True, bootstrap_seal_window_ref="run.x.w3", live_sealed_window_ref="run.x.w3",
                live_vacancy_count=1, last_heartbeat_age_ms=5_000)
    base.update(kw)
    return StandbyDispatch(**base)


def test_round_ledger_bans_preserves_and_gates_the_abort():
    led = RoundLedger("run.x.w4.step12", world=4)
    for r in range(4):
        led.record_result(r, f"grad.mb0.rank{r}")
    led.record_result(2, "grad.mb1.rank2")
    ev = led.on_failure(1, status=3)
    assert ev["decision"] == "abort_round" and ev["reasons"] == ["no_standby"] and ev["bannedForRound"] == [1]
    assert 1 not in ev["preservedResults"] and ev["preservedResults"][2] == ["grad.mb0.rank2", "grad.mb1.rank2"]
    assert not led.may_rejoin(1) and led.may_rejoin(0)
    with pytest.raises(ValueError):
        led.record_result(1, "late")                      # a banned rank contributes nothing more to this round
    assert led.on_failure(3, 3, standby=_standby())["decision"] == "promote_standby"
    held = led.on_failure(0, 3, standby=_standby(last_heartbeat_age_ms=500_000, bootstrap_seal_verified=False))
    assert held["decision"] == "abort_round" and "standby_heartbeat_stale" in held["reasons"]
    assert led.next_round("run.x.w4.step13").may_rejoin(1)      # bans last one round


def test_check_collectives_raises_on_new_timeouts():
    class Heap:
        st = (0, 0)

        def status(self):
            return self.st

    h = Heap()
    assert check_collectives(h, 0) == 0
    h.st = (3, 2)
    with pytest.raises(CollectiveFailure) as e:
        check_collectives(h, 5, since=0)
    assert e.value.status == 3 and e.value.timeouts == 2 and e.value.rank == 5
    assert check_collectives(h, 5, since=2) == 2


def test_latest_sealed_checkpoint_ignores_aborted_saves(tmp_path):
    for step, sealed in ((10, True), (20, True), (30, False)):
        d = tmp_path / f"step{step:08d}"
        d.mkdir()
        (d / "model-rank0.bin").write_bytes(b"x")
        if sealed:
            (d / "manifest.json").write_text("{}")
    assert latest_sealed_checkpoint(str(tmp_path)).endswith("step00000020")
    assert latest_sealed_checkpoint(str(tmp_path / "nope")) is None


# ---------------------------------------------------------------- gloo ranks: a rank leaves between steps / never joins
def _gloo_worker(rank, world, port, mode, out_dir):
    import torch.distributed as dist
    from openagents_b200.train import checkpoint as ck
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=3))
    store = dist.distributed_c10d._get_default_store()
    board = HeartbeatBoard(store, rank, world, ttl_s=30.0)
    state = torch.zeros(8)                   # "model": every step adds the all-reduced rank ids
    ledger = RoundLedger("round.0", world)
    ckpt_root = os.path.join(out_dir, "ckpt")
    events = []
    try:
        for step in range(1, 6):
            if mode == "leave" and rank == 1 and step == 4:
                board.leave(step)            # between steps: nothing of this rank is in flight; it never announces step 4 as alive
                break
            board.beat(step)
            dist.barrier() if step == 1 else None
            try:
                if step > 1:
                    board.wait_peers(step, timeout_s=5.0)     # peers post their heartbeat before they launch: a rendezvous on the host
                if mode == "never_joins" and rank == 1 and step == 4:
                    time.sleep(6.0)          # alive, heartbeat posted, but never enters the collective
                    break
                g = torch.full((8,), float(rank + 1))
                dist.all_reduce(g)           # gloo: ends with an error after the group's 3 s timeout if a rank is missing
                state += g
                ledger.record_result(rank, f"step{step}.rank{rank}")
                if step == 2 and rank == 0:  # seal a checkpoint: shard + manifest, read back and hashed
                    d = os.path.join(ckpt_root, f"step{step:08d}")
                    files = ck.save_shard(d, 0, state.clone(), torch.zeros(8), torch.zeros(8))
                    ck.write_manifest(d, files, run_ref="run.t", window_ref="run.t.w0", step=step, world_size=1, zero_stage=2,
                                      n_total=8, shard=8, term=1, train_config={}, model_config={})
            except PeerLeft as e:
                ev = ledger.on_failure(e.peers[0], 0)
                events.append(("peer_left", step, ev["decision"], ev["bannedForRound"]))
                break
            except Exception as e:           # noqa: BLE001 - the timed-out collective
                ev = ledger.on_failure(1, 3)
                events.append(("collective_failed", step, ev["decision"], type(e).__name__))
                break
        if rank == 0:
            # discard the failed step and go back to the last sealed checkpoint
            man, master, _, _ = ck.load_full(latest_sealed_checkpoint(ckpt_root))
            torch.save({"events": events, "state_before": state.clone(), "restored": master, "step": man["step"],
                        "preserved": ledger.events[-1]["preservedResults"] if ledger.events else {}}, os.path.join(out_dir, "r0.pt"))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:      # noqa: BLE001
            pass


@pytest.mark.parametrize("mode", ["leave", "never_joins"])
def test_gloo_rank_failure_is_detected_and_step_is_discarded(tmp_path, mode):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_gloo_worker, args=(2, port, mode, str(tmp_path)), nprocs=2, join=True)
    r = torch.load(str(tmp_path / "r0.pt"))
    kind, step, decision, _ = r["events"][0]
    assert step == 4 and decision == "abort_round"
    assert kind == ("peer_left" if mode == "leave" else "collective_failed")
    assert r["step"] == 2 and torch.equal(r["restored"], torch.full((8,), 6.0))       # two steps of (1 + 2)
    assert torch.equal(r["state_before"], torch.full((8,), 9.0))                       # step 3 had completed, step 4 never did
    assert r["preserved"][0] == ["step1.rank0", "step2.rank0", "step3.rank0"] and 1 not in r["preserved"]


def test_wait_peers_is_a_rendezvous_on_the_step():
    """The strict pre-launch check: a peer one step behind is waited for, a peer that left raises at once, a peer that never
    arrives raises when the time is up."""
    from openagents_b200.parallel.failure import HeartbeatBoard, PeerLeft

    class Store(dict):
        def set(self, k, v):
            self[k] = v

        def check(self, keys):
            return all(k in self for k in keys)

    store, clock = Store(), [0.0]
    a, b = (HeartbeatBoard(store, r, 2, now=lambda: clock[0]) for r in (0, 1))
    a.beat(3)
    b.beat(2)
    polls = []

    def sleep(dt):                      # the peer posts its step-3 heartbeat while rank 0 is polling
        polls.append(dt)
        clock[0] += dt
        if len(polls) == 3:
            b.beat(3)
    a.wait_peers(3, timeout_s=1.0, sleep=sleep)
    assert len(polls) == 3
    a.check_peers(4)                    # the lenient check lets a peer be one step behind ...
    with pytest.raises(PeerLeft) as e:  # ... the strict one does not, and says so when the time is up
        a.wait_peers(4, timeout_s=0.5, sleep=lambda dt: clock.__setitem__(0, clock[0] + dt))
    assert e.value.reason == "stopped reporting" and e.value.peers == [1]
    b.leave(4)
    with pytest.raises(PeerLeft) as e:
        a.wait_peers(4, timeout_s=100.0, sleep=lambda dt: (_ for _ in ()).throw(AssertionError("must not wait for a peer that left")))
    assert e.value.reason == "left the job"
