"""Failure detection and the collective failure semantics of a training round, on the host.

Device side, every wait in this package is bounded: a kernel that does not see its peer gives up, records
``B200_ERR_TIMEOUT_PEER`` in the heap's control block and returns, so the context stays usable.  This module is what
the host does with that:

* ``HeartbeatBoard``: each rank posts (step, time) to the job's key-value store before it launches a step and
  announces when it leaves; a rank checks its peers BEFORE launching, so a peer that left between steps is found on the
  host and no kernel is launched against it (``PeerLeft``).
* ``check_collectives``: reads a heap's status word after a step and raises ``CollectiveFailure``.
* ``RoundLedger``: the reference's semantics for a failed collective: the failing rank is banned for the rest of
  the round (never promoted back into the round it was ejected from), results that completed before the failure are
  preserved and reported, and the round is aborted only when no standby is admissible (standby-gated abort)
  (apps/openagents.com/workers/api/src/training-standby-dispatch.ts:6-12, 56-88; promotion predicate in
  ``control.lifecycle.decide_standby``).
* ``recover``: discard the failed step and reload the last sealed checkpoint.  The world size is static within a run:
  continuing with fewer ranks means restarting the launcher, which resumes from the same checkpoint and re-shards.

Nothing here faults, traps or hangs a GPU: failures are a rank that raises, leaves or never joins, a message that is
dropped, or a wait that runs out.
"""
from __future__ import annotations

import json
import os
import time
from dataclasses import dataclass, field

from ..control.lifecycle import StandbyDispatch, decide_standby

ERR_TIMEOUT_PEER = 3


class CollectiveFailure(RuntimeError):
    def __init__(self, status: int, timeouts: int, rank: int, detail: str = ""):
        super().__init__(f"rank {rank}: {timeouts} collective wait(s) ran out (status {status}){': ' + detail if detail else ''}")
        self.status, self.timeouts, self.rank = status, timeouts, rank


class PeerLeft(RuntimeError):
    def __init__(self, peers: list[int], reason: str):
        super().__init__(f"peer rank(s) {peers} {reason}")
        self.peers, self.reason = peers, reason


def check_collectives(heap, rank: int, since: int = 0) -> int:
    """Raise ``CollectiveFailure`` if the heap recorded more timed-out waits than ``since``; returns the current count."""
    code, n = heap.status()
    if n > since:
        raise CollectiveFailure(code, n - since, rank)
    return n


class HeartbeatBoard:
    """``store`` is a ``torch.distributed`` store (TCPStore / FileStore / HashStore): set / get / add."""

    def __init__(self, store, rank: int, world: int, ttl_s: float = 90.0, now=time.time, prefix: str = "hb"):
        self.store, self.rank, self.world, self.ttl_s, self.now, self.prefix = store, rank, world, ttl_s, now, prefix

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: int):
        self.store.set(self._key(self.rank), json.dumps({"step": step, "t": self.now(), "state": "alive"}))

    def leave(self, step: int, reason: str = "left"):
        self.store.set(self._key(self.rank), json.dumps({"step": step, "t": self.now(), "state": reason}))

    def read(self, r: int) -> dict | None:
        try:
            if hasattr(self.store, "check") and not self.store.check([self._key(r)]):
                return None
            return json.loads(self.store.get(self._key(r)))
        except Exception:      # noqa: BLE001 - a store that cannot answer is a missing heartbeat
            return None

    def check_peers(self, step: int):
        """Call before launching step ``step``: every peer must be alive, fresh, and at most one step behind."""
        gone, stale = [], []
        for r in range(self.world):
            if r == self.rank:
                continue
            hb = self.read(r)
            if hb is None or hb.get("state") != "alive":
                gone.append(r)
            elif self.now() - hb["t"] > self.ttl_s or hb["step"] < step - 1:
                stale.append(r)
        if gone:
            raise PeerLeft(gone, "left the job")
        if stale:
            raise PeerLeft(stale, "stopped reporting")

    def wait_peers(self, step: int, timeout_s: float = 5.0, poll_s: float = 0.01, sleep=time.sleep):
        """The strict form of ``check_peers``: return only once every peer has posted its heartbeat FOR ``step`` (ranks post it
        before they launch the step, so this is a host-side rendezvous through the store).  A peer that says it left raises
        ``PeerLeft`` at once, a peer that does not reach ``step`` within ``timeout_s`` raises it as "stopped reporting".  With
        ``check_peers`` alone a peer that is one step behind and about to leave passes the check, and its departure is then only
        noticed by the collective's own timeout."""
        deadline = self.now() + timeout_s
        while True:
            gone, behind = [], []
            for r in range(self.world):
                if r == self.rank:
                    continue
                hb = self.read(r)
                if hb is not None and hb.get("state") != "alive":
                    gone.append(r)
                elif hb is None or hb["step"] < step:
                    behind.append(r)
            if gone:
                raise PeerLeft(gone, "left the job")
            if not behind:
                return
            if self.now() > deadline:
                raise PeerLeft(behind, "stopped reporting")
            sleep(poll_s)


@dataclass
class RoundLedger:
    """One training round (an optimizer step, or a window of them) under the collective failure semantics."""
    round_ref: str
    world: int
    banned: set = field(default_factory=set)
    partial_results: dict = field(default_factory=dict)     # rank -> list of result refs that completed before a failure
    events: list = field(default_factory=list)

    def record_result(self, rank: int, result_ref: str):
        """A contribution that has completed (a micro-batch's gradients reduced, a window's update digest): it survives
        a later failure of the round."""
        if rank in self.banned:
            raise ValueError(f"rank {rank} is banned for round {self.round_ref}")
        self.partial_results.setdefault(rank, []).append(result_ref)

    def on_failure(self, failed_rank: int, status: int, standby: StandbyDispatch | None = None) -> dict:
        """Ban the rank for this round, keep what the others completed, and decide: promote an admissible standby into
        the vacancy, or abort the round (discard the step, reload the last sealed checkpoint)."""
        self.banned.add(failed_rank)
        preserved = {r: list(v) for r, v in self.partial_results.items() if r not in self.banned}
        decision, reasons = "abort_round", ("no_standby",)
        if standby is not None:
            verdict, why = decide_standby(standby)
            if verdict == "promote_standby":
                decision, reasons = "promote_standby", ()
            else:
                reasons = tuple(why)
        ev = {"roundRef": self.round_ref, "failedRank": failed_rank, "status": status, "bannedForRound": sorted(self.banned),
              "preservedResults": preserved, "decision": decision, "reasons": list(reasons)}
        self.events.append(ev)
        return ev

    def may_rejoin(self, rank: int) -> bool:
        return rank not in self.banned

    def next_round(self, round_ref: str) -> "RoundLedger":
        """Bans last for one round."""
        return RoundLedger(round_ref, self.world)


def latest_sealed_checkpoint(ckpt_root: str) -> str | None:
    """The newest ``step*`` directory under ``ckpt_root`` whose manifest exists (manifests are written last, after the
    shards were written, renamed into place and read back)."""
    if not os.path.isdir(ckpt_root):
        return None
    best = None
    for d in sorted(os.listdir(ckpt_root)):
        if d.startswith("step") and os.path.exists(os.path.join(ckpt_root, d, "manifest.json")):
            best = os.path.join(ckpt_root, d)
    return best


def recover(trainer, ckpt_root: str) -> dict:
    """Discard the failed step and go back to the last sealed checkpoint.  Returns the manifest it loaded."""
    path = latest_sealed_checkpoint(ckpt_root)
    if path is None:
        raise RuntimeError("no sealed checkpoint to recover from")
    trainer.grads.zero_()
    return trainer.load_checkpoint(path)
