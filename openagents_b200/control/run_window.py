"""Run / window / lease state machine of the training launcher.

Runs and windows move planned -> active -> sealed -> reconciled; a window is leased to workers,
sealed with staleness / churn / verification-overhead metadata and (optionally) a durable
checkpoint seal, then reconciled.  A window is the unit of merged progress; joiners bootstrap only
from the last durable seal.

Reference: apps/openagents.com/workers/api/src/training-run-window-authority.ts:43-56 (states),
:59-63 (homework kinds), :77 (default max stale 5), :89 (seal cadence 1), :166-172 (seal
metadata), :192-216 (manifest), :219-231 (plan request), :260-264 (lease claim).
"""
from __future__ import annotations

import hashlib
import time
from dataclasses import dataclass, field

from . import seal as seal_mod
from .lifecycle import DEFAULT_MAX_ALLOWED_STALE_STEPS

STATES = ("planned", "active", "sealed", "reconciled")
HOMEWORK_KINDS = ("admin_dispatched_homework", "operator_planned_homework", "auto_starter")
DEFAULT_SEAL_PUBLICATION_CADENCE_WINDOWS = 1
PLANNED_WITH_RECONCILED_WINDOWS_BLOCKER = "blocker.training.run_state_planned_with_reconciled_windows"
_NEXT = {"planned": "active", "active": "sealed", "sealed": "reconciled"}


class TransitionError(ValueError):
    pass


@dataclass
class SealMetadata:
    staleness: dict = field(default_factory=lambda: {"maxStepsBehind": 0, "contributions": []})
    churn: dict = field(default_factory=lambda: {"joined": 0, "left": 0, "events": []})
    verification_overhead: dict = field(default_factory=lambda: {"verificationSeconds": 0.0, "trainingSeconds": 0.0})
    checkpoint_digest_ref: str | None = None
    durable_checkpoint_seal: seal_mod.DurableCheckpointSeal | None = None


@dataclass
class Lease:
    lease_ref: str
    window_ref: str
    worker_ref: str
    claimed_at: float
    expires_at: float
    released: bool = False


@dataclass
class Window:
    window_ref: str
    run_ref: str
    index: int
    state: str = "planned"
    homework_kind: str = "operator_planned_homework"
    base_checkpoint_digest: str | None = None
    start_step: int = 0
    end_step: int = 0
    seal: SealMetadata | None = None
    leases: list[Lease] = field(default_factory=list)


@dataclass
class Run:
    run_ref: str
    promise_ref: str
    state: str = "planned"
    max_allowed_stale: int = DEFAULT_MAX_ALLOWED_STALE_STEPS
    seal_publication_cadence_windows: int = DEFAULT_SEAL_PUBLICATION_CADENCE_WINDOWS
    manifest: dict = field(default_factory=dict)
    windows: list[Window] = field(default_factory=list)
    term: int = 0                       # commit-authority term: bumped whenever the committing rank changes
    commit_authority_rank: int = 0


class Authority:
    """In-memory authority with an injectable clock (tests drive time by hand)."""

    def __init__(self, now=time.time, lease_ttl_s: float = 600.0):
        self.now, self.lease_ttl_s = now, lease_ttl_s
        self.runs: dict[str, Run] = {}

    # ---- runs
    def plan_run(self, promise_ref: str, run_ref: str | None = None, max_allowed_stale: int | None = None,
                 seal_publication_cadence_windows: int | None = None, manifest: dict | None = None) -> Run:
        if not seal_mod.is_public_safe_ref(promise_ref):
            raise ValueError("promiseRef must be a public-safe ref")
        if max_allowed_stale is not None and not 1 <= max_allowed_stale <= 100_000:
            raise ValueError("maxAllowedStale out of range")
        if seal_publication_cadence_windows is not None and not 1 <= seal_publication_cadence_windows <= 10_000:
            raise ValueError("sealPublicationCadenceWindows out of range")
        ref = run_ref or "run." + hashlib.sha256(f"{promise_ref}:{len(self.runs)}".encode()).hexdigest()[:16]
        if ref in self.runs:
            raise ValueError(f"run {ref} exists")
        r = Run(ref, promise_ref, max_allowed_stale=max_allowed_stale or DEFAULT_MAX_ALLOWED_STALE_STEPS,
                seal_publication_cadence_windows=seal_publication_cadence_windows or DEFAULT_SEAL_PUBLICATION_CADENCE_WINDOWS,
                manifest=dict(manifest or {}))
        self.runs[ref] = r
        return r

    def advance_run(self, run_ref: str, to: str) -> Run:
        r = self.runs[run_ref]
        if _NEXT.get(r.state) != to:
            raise TransitionError(f"run {run_ref}: {r.state} -> {to} is not allowed")
        if to in ("sealed", "reconciled") and any(w.state not in ("sealed", "reconciled") for w in r.windows):
            raise TransitionError("every window must be sealed before the run is")
        r.state = to
        return r

    def run_blockers(self, run_ref: str) -> list[str]:
        r = self.runs[run_ref]
        if r.state == "planned" and any(w.state == "reconciled" for w in r.windows):
            return [PLANNED_WITH_RECONCILED_WINDOWS_BLOCKER]
        return []

    def change_commit_authority(self, run_ref: str, rank: int) -> int:
        r = self.runs[run_ref]
        if rank != r.commit_authority_rank:
            r.commit_authority_rank, r.term = rank, r.term + 1
        return r.term

    # ---- windows
    def plan_window(self, run_ref: str, start_step: int, end_step: int, base_checkpoint_digest: str | None = None,
                    homework_kind: str = "operator_planned_homework") -> Window:
        r = self.runs[run_ref]
        if homework_kind not in HOMEWORK_KINDS:
            raise ValueError("unknown homework kind")
        if end_step <= start_step:
            raise ValueError("window must cover at least one step")
        w = Window(f"{run_ref}.w{len(r.windows)}", run_ref, len(r.windows), homework_kind=homework_kind,
                   base_checkpoint_digest=base_checkpoint_digest, start_step=start_step, end_step=end_step)
        r.windows.append(w)
        return w

    def _window(self, window_ref: str) -> Window:
        for r in self.runs.values():
            for w in r.windows:
                if w.window_ref == window_ref:
                    return w
        raise KeyError(window_ref)

    def activate_window(self, window_ref: str) -> Window:
        w = self._window(window_ref)
        if w.state != "planned":
            raise TransitionError(f"window {window_ref}: {w.state} -> active is not allowed")
        w.state = "active"
        return w

    def claim_lease(self, window_ref: str, worker_ref: str) -> Lease:
        w = self._window(window_ref)
        if w.state != "active":
            raise TransitionError("leases are claimed on active windows only")
        t = self.now()
        for l in w.leases:
            if l.worker_ref == worker_ref and not l.released and l.expires_at > t:
                return l                       # idempotent re-claim
        l = Lease(f"{window_ref}.lease{len(w.leases)}", window_ref, worker_ref, t, t + self.lease_ttl_s)
        w.leases.append(l)
        return l

    def live_leases(self, window_ref: str) -> list[Lease]:
        t = self.now()
        return [l for l in self._window(window_ref).leases if not l.released and l.expires_at > t]

    def seal_window(self, window_ref: str, meta: SealMetadata) -> tuple[Window, seal_mod.SealGate | None]:
        """Seal an active window.  When the run publishes a durable seal for this window (cadence),
        the durable-checkpoint predicate must pass, otherwise the window stays active (HOLD)."""
        w = self._window(window_ref)
        if w.state != "active":
            raise TransitionError(f"window {window_ref}: {w.state} -> sealed is not allowed")
        r = self.runs[w.run_ref]
        gate = None
        if (w.index + 1) % r.seal_publication_cadence_windows == 0:
            if meta.durable_checkpoint_seal is None:
                gate = seal_mod.SealGate(seal_mod.HOLD, False, ("durable_checkpoint_seal_missing",))
            else:
                gate = seal_mod.evaluate(meta.durable_checkpoint_seal)
            if not gate.durable:
                return w, gate
        w.seal, w.state = meta, "sealed"
        for l in w.leases:
            l.released = True
        return w, gate

    def reconcile_window(self, window_ref: str) -> Window:
        w = self._window(window_ref)
        if w.state != "sealed":
            raise TransitionError(f"window {window_ref}: {w.state} -> reconciled is not allowed")
        w.state = "reconciled"
        return w

    def last_durable_seal(self, run_ref: str) -> Window | None:
        """The window a joiner bootstraps from."""
        for w in reversed(self.runs[run_ref].windows):
            if w.state in ("sealed", "reconciled") and w.seal and w.seal.durable_checkpoint_seal is not None:
                return w
        return None

    def projection(self, run_ref: str) -> dict:
        r = self.runs[run_ref]
        return {"trainingRunRef": r.run_ref, "state": r.state, "maxAllowedStale": r.max_allowed_stale,
                "sealPublicationCadenceWindows": r.seal_publication_cadence_windows, "term": r.term,
                "commitAuthorityRank": r.commit_authority_rank, "blockerRefs": self.run_blockers(run_ref),
                "windows": [{"windowRef": w.window_ref, "state": w.state, "startStep": w.start_step,
                             "endStep": w.end_step, "checkpointDigestRef": w.seal.checkpoint_digest_ref if w.seal else None}
                            for w in r.windows]}
