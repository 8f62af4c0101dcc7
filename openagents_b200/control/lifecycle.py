"""Participant lifecycle predicates of the training control plane: the join ladder, staleness
routing, standby promotion and the curtailment drill.  All are pure functions that fail toward
HOLD / re-entry, never toward silently trusting a participant.

Reference: apps/openagents.com/workers/api/src/pylon-join-lifecycle.ts:17-25 (states), :56-93
(closed transition set); training-staleness-acceptance.ts:18-31 (beyond ``maxAllowedStale`` routes
to sync re-entry, never a bare reject), :75-95 (decision union);
training-standby-dispatch.ts:39 (120 s heartbeat bound), :56-88 (descriptor and reasons);
training-curtailment-drill.ts:42,49 (30 s ack, 300 s halt), :66-99 (descriptor).
"""
from __future__ import annotations

from dataclasses import dataclass

# ---------------------------------------------------------------- join ladder
JOIN_STATES = ("registered", "qualified", "state_synced", "warmup", "active", "lagged", "sync_reentry")

JOIN_TRANSITIONS = (
    ("registered", "qualified", "join_lifecycle.public.qualification_gate_passed"),
    ("qualified", "state_synced", "join_lifecycle.public.durable_seal_digest_synced"),
    ("state_synced", "warmup", "join_lifecycle.public.warmup_started"),
    ("warmup", "active", "join_lifecycle.public.shadow_work_verified"),
    ("active", "lagged", "join_lifecycle.public.beyond_max_allowed_stale"),
    ("lagged", "sync_reentry", "join_lifecycle.public.sync_reentry_started"),
    ("sync_reentry", "state_synced", "join_lifecycle.public.reentry_seal_digest_synced"),
)


class JoinTransitionError(ValueError):
    pass


def join_transition(state: str, to: str, reason: str) -> str:
    """Apply one edge of the ladder; anything outside the closed set raises."""
    if (state, to, reason) not in JOIN_TRANSITIONS:
        raise JoinTransitionError(f"no transition {state} -> {to} with reason {reason}")
    return to


def join_next(state: str) -> tuple[str, str] | None:
    for f, t, r in JOIN_TRANSITIONS:
        if f == state:
            return t, r
    return None


# ---------------------------------------------------------------- staleness routing
DEFAULT_MAX_ALLOWED_STALE_STEPS = 5
MAX_STALENESS_STEPS_BEHIND = 100_000
REENTRY_REASON = "training.staleness.public.beyond_max_allowed_stale"


@dataclass(frozen=True)
class StalenessDecision:
    outcome: str                     # "accept" | "sync_reentry"
    steps_behind: int
    effective_max_steps_behind: int
    threshold_source: str            # "run_config" | "verification_class_override"
    reason_code: str | None = None


def decide_staleness(steps_behind: int, run_max_allowed_stale: int = DEFAULT_MAX_ALLOWED_STALE_STEPS,
                     class_override: int | None = None) -> StalenessDecision:
    """A contribution more than the effective bound behind the sealed head goes to sync re-entry."""
    for v, lo in ((steps_behind, 0), (run_max_allowed_stale, 1)):
        if not isinstance(v, int) or v < lo or v > MAX_STALENESS_STEPS_BEHIND:
            raise ValueError("staleness values must be bounded integers")
    bound, source = run_max_allowed_stale, "run_config"
    if class_override is not None:
        if not isinstance(class_override, int) or class_override < 1 or class_override > MAX_STALENESS_STEPS_BEHIND:
            raise ValueError("class override must be a bounded positive integer")
        bound, source = class_override, "verification_class_override"
    if steps_behind > bound:
        return StalenessDecision("sync_reentry", steps_behind, bound, source, REENTRY_REASON)
    return StalenessDecision("accept", steps_behind, bound, source)


# ---------------------------------------------------------------- standby promotion
MAX_STANDBY_HEARTBEAT_STALENESS_MS = 120_000


@dataclass(frozen=True)
class StandbyDispatch:
    standby_contributor_ref: str
    run_ref: str
    qualified: bool
    banned_for_round: bool
    bootstrap_seal_verified: bool
    bootstrap_seal_window_ref: str
    live_sealed_window_ref: str
    live_vacancy_count: int
    last_heartbeat_age_ms: int


def decide_standby(d: StandbyDispatch) -> tuple[str, tuple[str, ...]]:
    """("promote_standby" | "hold_standby", reasons)."""
    reasons = []
    if not d.qualified:
        reasons.append("standby_not_qualified")
    if d.banned_for_round:
        reasons.append("standby_banned_for_round")
    if not d.bootstrap_seal_verified:
        reasons.append("bootstrap_seal_not_verified")
    if d.bootstrap_seal_window_ref != d.live_sealed_window_ref:
        reasons.append("bootstrap_seal_window_mismatch")
    if d.live_vacancy_count < 1:
        reasons.append("no_live_vacancy")
    if d.last_heartbeat_age_ms > MAX_STANDBY_HEARTBEAT_STALENESS_MS:
        reasons.append("standby_heartbeat_stale")
    return ("promote_standby" if not reasons else "hold_standby"), tuple(reasons)


# ---------------------------------------------------------------- curtailment drill
MAX_CURTAILMENT_ACK_LATENCY_MS = 30_000
MAX_CURTAILMENT_HALT_LATENCY_MS = 300_000


@dataclass(frozen=True)
class CurtailmentDrill:
    drill_ref: str
    run_ref: str
    scheduled: bool
    signal_acknowledged: bool
    ack_latency_ms: int
    halt_completed: bool
    halt_latency_ms: int
    durable_checkpoint_sealed: bool
    resume_verified: bool


def decide_curtailment(d: CurtailmentDrill) -> tuple[str, tuple[str, ...]]:
    """("drill_passed" | "drill_incomplete", reasons)."""
    reasons = []
    if not d.scheduled:
        reasons.append("drill_not_scheduled")
    if not d.signal_acknowledged:
        reasons.append("signal_not_acknowledged")
    elif d.ack_latency_ms > MAX_CURTAILMENT_ACK_LATENCY_MS:
        reasons.append("ack_latency_exceeds_sla")
    if not d.halt_completed:
        reasons.append("halt_not_completed")
    elif d.halt_latency_ms > MAX_CURTAILMENT_HALT_LATENCY_MS:
        reasons.append("halt_latency_exceeds_sla")
    if not d.durable_checkpoint_sealed:
        reasons.append("durable_checkpoint_not_sealed_before_halt")
    if not d.resume_verified:
        reasons.append("resume_not_verified")
    return ("drill_passed" if not reasons else "drill_incomplete"), tuple(reasons)
