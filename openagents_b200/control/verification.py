"""Training verification classes and the challenge queue.

Five pluggable classes decide whether a contribution is accepted: ``freivalds_merkle`` (checks
A(Br) == Cr mod p against a committed product, optionally the exact product), ``deterministic_recompute``
(digest equality), ``exact_trace_replay`` (trace digest equality over a sampled window) and the two
threshold classes ``statistical_cross_check`` / ``seeded_replication``.  Challenges move
Queued -> Leased -> (Retrying ->) Verified | Rejected | TimedOut.

Reference: apps/openagents.com/workers/api/src/training-verification.ts:21-27 (classes), :30-37
(states), :48-63 (failure codes), :428-516 (Freivalds), :518-551 (recompute), :553-597 (trace
replay), :609-632 (threshold), :634-694 (registry with per-class staleness override).  The mod-p
product it checks is the one of cs336-a1-homework-workload.ts:209-221 (p = 2^31 - 1, :20).
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field

import numpy as np

CLASSES = ("deterministic_recompute", "exact_trace_replay", "freivalds_merkle", "seeded_replication",
           "statistical_cross_check")
STATES = ("Queued", "Leased", "Retrying", "Verified", "Rejected", "TimedOut")
TERMINAL = ("Verified", "Rejected", "TimedOut")
DEFAULT_MODULUS = 2_147_483_647


@dataclass(frozen=True)
class Verdict:
    class_name: str
    outcome: str                       # "Verified" | "Rejected"
    failure_codes: tuple[str, ...]
    challenge_ref: str
    public_details: dict = field(default_factory=dict)


def _matrix(x):
    try:
        a = np.asarray(x, dtype=np.int64)
    except (TypeError, ValueError):
        return None
    return a if a.ndim == 2 and a.shape[0] > 0 and a.shape[1] > 0 else None


def matvec_mod(m: np.ndarray, v: np.ndarray, p: int) -> np.ndarray:
    """(m @ v) mod p with Python integers, so products up to p^2 * n never overflow."""
    return np.array([sum(int(a) * int(b) for a, b in zip(row, v)) % p for row in m], dtype=np.int64)


def matmul_mod(a: np.ndarray, b: np.ndarray, p: int) -> np.ndarray:
    return np.stack([matvec_mod(a, b[:, j], p) for j in range(b.shape[1])], axis=1)


def verify_freivalds_merkle(payload: dict, challenge_ref: str = "challenge.local") -> Verdict:
    p = payload.get("fieldModulus", DEFAULT_MODULUS)
    p = p if isinstance(p, int) and p > 0 else DEFAULT_MODULUS
    left, right, claimed = (_matrix(payload.get(k)) for k in ("leftMatrix", "rightMatrix", "claimedProductMatrix"))
    try:
        r = np.asarray(payload.get("challengeVector", []), dtype=np.int64).reshape(-1)
    except (TypeError, ValueError):
        r = np.zeros(0, dtype=np.int64)
    codes = []
    if left is None or right is None or claimed is None:
        codes.append("DimensionMismatch")
    elif left.shape[1] != right.shape[0] or claimed.shape != (left.shape[0], right.shape[1]):
        codes.append("DimensionMismatch")
    cells = [a for a in (left, right, claimed) if a is not None] + [r]
    if any(((c < 0) | (c >= p)).any() for c in cells if c.size):
        codes.append("FieldMismatch")
    if claimed is not None and r.size != claimed.shape[1] and "DimensionMismatch" not in codes:
        codes.append("DimensionMismatch")
    openings = payload.get("rowOpenings") if isinstance(payload.get("rowOpenings"), (list, tuple)) else []
    if len(openings) == 0:
        codes.append("RowOpeningMissing")
    if payload.get("merkleProofValid") is False:
        codes.append("MerkleProofInvalid")
    if not codes:
        lhs = matvec_mod(left, matvec_mod(right, r, p), p)
        rhs = matvec_mod(claimed, r, p)
        if not np.array_equal(lhs, rhs):
            codes.append("FreivaldsMismatch")
        elif payload.get("expectExactProduct") is True and not np.array_equal(matmul_mod(left, right, p), claimed):
            codes.append("FreivaldsMismatch")
    return Verdict("freivalds_merkle", "Verified" if not codes else "Rejected", tuple(codes), challenge_ref,
                   {"fieldModulus": p, "rowOpeningCount": len(openings)})


def freivalds_check_cuda(left, right, claimed, r, p: int = DEFAULT_MODULUS, exact: bool = False, device="cuda:0") -> dict:
    """The arithmetic of ``verify_freivalds_merkle`` on the GPU for matrices too large to check comfortably on the host:
    ``A (B r) == C r (mod p)`` with three exact mat-vecs and, with ``exact``, the full product.  Inputs are integer arrays
    of residues in ``[0, p)``; the answer is bit-identical to the host check (``matvec_mod`` / ``matmul_mod``)."""
    import torch
    from ..ops import cuda_ops as ops
    if not 2 <= p <= 2 ** 31 - 1:
        raise ValueError("the device check needs a modulus below 2^31")
    A, B, C, rv = (torch.as_tensor(np.asarray(a, dtype=np.int64)).to(torch.int32).to(device).contiguous() for a in (left, right, claimed, r))
    if A.shape[1] != B.shape[0] or C.shape != (A.shape[0], B.shape[1]) or rv.numel() != C.shape[1]:
        return {"verified": False, "code": "DimensionMismatch", "mismatchedRows": None}
    lhs = ops.modp_matvec(A, ops.modp_matvec(B, rv, p), p)
    rhs = ops.modp_matvec(C, rv, p)
    bad = int(ops.count_mismatch(lhs, rhs).item())
    out = {"verified": bad == 0, "code": None if bad == 0 else "FreivaldsMismatch", "mismatchedRows": bad}
    if exact and bad == 0:
        cells = int(ops.count_mismatch(ops.modp_matmul(A, B, p), C).item())
        out.update(verified=cells == 0, code=None if cells == 0 else "FreivaldsMismatch", mismatchedCells=cells)
    return out


def verify_deterministic_recompute(payload: dict, challenge_ref: str = "challenge.local") -> Verdict:
    expected = payload.get("expectedDigestRef", payload.get("outputDigestRef"))
    actual = payload.get("recomputedDigestRef")
    codes = []
    if not isinstance(expected, str) or not isinstance(actual, str):
        codes.append("OutputDigestMissing")
    elif expected != actual:
        codes.append("DigestMismatch")
    return Verdict("deterministic_recompute", "Verified" if not codes else "Rejected", tuple(codes), challenge_ref,
                   {"digestRef": expected if isinstance(expected, str) else "digest.missing"})


def _trace_comparable(ref: str) -> str:
    for prefix in ("trace.tassadar.commitment.", "trace.tassadar.replay."):
        if ref.startswith(prefix):
            return ref[len(prefix):]
    return ref


def verify_exact_trace_replay(payload: dict, challenge_ref: str = "challenge.local") -> Verdict:
    expected, actual = payload.get("traceCommitmentDigestRef"), payload.get("replayDigestRef")
    win = payload.get("sampledWindow") if isinstance(payload.get("sampledWindow"), dict) else {}
    codes = []
    if not isinstance(expected, str) or not isinstance(actual, str) or \
            not isinstance(win.get("startStep"), (int, float)) or not isinstance(win.get("endStep"), (int, float)):
        codes.append("OutputDigestMissing")
    elif _trace_comparable(expected) != _trace_comparable(actual):
        codes.append("ExecutorTraceMismatch")
    return Verdict("exact_trace_replay", "Verified" if not codes else "Rejected", tuple(codes), challenge_ref,
                   {"sampledWindowRef": payload.get("sampledWindowRef", "trace.window.redacted")})


def _verify_threshold(class_name: str, payload: dict, challenge_ref: str) -> Verdict:
    obs = payload.get("observedScore")
    thr = payload.get("minimumScore", 1)
    num = lambda x: isinstance(x, (int, float)) and not isinstance(x, bool) and np.isfinite(x)      # noqa: E731
    ok = num(obs) and num(thr) and obs >= thr
    return Verdict(class_name, "Verified" if ok else "Rejected", () if ok else ("StatisticalThresholdFailed",),
                   challenge_ref, {"observedScore": obs if num(obs) else None, "threshold": thr if num(thr) else None})


@dataclass(frozen=True)
class Registration:
    class_name: str
    default_sampling_policy: str        # "per_contribution" | "aggregate"
    failure_codes: tuple[str, ...]
    max_steps_behind_override: int | None
    verify: object


REGISTRY = {
    "freivalds_merkle": Registration("freivalds_merkle", "per_contribution",
                                     ("DimensionMismatch", "FieldMismatch", "FreivaldsMismatch", "MerkleProofInvalid",
                                      "RowOpeningMissing"), None, verify_freivalds_merkle),
    "deterministic_recompute": Registration("deterministic_recompute", "per_contribution",
                                            ("DigestMismatch", "OutputDigestMissing"), None, verify_deterministic_recompute),
    "exact_trace_replay": Registration("exact_trace_replay", "per_contribution",
                                       ("ExecutorTraceMismatch", "OutputDigestMissing"), None, verify_exact_trace_replay),
    "statistical_cross_check": Registration("statistical_cross_check", "aggregate", ("StatisticalThresholdFailed",), 2,
                                            lambda p, c="challenge.local": _verify_threshold("statistical_cross_check", p, c)),
    "seeded_replication": Registration("seeded_replication", "aggregate", ("StatisticalThresholdFailed",), 3,
                                       lambda p, c="challenge.local": _verify_threshold("seeded_replication", p, c)),
}


def run_verification_class(class_name: str, payload: dict, challenge_ref: str = "challenge.local") -> Verdict:
    reg = REGISTRY.get(class_name)
    if reg is None:
        return Verdict(class_name, "Rejected", ("VerificationClassUnknown",), challenge_ref)
    return reg.verify(payload, challenge_ref)


# ---------------------------------------------------------------- challenge queue
@dataclass
class Challenge:
    challenge_ref: str
    class_name: str
    payload: dict
    state: str = "Queued"
    attempts: int = 0
    lease_expires_at: float = 0.0
    validator_ref: str | None = None
    verdict: Verdict | None = None
    failure_code: str | None = None


class ChallengeQueue:
    def __init__(self, now=time.time, lease_ttl_s: float = 60.0, retry_budget: int = 3):
        self.now, self.lease_ttl_s, self.retry_budget = now, lease_ttl_s, retry_budget
        self.items: dict[str, Challenge] = {}

    def enqueue(self, challenge_ref: str, class_name: str, payload: dict) -> Challenge:
        c = Challenge(challenge_ref, class_name, payload)
        self.items[challenge_ref] = c
        return c

    def claim(self, validator_ref: str) -> Challenge | None:
        self.expire()
        for c in self.items.values():
            if c.state in ("Queued", "Retrying"):
                c.state, c.validator_ref = "Leased", validator_ref
                c.attempts += 1
                c.lease_expires_at = self.now() + self.lease_ttl_s
                return c
        return None

    def expire(self):
        """Leases past their deadline go back to Retrying, or TimedOut once the budget is spent."""
        t = self.now()
        for c in self.items.values():
            if c.state == "Leased" and c.lease_expires_at <= t:
                if c.attempts >= self.retry_budget:
                    c.state, c.failure_code = "TimedOut", "RetryBudgetExhausted"
                else:
                    c.state, c.failure_code = "Retrying", "LeaseExpired"

    def finalize(self, challenge_ref: str) -> Verdict:
        c = self.items[challenge_ref]
        if c.state in TERMINAL:
            raise ValueError("ChallengeAlreadyTerminal")
        if c.state != "Leased" or c.lease_expires_at <= self.now():
            self.expire()
            raise ValueError("LeaseExpired")
        c.verdict = run_verification_class(c.class_name, c.payload, challenge_ref)
        c.state = c.verdict.outcome
        return c.verdict
