"""The local-inference part of a node's assignment runner: lease -> admission -> accept -> run -> progress -> closeout.

A coordinator offers a node a lease (assignment ref, lease ref, goal, payment mode, capability refs, expiry and, for
local inference, the requirements block: work class, task mode, optionally a required model).  The node decides admission
from its own model rows, accepts or rejects with blocker refs, runs the work on its model server, reports numbered
progress events with bounded messages and exact token counts, and closes out with a redacted record whose settlement
fields follow the payment mode (a no-spend lease can never carry a payout claim).  Everything that leaves the node is a
ref or a count; prompts and outputs stay local.

Restates the Psionic-relevant parts of apps/pylon/src/assignment.ts: lease and requirement types :97-122, acceptance
:130-138, progress :140-156, closeout :191-211, bounded progress message :338-346, admission :1291-1397, the no-spend run
loop :1912-2465.  Model selection and receipt refs come from ``node_bridge`` (``admit_inference_lease``,
``closeout_receipt_refs``).  Transport is injected: ``post(kind, body)`` stands for the coordinator's HTTP API.
"""
from __future__ import annotations

import re
import time
from datetime import datetime, timezone

from . import node_bridge as nb

LEASE_SCHEMA = "openagents.pylon.assignment_lease.v0.3"
PROGRESS_SCHEMA = "openagents.pylon.assignment_progress.v0.3"
CLOSEOUT_SCHEMA = "openagents.pylon.assignment_closeout.v0.3"
PROGRESS_MESSAGE_MAX = 240
PROGRESS_STATUSES = ("accepted", "running", "artifact-ready", "proof-ready", "closeout-submitted")
CLOSEOUT_STATUSES = ("accepted", "rejected", "cancelled", "timed-out", "stale")
_SAFE_REF = re.compile(r"^[A-Za-z0-9][A-Za-z0-9_.:/-]*$")


class LeaseError(ValueError):
    pass


def _iso(t: float) -> str:
    return datetime.fromtimestamp(t, timezone.utc).strftime("%Y-%m-%dT%H:%M:%S.") + f"{int(t * 1000) % 1000:03d}Z"


def _parse_iso(s: str) -> float:
    return datetime.fromisoformat(s.replace("Z", "+00:00")).timestamp()


def unique_refs(refs) -> list[str]:
    out = []
    for r in refs:
        r = (r or "").strip()
        if r and r not in out:
            out.append(r)
    return out


def bounded_progress_message(value: str, fallback: str = "Assignment progress updated.") -> str:
    msg = re.sub(r"\s+", " ", value or "").strip() or fallback
    return msg if len(msg) <= PROGRESS_MESSAGE_MAX else msg[: PROGRESS_MESSAGE_MAX - 3].rstrip() + "..."


def decode_lease(obj) -> dict:
    """Validate what the coordinator sent; refs must be public-safe tokens."""
    if not isinstance(obj, dict) or obj.get("schema") != LEASE_SCHEMA:
        raise LeaseError("lease.schema")
    for k in ("assignmentRef", "leaseRef", "goal", "expiresAt"):
        if not isinstance(obj.get(k), str) or not obj[k].strip():
            raise LeaseError(f"lease.{k}")
    for k in ("assignmentRef", "leaseRef"):
        if not _SAFE_REF.match(obj[k]):
            raise LeaseError(f"lease.{k}.unsafe")
    if obj.get("paymentMode") not in ("no-spend", "paid"):
        raise LeaseError("lease.paymentMode")
    try:
        _parse_iso(obj["expiresAt"])
    except ValueError:
        raise LeaseError("lease.expiresAt")
    req = obj.get("psionicQwenRequirements")
    if req is not None:
        if not isinstance(req, dict) or req.get("workClass") != "local_inference" or req.get("mode") not in nb.TASK_MODES:
            raise LeaseError("lease.psionicQwenRequirements")
    caps = obj.get("capabilityRefs")
    return {**obj, "capabilityRefs": [c for c in caps if isinstance(c, str)] if isinstance(caps, list) else []}


def compute_admission(lease: dict, model_rows, now: float, node_capability_refs=(), delegation_valid: bool = True) -> dict:
    """Accept only what this node can do now: lease not expired, delegation chain valid, every required capability
    advertised, and, for local inference, a ready model that satisfies the task mode."""
    blockers = []
    if _parse_iso(lease["expiresAt"]) <= now:
        blockers.append("blocker.assignment.lease_expired")
    if lease.get("delegationInvalid") or not delegation_valid:
        blockers.append("blocker.assignment.delegation_invalid")
    missing = [c for c in lease["capabilityRefs"] if c not in node_capability_refs]
    if missing:
        blockers.append("blocker.assignment.capability_not_advertised")
    selected = None
    req = lease.get("psionicQwenRequirements")
    if req is not None:
        adm = nb.admit_inference_lease(req, nb.admission_from_model_rows(model_rows))
        blockers += adm["blockerRefs"]
        selected = adm["selectedModelRef"] if adm["admitted"] else None
    blockers = unique_refs(blockers)
    return {"admitted": not blockers, "blockerRefs": blockers, "selectedModelRef": selected, "missingCapabilityRefs": missing}


class AssignmentRun:
    """One accepted lease.  ``post(kind, body)`` sends ``acceptance`` / ``progress`` / ``closeout`` to the coordinator and
    may raise; a rejected progress post is recorded as a blocker and does not stop the work."""

    def __init__(self, lease: dict, post, now=time.time):
        self.lease, self.post, self.now = lease, post, now
        self.sequence = 0
        self.started = now()
        self.tokens = 0
        self.blockers: list[str] = []
        self.artifacts: list[str] = []
        self.proofs: list[str] = []
        self.closed: dict | None = None

    def accept(self, admission: dict) -> dict:
        a = self.lease
        ok = admission["admitted"]
        rec = {"ok": True, "accepted": ok, "assignmentRef": a["assignmentRef"], "leaseRef": a["leaseRef"],
               "statusRef": f"status.assignment.{'accepted' if ok else 'rejected'}", "blockerRefs": list(admission["blockerRefs"])}
        if not ok:
            rec["denialRef"] = admission["blockerRefs"][0]
        self.post("acceptance", rec)
        return rec

    def progress(self, status: str, message: str, artifact_refs=(), proof_refs=(), tokens_so_far: int | None = None,
                 last_event: str | None = None) -> dict:
        if status not in PROGRESS_STATUSES:
            raise ValueError(f"progress status must be one of {PROGRESS_STATUSES}")
        self.sequence += 1
        self.artifacts = unique_refs([*self.artifacts, *artifact_refs])
        self.proofs = unique_refs([*self.proofs, *proof_refs])
        rec = {"schema": PROGRESS_SCHEMA, "assignmentRef": self.lease["assignmentRef"], "leaseRef": self.lease["leaseRef"],
               "sequence": self.sequence, "status": status, "message": bounded_progress_message(message),
               "artifactRefs": list(self.artifacts), "proofRefs": list(self.proofs), "observedAt": _iso(self.now()),
               "elapsedMs": int((self.now() - self.started) * 1000), "phase": "runtime_active"}
        if tokens_so_far is not None:
            rec["tokensSoFar"], rec["tokenCountKind"] = int(tokens_so_far), "exact"
        if last_event:
            rec["lastProgressEvent"] = last_event
        try:
            self.post("progress", rec)
        except Exception as e:      # noqa: BLE001 - the coordinator refusing an update must not lose the work done so far
            m = re.search(r"\((\d{3})\)", str(e))
            self.blockers = unique_refs([*self.blockers, "blocker.assignment.progress_or_artifact_rejected",
                                         f"blocker.assignment.progress_or_artifact_http_{m.group(1)}" if m else None])
        return rec

    def closeout(self, status: str, receipt_refs=(), result_refs=(), summary_refs=(), extra_blockers=()) -> dict:
        """Idempotent: a second call returns the first record and posts nothing."""
        if self.closed is not None:
            return self.closed
        if status not in CLOSEOUT_STATUSES:
            raise ValueError(f"closeout status must be one of {CLOSEOUT_STATUSES}")
        paid = self.lease["paymentMode"] == "paid"
        blockers = unique_refs([*self.blockers, *extra_blockers])
        good = status == "accepted" and not blockers
        rec = {"schema": CLOSEOUT_SCHEMA, "assignmentRef": self.lease["assignmentRef"], "leaseRef": self.lease["leaseRef"], "status": status,
               "paymentMode": self.lease["paymentMode"],
               "settlementState": ("pending" if good else "blocked") if paid else "not_applicable",
               "payoutClaimAllowed": bool(paid and good), "artifactRefs": list(self.artifacts), "blockerRefs": blockers, "buildRefs": [],
               "closeoutRefs": [f"closeout.{self.lease['assignmentRef']}"], "previewRefs": [], "proofRefs": list(self.proofs),
               "receiptRefs": unique_refs(receipt_refs), "resultRefs": unique_refs(result_refs), "summaryRefs": unique_refs(summary_refs),
               "testRefs": [], "redacted": True, "completedAt": _iso(self.now())}
        self.post("closeout", rec)
        self.closed = rec
        return rec


def run_local_inference_assignment(lease_obj, model_rows, complete, post, now=time.time, node_capability_refs=(), max_tokens: int = 256,
                                   should_cancel=lambda: False) -> dict:
    """The whole loop for one offered lease.  ``complete(model_ref, goal, max_tokens) -> (text, usage)`` is the local model
    server (usage = OpenAI usage object).  Returns the closeout record (or the rejection).  The answer itself never leaves:
    the closeout carries a digest ref of it."""
    import hashlib
    lease = decode_lease(lease_obj)
    run = AssignmentRun(lease, post, now)
    adm = compute_admission(lease, model_rows, now(), node_capability_refs)
    acc = run.accept(adm)
    if not acc["accepted"]:
        return {"accepted": False, "acceptance": acc}
    run.progress("accepted", f"Lease accepted; model {adm['selectedModelRef'] or 'n/a'}.", last_event="lease_accepted")
    if should_cancel():
        return {"accepted": True, "closeout": run.closeout("cancelled", extra_blockers=["blocker.assignment.cancelled_by_operator"])}
    run.progress("running", "Local inference started.", tokens_so_far=0, last_event="runtime_started")
    try:
        text, usage = complete(adm["selectedModelRef"], lease["goal"], max_tokens)
    except Exception as e:      # noqa: BLE001
        return {"accepted": True, "closeout": run.closeout("rejected", extra_blockers=["blocker.assignment.local_inference_failed",
                                                                                        f"blocker.assignment.error.{type(e).__name__}"])}
    if _parse_iso(lease["expiresAt"]) <= now():
        return {"accepted": True, "closeout": run.closeout("timed-out", extra_blockers=["blocker.assignment.lease_expired_during_run"])}
    total = int(usage["total_tokens"])
    digest = "result.sha256." + hashlib.sha256(text.encode()).hexdigest()[:32]
    run.progress("artifact-ready", "Answer produced locally.", artifact_refs=[digest], tokens_so_far=total, last_event="answer_ready")
    receipts = nb.closeout_receipt_refs(lease.get("psionicQwenRequirements"), nb.admission_from_model_rows(model_rows))
    run.progress("closeout-submitted", "Closeout submitted.", tokens_so_far=total, last_event="closeout")
    return {"accepted": True, "closeout": run.closeout("accepted", receipt_refs=receipts, result_refs=[digest],
                                                       summary_refs=[f"summary.tokens.exact.{total}"]), "usage": usage}


# ---------------------------------------------------------------- executor-trace assignments (assignment.ts:678-790)
TASSADAR_TRACE_JOB_KINDS = ("tassadar_executor_trace", "tassadar_executor_trace_homework")      # packages/tassadar-executor/src/lane.ts:4-6


def tassadar_payload_from(assignment) -> dict | None:
    """The embedded workload of an executor-trace lease, or None when the lease is something else.  The dispatch renames
    the model's ``seed_writes`` to ``initialChannelWrites`` so that it passes the public-projection scanner; the executor's
    own field name is restored here."""
    if not isinstance(assignment, dict) or assignment.get("kind") not in TASSADAR_TRACE_JOB_KINDS:
        return None
    t = assignment.get("tassadar")
    if not isinstance(t, dict) or "model" not in t or not isinstance(t.get("steps"), list):
        return None
    model = t["model"]
    if isinstance(model, dict) and "seed_writes" not in model and "initialChannelWrites" in model:
        model = {k: v for k, v in model.items() if k != "initialChannelWrites"}
        model["seed_writes"] = t["model"]["initialChannelWrites"]
        t = {**t, "model": model}
    return t


def execute_tassadar_assignment(lease: dict, now=time.time) -> dict | None:
    """Run the lease's digest-pinned numeric-model workload on this node and report what it computed: accepted when the
    trace digest equals the dispatched expectation (or none was given), rejected on a mismatch or when the executor refuses
    the model.  Exact-replay verification is a validator's job on another device; this only reports."""
    import hashlib
    from ..oracle import tassadar as tz
    payload = tassadar_payload_from(lease.get("codingAssignment"))
    if payload is None:
        return None

    def ref(prefix, text):
        return f"{prefix}.{hashlib.sha256(text.encode()).hexdigest()[:24]}"

    run_ref = ref("run.pylon.tassadar_executor_trace", f"{lease['leaseRef']}:{payload.get('fixtureId', 'workload')}:{_iso(now())}")
    try:
        trace = tz.execute_numeric_model(payload["model"], payload["steps"])
    except Exception as e:      # noqa: BLE001 - a typed refusal of the model (window overflow, malformed wiring) becomes a rejected closeout
        fail = ref("proof.pylon.tassadar_executor_trace.refused", f"{lease['leaseRef']}:{type(e).__name__}:{e}")
        return {"artifactRefs": [], "blockerRefs": ["blocker.assignment.tassadar_execution_refused"], "buildRefs": [run_ref],
                "message": "Tassadar executor-trace workload refused with a typed execution error.", "previewRefs": [], "proofRefs": [fail],
                "resultRefs": ["result.tassadar_poc.execution_refused"], "runRefs": [run_ref], "status": "rejected",
                "summaryRefs": ["summary.tassadar_poc.execution_refused"], "testRefs": [fail]}
    out = tz.collect_interpreter_outputs(trace["stepOutputs"])
    digest = trace["traceDigest"]
    want = payload.get("expectedTraceDigest")
    ok = want is None or want == digest
    halted = "true" if out["halted"] else "false"
    proof = ref("proof.pylon.tassadar_executor_trace", f"{lease['assignmentRef']}:{digest}:{trace['stepCount']}")
    msg = (f"Tassadar executor-trace workload executed: {trace['stepCount']} steps, halted={halted}, {len(out['outputs'])} output(s), trace digest "
           f"{digest[:16]}... matches the dispatched expectation." if ok else
           "Tassadar executor-trace workload executed but the trace digest does not match the dispatched expectation.")
    return {"artifactRefs": [f"artifact.tassadar_poc.trace_digest.{digest}"], "blockerRefs": [] if ok else ["blocker.assignment.tassadar_trace_digest_mismatch"],
            "buildRefs": [run_ref], "message": bounded_progress_message(msg), "previewRefs": [], "proofRefs": [proof],
            "resultRefs": [f"result.tassadar_poc.trace_digest.{digest}", f"result.tassadar_poc.step_count.{trace['stepCount']}", f"result.tassadar_poc.halted.{halted}"],
            "runRefs": [run_ref], "status": "accepted" if ok else "rejected",
            "summaryRefs": ["summary.tassadar_poc.trace_digest_match" if ok else "summary.tassadar_poc.trace_digest_mismatch"], "testRefs": [proof]}


def run_tassadar_assignment(lease_obj, post, now=time.time, node_capability_refs=()) -> dict:
    """Lease -> admission (the executor capability must be advertised WITH its self-test receipt) -> accept -> run -> closeout."""
    from ..oracle import tassadar as tz
    lease = decode_lease(lease_obj)
    run = AssignmentRun(lease, post, now)
    adm = compute_admission(lease, [], now(), node_capability_refs)
    if tz.CAPABILITY_REF in lease["capabilityRefs"] and not tz.has_receipted_capability(list(node_capability_refs)):
        adm = {**adm, "admitted": False, "blockerRefs": unique_refs([*adm["blockerRefs"], "blocker.assignment.tassadar_capability_unreceipted"])}
    acc = run.accept(adm)
    if not acc["accepted"]:
        return {"accepted": False, "acceptance": acc}
    run.progress("running", "Executor-trace workload started.", last_event="runtime_started")
    res = execute_tassadar_assignment(lease, now)
    if res is None:
        return {"accepted": True, "closeout": run.closeout("rejected", extra_blockers=["blocker.assignment.tassadar_payload_missing"])}
    run.progress("proof-ready", res["message"], artifact_refs=res["artifactRefs"], proof_refs=res["proofRefs"], last_event="trace_digest_ready")
    return {"accepted": True, "execution": res,
            "closeout": run.closeout(res["status"], result_refs=res["resultRefs"], summary_refs=res["summaryRefs"], extra_blockers=res["blockerRefs"])}
