"""Tassadar ALM numeric executor, replay verdicts, dense-weight modules and linked compositions.

A numeric model is portable data: phase-ordered rows over a residual vector of ``slot_count``
numbers, executed once per input step.

* wiring row - ``residual[out] = bias + input_field + sum(coefficient * residual[slot])``
* keyed read - hard-max "parabolic" attention over the points written to a channel: score
  ``2 q k - k^2`` is maximal where ``k == q``; equal scores go to the latest write; a best point whose
  key differs from the query is a ``missing_key`` refusal
* cumulative sum - a per-channel accumulator
* gated FFN row - ``residual[out] = residual[value] * max(residual[gate], 0)``
* after the rows, the step's writes append ``(key, value)`` points to their channels

Every value must stay inside +-2^53 (doubles are exact there) or the run is refused.  The trace
digest is SHA-256 over ``"tassadar_alm_trace|" + graph_digest`` and, per step, ``"|row|"`` followed by
the output slots as little-endian signed 64-bit integers; it must match the digest of the other
implementations byte for byte.

Reference: packages/tassadar-executor/src/numeric-executor.ts:14 (window), :55-69 (model), :138-153
(digest), :159-275 (execution: attention :213-240, cumulative sum :241-249, FFN :250-257);
src/replay.ts (full and window verdicts); src/dense-weight-module-runtime.ts:171-281 (lowering with
one-hot validation); src/linked-dense-module-runtime.ts:565 (composition verification).
"""
from __future__ import annotations

import hashlib
import math
import re
import struct

EXACT_WINDOW = 9_007_199_254_740_992           # 2^53
EXECUTOR_ID = "tassadar.alm_numeric_executor.b200.v1"
REPLAY_CLASS_ID = "exact_trace_replay.alm_numeric.v1"
DENSE_MODULE_KIND = "tassadar_alm_dense_weight_module.v1"
LINKED_MODULE_KIND = "tassadar_alm_linked_dense_module.v1"
_B = "blocker.public.tassadar_compiled_module."


class NumericExecutionError(Exception):
    def __init__(self, kind: str, step: int, detail: str):
        super().__init__(f"{kind} at step {step}: {detail}")
        self.kind, self.step, self.detail = kind, step, detail


class DenseModuleError(Exception):
    def __init__(self, field: str, detail: str):
        super().__init__(f"{field}: {detail}")
        self.field = field


def digest_trace_rows(graph_digest: str, rows) -> str:
    h = hashlib.sha256()
    h.update(b"tassadar_alm_trace|")
    h.update(graph_digest.encode())
    for row in rows:
        h.update(b"|row|")
        for v in row:
            h.update(struct.pack("<q", int(v)))
    return h.hexdigest()


def _check(value: float, step: int) -> float:
    if abs(value) > EXACT_WINDOW:
        raise NumericExecutionError("exactness_window_exceeded", step, f"value {value} left the 2^53 exactness window")
    return value


def execute_numeric_model(model: dict, steps) -> dict:
    points: dict[int, list] = {}
    acc: dict[int, float] = {}
    order = 0

    def push(channel, key, value):
        nonlocal order
        points.setdefault(channel, []).append((float(key), float(value), order))
        order += 1

    for channel, key, value in model["seed_writes"]:
        push(channel, key, value)
    plan = []
    for i, row in enumerate(model["attention"]):
        body = row.get("keyed_read") or row.get("cum_sum")
        plan.append((body["phase"], 0, i))
    plan += [(row["phase"], 1, i) for i, row in enumerate(model["wiring"])]
    plan += [(row["phase"], 2, i) for i, row in enumerate(model["ffn"])]
    plan.sort()
    outputs = []
    for si, fields in enumerate(steps):
        if len(fields) != model["input_field_count"]:
            raise NumericExecutionError("input_arity_mismatch", si, f"step supplies {len(fields)} fields, expected {model['input_field_count']}")
        r = [0.0] * model["slot_count"]
        for _, kind, i in plan:
            if kind == 1:
                row = model["wiring"][i]
                total = float(row["bias"])
                if row.get("input_field") is not None:
                    total += fields[row["input_field"]]
                for coefficient, slot in row["terms"]:
                    total += coefficient * r[slot]
                r[row["out_slot"]] = _check(total, si)
            elif kind == 0:
                row = model["attention"][i]
                if "keyed_read" in row:
                    kr = row["keyed_read"]
                    q = r[kr["query_slot"]]
                    best, best_score = None, -math.inf
                    for p in points.get(kr["channel"], ()):
                        score = 2 * q * p[0] - p[0] * p[0]
                        if best is None or score > best_score or (score == best_score and p[2] > best[2]):
                            best, best_score = p, score
                    if best is None or best[0] != q:
                        raise NumericExecutionError("missing_key", si, f"missing key {q} on channel {kr['channel']}")
                    r[kr["out_slot"]] = best[1]
                else:
                    cs = row["cum_sum"]
                    total = _check(acc.get(cs["channel"], 0.0) + r[cs["value_slot"]], si)
                    acc[cs["channel"]] = total
                    r[cs["out_slot"]] = total
            else:
                row = model["ffn"][i]
                r[row["out_slot"]] = _check(r[row["value_slot"]] * max(r[row["gate_slot"]], 0.0), si)
        for w in model["writes"]:
            push(w["channel"], r[w["key_slot"]], r[w["value_slot"]])
        outputs.append([int(math.trunc(r[s])) for s in model["output_slots"]])
    return {"executorId": EXECUTOR_ID, "graphDigest": model["graph_digest"], "stepCount": len(steps), "stepOutputs": outputs,
            "traceDigest": digest_trace_rows(model["graph_digest"], outputs)}


def collect_interpreter_outputs(step_outputs) -> dict:
    """Rows are (out_flag, out_value, ..., halt at index 4): emitted values and whether the program halted."""
    outs = [row[1] if len(row) > 1 else 0 for row in step_outputs if row and row[0] == 1]
    last = step_outputs[-1] if step_outputs else None
    return {"outputs": outs, "halted": last is not None and (last[4] if len(last) > 4 else 0) >= 1}


# ---------------------------------------------------------------- replay verdicts
def _verdict(model, claimed, validator, **kw):
    v = {"classId": REPLAY_CLASS_ID, "graphDigest": model["graph_digest"], "claimedTraceDigest": claimed,
         "validatorDeviceRef": validator, "rejection": None}
    v.update(kw)
    return v


def verify_full_replay(model: dict, steps, claimed_trace_digest: str, validator_device_ref: str) -> dict:
    try:
        t = execute_numeric_model(model, steps)
    except NumericExecutionError as e:
        return _verdict(model, claimed_trace_digest, validator_device_ref, outcome="rejected", replayedSteps=0, comparedSteps=0,
                        replayedTraceDigest=None, rejection={"reason": "execution_refused", "detail": str(e)})
    ok = t["traceDigest"] == claimed_trace_digest
    return _verdict(model, claimed_trace_digest, validator_device_ref, outcome="verified" if ok else "rejected",
                    replayedSteps=t["stepCount"], comparedSteps=t["stepCount"], replayedTraceDigest=t["traceDigest"],
                    rejection=None if ok else {"reason": "trace_digest_mismatch", "actual": t["traceDigest"]})


def verify_window(model: dict, steps, window_start: int, claimed_rows, validator_device_ref: str) -> dict:
    """Spot check: replay everything, compare only rows [window_start, window_start + len(claimed_rows))."""
    t = execute_numeric_model(model, steps)
    for off, claimed in enumerate(claimed_rows):
        step = window_start + off
        actual = t["stepOutputs"][step] if 0 <= step < len(t["stepOutputs"]) else None
        if actual is None or list(actual) != [int(v) for v in claimed]:
            return _verdict(model, "", validator_device_ref, outcome="rejected", replayedSteps=t["stepCount"],
                            comparedSteps=len(claimed_rows), replayedTraceDigest=t["traceDigest"],
                            rejection={"reason": "row_mismatch", "step": step})
    return _verdict(model, "", validator_device_ref, outcome="verified", replayedSteps=t["stepCount"],
                    comparedSteps=len(claimed_rows), replayedTraceDigest=t["traceDigest"])


# ---------------------------------------------------------------- dense-weight modules
def _need(field, found, expected):
    if found != expected:
        raise DenseModuleError(field, f"dimension {found} does not match expected {expected}")


def _one_hot_row(row, field) -> int:
    slot = None
    for i, v in enumerate(row):
        if v == 1 and slot is None:
            slot = i
        elif v != 0:
            raise DenseModuleError(field, "row is not one-hot")
    if slot is None:
        raise DenseModuleError(field, "row is not one-hot")
    return slot


def _one_hot_col(matrix, col, field) -> int:
    return _one_hot_row([row[col] if col < len(row) else 0 for row in matrix], field.replace("row", "column"))


def _zero_row(row, field):
    if any(v != 0 for v in row):
        raise DenseModuleError(field, "row is not zero")


def dense_module_to_numeric_model(m: dict) -> dict:
    """Lower explicit matrices (W_Q/K/V/O, FFN value/gate/out, wiring) to numeric rows.  The selector
    matrices must be one-hot (or zero where the head kind says so); anything else is refused."""
    if m.get("moduleKind") != DENSE_MODULE_KIND:
        raise DenseModuleError("moduleKind", "unsupported module kind")
    d = m["dModel"]
    wiring, attention, ffn = [], [], []
    for b in m["wiringBlocks"]:
        n = len(b["wResidual"])
        _need("wiring.outSlots", len(b["outSlots"]), n)
        _need("wiring.bias", len(b["bias"]), n)
        _need("wiring.inputFields", len(b["inputFields"]), n)
        for i, row in enumerate(b["wResidual"]):
            _need("wiring.wResidual.row", len(row), d)
            wiring.append({"bias": b["bias"][i], "input_field": b["inputFields"][i], "out_slot": b["outSlots"][i],
                           "phase": b["phase"], "terms": [[c, s] for s, c in enumerate(row) if c != 0]})
    for b in m["attentionBlocks"]:
        H = len(b["heads"])
        for k in ("wQ", "wK", "wV"):
            _need("attention." + k, len(b[k]), H)
        _need("attention.wO", len(b["wO"]), d)
        for row in b["wO"]:
            _need("attention.wO.row", len(row), H)
        for h, head in enumerate(b["heads"]):
            q, k, v = b["wQ"][h], b["wK"][h], b["wV"][h]
            for name, row in (("wQ", q), ("wK", k), ("wV", v)):
                _need(f"attention.{name}.row", len(row), d)
            _zero_row(k, "attention.wK")
            out = _one_hot_col(b["wO"], h, "attention.wO")
            if "keyedRead" in head:
                qs = _one_hot_row(q, "attention.wQ")
                _zero_row(v, "attention.wV.keyedRead")
                kr = head["keyedRead"]
                if qs != kr["query_slot"] or out != kr["out_slot"]:
                    raise DenseModuleError("attention.keyedRead", "descriptor mismatch")
                attention.append({"keyed_read": {"channel": kr["channel"], "out_slot": out, "phase": b["phase"], "query_slot": qs}})
            else:
                _zero_row(q, "attention.wQ.cumSum")
                vs = _one_hot_row(v, "attention.wV")
                cs = head["cumSum"]
                if vs != cs["value_slot"] or out != cs["out_slot"]:
                    raise DenseModuleError("attention.cumSum", "descriptor mismatch")
                attention.append({"cum_sum": {"channel": cs["channel"], "out_slot": out, "phase": b["phase"], "value_slot": vs}})
    for b in m["ffnBlocks"]:
        n = len(b["wValue"])
        _need("ffn.wGate", len(b["wGate"]), n)
        _need("ffn.wOut", len(b["wOut"]), d)
        for row in b["wOut"]:
            _need("ffn.wOut.row", len(row), n)
        for j in range(n):
            _need("ffn.wValue.row", len(b["wValue"][j]), d)
            _need("ffn.wGate.row", len(b["wGate"][j]), d)
            ffn.append({"gate_slot": _one_hot_row(b["wGate"][j], "ffn.wGate"), "out_slot": _one_hot_col(b["wOut"], j, "ffn.wOut"),
                        "phase": b["phase"], "value_slot": _one_hot_row(b["wValue"][j], "ffn.wValue")})
    return {"attention": attention, "bundle_digest": m["bundleDigest"], "ffn": ffn, "graph_digest": m["graphDigest"],
            "input_field_count": m["inputFieldCount"], "layer_count": m["layerCount"], "model_id": m["sourceModelId"],
            "output_slots": m["outputSlots"], "schema_version": 1, "seed_writes": m["seedWrites"], "slot_count": d,
            "wiring": wiring, "writes": m["writeRows"]}


def execute_dense_module(module: dict, steps) -> dict:
    return execute_numeric_model(dense_module_to_numeric_model(module), steps)


def numeric_model_to_dense_module(model: dict, module_id: str = "module") -> dict:
    """Inverse of the lowering (one block per phase): explicit matrices for a numeric model."""
    d = model["slot_count"]
    row = lambda slot=None: [1 if i == slot else 0 for i in range(d)]
    phases = sorted({r["phase"] for r in model["wiring"]})
    wiring = []
    for ph in phases:
        rows = [r for r in model["wiring"] if r["phase"] == ph]
        W = []
        for r in rows:
            w = [0] * d
            for c, s in r["terms"]:
                w[s] += c
            W.append(w)
        wiring.append({"phase": ph, "outSlots": [r["out_slot"] for r in rows], "wResidual": W, "bias": [r["bias"] for r in rows],
                       "inputFields": [r.get("input_field") for r in rows]})
    attention = []
    for ph in sorted({(a.get("keyed_read") or a.get("cum_sum"))["phase"] for a in model["attention"]}):
        heads, wq, wk, wv, outs = [], [], [], [], []
        for a in model["attention"]:
            body = a.get("keyed_read") or a.get("cum_sum")
            if body["phase"] != ph:
                continue
            if "keyed_read" in a:
                heads.append({"keyedRead": {"channel": body["channel"], "query_slot": body["query_slot"], "out_slot": body["out_slot"]}})
                wq.append(row(body["query_slot"])); wv.append(row())
            else:
                heads.append({"cumSum": {"channel": body["channel"], "value_slot": body["value_slot"], "out_slot": body["out_slot"]}})
                wq.append(row()); wv.append(row(body["value_slot"]))
            wk.append(row()); outs.append(body["out_slot"])
        wo = [[1 if outs[h] == i else 0 for h in range(len(heads))] for i in range(d)]
        attention.append({"phase": ph, "heads": heads, "wQ": wq, "wK": wk, "wV": wv, "wO": wo})
    ffn = []
    for ph in sorted({f["phase"] for f in model["ffn"]}):
        rows = [f for f in model["ffn"] if f["phase"] == ph]
        ffn.append({"phase": ph, "wValue": [row(f["value_slot"]) for f in rows], "wGate": [row(f["gate_slot"]) for f in rows],
                    "wOut": [[1 if rows[j]["out_slot"] == i else 0 for j in range(len(rows))] for i in range(d)]})
    return {"schemaVersion": 1, "moduleKind": DENSE_MODULE_KIND, "moduleId": module_id, "sourceModelId": model["model_id"],
            "sourceModelDigest": "", "graphDigest": model["graph_digest"], "bundleDigest": model["bundle_digest"],
            "inputFieldCount": model["input_field_count"], "dModel": d, "layerCount": model["layer_count"],
            "seedWrites": model["seed_writes"], "wiringBlocks": wiring, "attentionBlocks": attention, "ffnBlocks": ffn,
            "writeRows": model["writes"], "outputSlots": model["output_slots"], "claimBoundary": "exact replay only"}


# ---------------------------------------------------------------- linked compositions
def compose_numeric_models(banks: list[dict], graph_digest: str, model_id: str = "composed") -> tuple[dict, list[dict]]:
    """Place several numeric models side by side in one residual vector: bank i's slots move by its
    slot offset, its channels by its channel offset, and its outputs occupy a contiguous range of the
    composed output row.  Returns (composed model, per-bank placement)."""
    slot_off = chan_off = out_off = 0
    out = {"schema_version": 1, "model_id": model_id, "graph_digest": graph_digest, "bundle_digest": "", "input_field_count": 0,
           "slot_count": 0, "layer_count": 0, "seed_writes": [], "wiring": [], "attention": [], "ffn": [], "writes": [], "output_slots": []}
    placements = []
    for m in banks:
        if m["input_field_count"] != banks[0]["input_field_count"]:
            raise ValueError("banks must take the same input fields")
        n_chan = 1 + max([c for c, _, _ in m["seed_writes"]] + [w["channel"] for w in m["writes"]] +
                         [(a.get("keyed_read") or a.get("cum_sum"))["channel"] for a in m["attention"]] + [-1])
        s, c = slot_off, chan_off
        out["seed_writes"] += [[ch + c, k, v] for ch, k, v in m["seed_writes"]]
        out["wiring"] += [{**r, "out_slot": r["out_slot"] + s, "terms": [[co, sl + s] for co, sl in r["terms"]]} for r in m["wiring"]]
        for a in m["attention"]:
            if "keyed_read" in a:
                b = a["keyed_read"]
                out["attention"].append({"keyed_read": {**b, "channel": b["channel"] + c, "query_slot": b["query_slot"] + s, "out_slot": b["out_slot"] + s}})
            else:
                b = a["cum_sum"]
                out["attention"].append({"cum_sum": {**b, "channel": b["channel"] + c, "value_slot": b["value_slot"] + s, "out_slot": b["out_slot"] + s}})
        out["ffn"] += [{**f, "value_slot": f["value_slot"] + s, "gate_slot": f["gate_slot"] + s, "out_slot": f["out_slot"] + s} for f in m["ffn"]]
        out["writes"] += [{"channel": w["channel"] + c, "key_slot": w["key_slot"] + s, "value_slot": w["value_slot"] + s} for w in m["writes"]]
        out["output_slots"] += [o + s for o in m["output_slots"]]
        placements.append({"slotOffset": s, "channelOffset": c, "projectedOutputStart": out_off, "projectedOutputEnd": out_off + len(m["output_slots"])})
        slot_off += m["slot_count"]
        chan_off += n_chan
        out_off += len(m["output_slots"])
        out["layer_count"] = max(out["layer_count"], m["layer_count"])
    out["slot_count"], out["input_field_count"] = slot_off, banks[0]["input_field_count"]
    return out, placements


def verify_linked_composition(composed_model: dict, banks: list[dict], steps, expected_composed_digest: str | None = None) -> dict:
    """``banks``: dicts with ``bankId``, ``model``, ``expectedTraceDigest``, ``projectedOutputStart/End``.
    The composition clears when the composed run matches its expected digest and every bank's own run
    both matches its expected digest and equals its projection of the composed rows."""
    blockers, verdicts = [], []
    try:
        ct = execute_numeric_model(composed_model, steps)
    except NumericExecutionError:
        return {"replayVerificationCleared": False, "blockerRefs": [_B + "composed_execution_refused"], "composedTraceDigest": None,
                "constituentVerifications": []}
    if expected_composed_digest is not None and ct["traceDigest"] != expected_composed_digest:
        blockers.append(_B + "composed_trace_mismatch")
    for b in banks:
        refs = []
        try:
            st = execute_numeric_model(b["model"], steps)
        except NumericExecutionError:
            verdicts.append({"bankId": b["bankId"], "verified": False, "blockerRefs": [_B + "constituent_execution_refused"]})
            continue
        proj = [row[b["projectedOutputStart"]: b["projectedOutputEnd"]] for row in ct["stepOutputs"]]
        if st["traceDigest"] != b.get("expectedTraceDigest", st["traceDigest"]):
            refs.append(_B + "source_trace_mismatch")
        same = proj == st["stepOutputs"]
        if not same:
            refs.append(_B + "projected_rows_diverged")
        verdicts.append({"bankId": b["bankId"], "sourceTraceDigest": st["traceDigest"], "projectedRowsMatchSource": same,
                         "projectedTraceDigest": digest_trace_rows(st["graphDigest"], proj), "verified": not refs, "blockerRefs": refs})
    blockers += [r for v in verdicts for r in v["blockerRefs"]]
    return {"replayVerificationCleared": not blockers, "blockerRefs": blockers, "composedTraceDigest": ct["traceDigest"],
            "constituentVerifications": verdicts, "verifierId": "tassadar.linked_dense.replay_verifier.b200.v1"}


# ---------------------------------------------------------------- capability envelope and self-test
# A node may only advertise the executor capability together with a receipt that its own executor replayed the
# digest-pinned fixture to the expected trace digest (packages/tassadar-executor/src/capability-envelope.ts:109-160
# self-test, :187-222 declaration, :241-266 matrix row, :286-349 row decoder, :351-388 ref filter).
CAPABILITY_REF = "capability.tassadar_poc.numeric_model_executor"     # packages/tassadar-executor/src/lane.ts:7
SELF_TEST_RECEIPT_SCHEMA = "openagents.tassadar_executor.self_test_receipt.v1"
CAPABILITY_ENVELOPE_SCHEMA = "openagents.pylon.tassadar_capability_envelope.v1"
CAPABILITY_MATRIX_ROW_SCHEMA = "openagents.tassadar_executor.capability_matrix_row.v1"
WINDOW_VERSION_REF = "window.tassadar_executor.exact_2p53.v1"
WORKLOAD_FAMILY_REF = "workload.tassadar_executor.alm_numeric_trace.v1"
LEG_REFS = ("leg.tassadar_executor.alm_numeric_execute.v1", "leg.tassadar_executor.exact_trace_replay_full.v1",
            "leg.tassadar_executor.exact_trace_replay_window.v1")
_SELF_TEST_PREFIX = "receipt.tassadar_executor.self_test.v1"
_COMPILE_PREFIX = "receipt.tassadar_compile.model_digest"
_SELF_TEST_REF = re.compile(r"^receipt\.tassadar_executor\.self_test\.v1\.[0-9a-f]{16}$")
_COMPILE_REF = re.compile(r"^receipt\.tassadar_compile\.model_digest\.[0-9a-f]{16}$")


class CapabilityShapeError(Exception):
    pass


def run_self_test(workload: dict, observed_at: str = "1970-01-01T00:00:00Z") -> dict:
    """workload = {fixtureId, expectedModelDigest, expectedTraceDigest, model, steps}.  The receipt carries digests only."""
    v = verify_full_replay(workload["model"], workload["steps"], workload["expectedTraceDigest"], "device.self_test.local")
    ok = v["outcome"] == "verified"
    rej = v["rejection"]
    detail = None if ok else ("self-test replay rejected without a named rejection" if rej is None else
                              f"execution_refused: {rej['detail']}" if rej["reason"] == "execution_refused" else rej["reason"])
    return {"schema": SELF_TEST_RECEIPT_SCHEMA, "capabilityRef": CAPABILITY_REF, "executorId": EXECUTOR_ID, "fixtureId": workload["fixtureId"],
            "graphDigest": workload["model"]["graph_digest"], "modelDigest": workload["expectedModelDigest"],
            "expectedTraceDigest": workload["expectedTraceDigest"], "replayedTraceDigest": v["replayedTraceDigest"],
            "stepCount": v["replayedSteps"], "replayClassId": REPLAY_CLASS_ID, "observedAt": observed_at,
            "outcome": "verified" if ok else "failed", "refusalDetail": detail,
            "receiptRef": f"{_SELF_TEST_PREFIX}.{v['replayedTraceDigest'][:16]}" if ok and v["replayedTraceDigest"] else None}


def capability_matrix_row(envelope: dict) -> dict:
    r = envelope["selfTestReceipt"]
    if r["receiptRef"] is None:
        raise CapabilityShapeError("capability matrix row requires a verified self-test receipt ref")
    return {"schema": CAPABILITY_MATRIX_ROW_SCHEMA, "capabilityRef": CAPABILITY_REF, "workloadFamilyRef": WORKLOAD_FAMILY_REF,
            "windowVersionRef": WINDOW_VERSION_REF, "legRefs": list(envelope["legRefs"]), "replayClassId": envelope["replayClassId"],
            "compileReceiptRef": f"{_COMPILE_PREFIX}.{r['modelDigest'][:16]}", "replayReceiptRef": r["receiptRef"],
            "posture": "execute_exact_or_refuse"}


def build_capability_declaration(receipt: dict) -> dict:
    """A failed or receipt-less self-test yields a typed refusal, never a declaration."""
    if receipt["outcome"] != "verified" or receipt["receiptRef"] is None:
        return {"declared": False, "refusal": {
            "kind": "self_test_receipt_missing" if receipt["outcome"] == "verified" else "self_test_failed",
            "refusalRef": "refusal.tassadar_executor.capability_undeclarable",
            "detail": receipt.get("refusalDetail") or "executor self-test did not verify the pinned trace digest"}}
    env = {"schema": CAPABILITY_ENVELOPE_SCHEMA, "capabilityRef": CAPABILITY_REF, "windowVersionRef": WINDOW_VERSION_REF,
           "exactnessWindowLabel": "2^53", "exactnessWindow": EXACT_WINDOW, "legRefs": list(LEG_REFS), "replayClassId": receipt["replayClassId"],
           "executorId": receipt["executorId"], "selfTestReceipt": receipt}
    return {"declared": True, "envelope": env, "matrixRow": capability_matrix_row(env), "capabilityRefs": [CAPABILITY_REF, receipt["receiptRef"]]}


def decode_capability_matrix_row(row) -> dict:
    """Every fixed field must equal its constant and every receipt field its receipt-derived pattern."""
    if not isinstance(row, dict):
        raise CapabilityShapeError("capability matrix row must be an object")
    for k, want in (("schema", CAPABILITY_MATRIX_ROW_SCHEMA), ("capabilityRef", CAPABILITY_REF), ("workloadFamilyRef", WORKLOAD_FAMILY_REF),
                    ("windowVersionRef", WINDOW_VERSION_REF), ("replayClassId", REPLAY_CLASS_ID), ("posture", "execute_exact_or_refuse")):
        if row.get(k) != want:
            raise CapabilityShapeError(f"capability matrix row field {k} must be {want}, got {row.get(k)}")
    legs = row.get("legRefs")
    if not isinstance(legs, list) or not legs or any(l not in LEG_REFS for l in legs):
        raise CapabilityShapeError("legRefs must be a non-empty subset of the known executor legs")
    if not isinstance(row.get("compileReceiptRef"), str) or not _COMPILE_REF.match(row["compileReceiptRef"]):
        raise CapabilityShapeError("compileReceiptRef must derive from a model digest")
    if not isinstance(row.get("replayReceiptRef"), str) or not _SELF_TEST_REF.match(row["replayReceiptRef"]):
        raise CapabilityShapeError("replayReceiptRef must derive from a verified self-test receipt")
    return {k: row[k] for k in ("schema", "capabilityRef", "workloadFamilyRef", "windowVersionRef", "legRefs", "replayClassId",
                                "compileReceiptRef", "replayReceiptRef", "posture")}


def has_receipted_capability(refs) -> bool:
    return CAPABILITY_REF in refs and any(_SELF_TEST_REF.match(r) for r in refs)


def strip_unreceipted_capability(refs) -> list:
    """Drop a configuration-asserted capability claim (and orphaned receipt refs) that has no self-test receipt beside it."""
    refs = list(refs)
    return refs if has_receipted_capability(refs) else [r for r in refs if r != CAPABILITY_REF and not _SELF_TEST_REF.match(r)]
