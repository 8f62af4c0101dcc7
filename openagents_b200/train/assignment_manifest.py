"""The zero-touch path: a training assignment manifest in, a run and its receipts out, no flags in between.

The reference names the contract (``psionic.training_assignment.v1``, beside ``psionic.worker_receipt.v1``) among the schemas a
node and the training stack exchange, and describes the shape of the flow: assignment -> local execution -> signed receipts ->
closeout (apps/pylon/docs/2026-06-09-pylon-psionic-ml-connection-audit.md:296-303;
docs/2026-06-10-cs336-distributed-homework-continuation-audit.md:380-392: the packaged demo lane "was built for zero-touch manifest
dispatch").  The fields are not spelled out there, so this module defines them for this trainer:

* what to run: a lane (``pretrain`` | ``sft`` | ``dpo``), the model preset and depth, the batch geometry, the step budget, the
  schedule and seed;
* on what: input files by ref, each pinned by SHA-256 and byte length; a file that does not match is a refusal, not a warning;
* under which bounds: a wall-clock budget and a step budget the run may not exceed;
* what must come back: a checkpoint directory, optionally a GGUF export, and the receipts.

``validate`` checks a manifest, ``verify_inputs`` hashes the inputs, ``launcher_argv`` lowers it to ``b200-train`` flags, ``receipts``
builds the worker receipt and the training worker receipt once the run has finished.  ``b200-train --manifest FILE`` ties them together.
"""
from __future__ import annotations

import hashlib
import json
import os
import re

from ..receipts import manifests as mf

SCHEMA = "psionic.training_assignment.v1"
LANES = ("pretrain", "sft", "dpo")
_SAFE = re.compile(r"^[A-Za-z0-9][A-Za-z0-9_.:/-]{2,200}$")
_DIGEST = re.compile(r"^sha256:[0-9a-f]{64}$")


class AssignmentRefused(ValueError):
    def __init__(self, blockers: list[str]):
        super().__init__(", ".join(blockers))
        self.blockers = blockers


def file_digest(path: str) -> tuple[str, int]:
    h, n = hashlib.sha256(), 0
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
            n += len(chunk)
    return "sha256:" + h.hexdigest(), n


def make_manifest(assignment_id: str, lane: str, inputs: list[dict], steps: int, model: str = "gpt2-small-shape", layers: int = 0, global_batch: int = 512,
                  micro_batch: int = 16, seq_len: int = 1024, lr: float = 6e-4, schedule: str = "cosine", warmup_steps: int = 0, seed: int = 0,
                  max_wall_seconds: int = 3600, export_gguf: bool = True, beta: float = 0.1, nproc: int = 1, run_ref: str | None = None) -> dict:
    """``inputs``: ``{"role": "shard"|"records"|"pairs"|"tokenizer", "path": ...}``; digests and sizes are taken here."""
    ins = []
    for i in inputs:
        d, n = file_digest(i["path"])
        ins.append({"role": i["role"], "ref": i.get("ref") or f"input.{i['role']}.{d[7:23]}", "path": os.path.abspath(i["path"]), "sha256": d, "bytes": n})
    m = {"schema": SCHEMA, "assignmentId": assignment_id, "runRef": run_ref or f"run.{assignment_id}", "workClass": "small_model_local_training", "lane": lane,
         "model": {"preset": model, "layers": layers}, "batch": {"global": global_batch, "micro": micro_batch, "seqLen": seq_len},
         "optimizer": {"lr": lr, "schedule": schedule, "warmupSteps": warmup_steps, "beta": beta}, "seed": seed, "nproc": nproc,
         "budget": {"steps": steps, "maxWallSeconds": max_wall_seconds}, "inputs": ins,
         "expectedOutputs": {"checkpoint": True, "gguf": bool(export_gguf), "receipts": ["psionic.worker_receipt.v1", mf.TRAINING_WORKER_RECEIPT_VERSION]}}
    m["manifestDigest"] = mf.canonical_digest({k: v for k, v in m.items() if k != "manifestDigest"})
    return m


def _int(v, lo: int = 1, hi: int | None = None) -> bool:
    return isinstance(v, int) and not isinstance(v, bool) and v >= lo and (hi is None or v <= hi)


def _num(v, lo: float = 0.0) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool) and v == v and lo <= v < float("inf")


SCHEDULES = ("cosine", "wsd", "constant")
INPUT_ROLES = ("shard", "records", "pairs", "tokenizer")


def validate(m) -> list[str]:
    """Blocker refs (empty = the manifest can be executed here).  A manifest arrives from a coordinator: every field the lowering
    reads is type-checked here, so that a malformed one is refused with a named blocker and never raises further down."""
    b = []
    if not isinstance(m, dict) or m.get("schema") != SCHEMA:
        return ["blocker.training_assignment.schema"]
    if not isinstance(m.get("assignmentId"), str) or not _SAFE.match(m["assignmentId"]):
        b.append("blocker.training_assignment.assignment_id")
    if m.get("lane") not in LANES:
        b.append("blocker.training_assignment.unknown_lane")
    bud = m.get("budget") if isinstance(m.get("budget"), dict) else {}
    if not (_int(bud.get("steps"), 1, 10_000_000) and _int(bud.get("maxWallSeconds"))):
        b.append("blocker.training_assignment.budget")
    bt = m.get("batch") if isinstance(m.get("batch"), dict) else {}
    nproc = m.get("nproc", 1)
    if not _int(nproc, 1, 4096):
        b.append("blocker.training_assignment.nproc")
        nproc = 1
    if not all(_int(bt.get(k)) for k in ("global", "micro", "seqLen")) or bt["global"] % (bt["micro"] * nproc):
        b.append("blocker.training_assignment.batch_geometry")
    model = m.get("model") if isinstance(m.get("model"), dict) else {}
    if not (isinstance(model.get("preset"), str) and _SAFE.match(model["preset"]) and (model.get("layers") is None or _int(model["layers"], 0, 4096))):
        b.append("blocker.training_assignment.model")
    opt = m.get("optimizer") if isinstance(m.get("optimizer"), dict) else {}
    if not (_num(opt.get("lr")) and opt["lr"] > 0 and isinstance(opt.get("schedule"), str) and opt["schedule"] in SCHEDULES
            and _int(opt.get("warmupSteps"), 0) and _num(opt.get("beta", 0.1))):
        b.append("blocker.training_assignment.optimizer")
    if not _int(m.get("seed"), 0, 2 ** 63 - 1):
        b.append("blocker.training_assignment.seed")
    if not isinstance(m.get("expectedOutputs"), dict):
        b.append("blocker.training_assignment.expected_outputs")
    inputs = m.get("inputs") if isinstance(m.get("inputs"), list) else None
    if inputs is None or not all(isinstance(i, dict) for i in inputs):
        b.append("blocker.training_assignment.inputs")
        inputs = []
    need = {"pretrain": None, "sft": "records", "dpo": "pairs"}.get(m.get("lane") if isinstance(m.get("lane"), str) else None)
    if need and need not in [i.get("role") for i in inputs]:
        b.append(f"blocker.training_assignment.missing_input.{need}")
    for i in inputs:
        if not (isinstance(i.get("sha256"), str) and _DIGEST.match(i["sha256"]) and _int(i.get("bytes"), 0) and isinstance(i.get("path"), str) and i["path"]
                and i.get("role") in INPUT_ROLES and isinstance(i.get("ref"), str) and _SAFE.match(i["ref"])):
            b.append("blocker.training_assignment.input_not_pinned")
            break
    try:
        digest = mf.canonical_digest({k: v for k, v in m.items() if k != "manifestDigest"})
    except (TypeError, ValueError):
        digest = None
    if digest is None or m.get("manifestDigest") != digest:
        b.append("blocker.training_assignment.manifest_digest_mismatch")
    return b


def verify_inputs(m: dict) -> list[str]:
    b = []
    for i in m["inputs"]:
        if not os.path.exists(i["path"]):
            b.append(f"blocker.training_assignment.input_missing.{i['ref']}")
            continue
        d, n = file_digest(i["path"])
        if d != i["sha256"] or n != i["bytes"]:
            b.append(f"blocker.training_assignment.input_digest_mismatch.{i['ref']}")
    return b


def launcher_argv(m: dict, work_dir: str) -> list[str]:
    """The ``b200-train`` flags this manifest stands for (everything a person would have typed)."""
    by = {}
    for i in m["inputs"]:
        by.setdefault(i["role"], []).append(i["path"])
    a = ["--lane", m["lane"], "--model", m["model"]["preset"], "--steps", str(m["budget"]["steps"]), "--global-batch", str(m["batch"]["global"]),
         "--micro-batch", str(m["batch"]["micro"]), "--seq-len", str(m["batch"]["seqLen"]), "--lr", str(m["optimizer"]["lr"]),
         "--schedule", m["optimizer"]["schedule"], "--total-steps", str(m["budget"]["steps"]), "--warmup-steps", str(m["optimizer"]["warmupSteps"]),
         "--seed", str(m["seed"]), "--ckpt-dir", os.path.join(work_dir, "ckpt"), "--log-jsonl", os.path.join(work_dir, "steps.jsonl")]
    if m["model"].get("layers"):
        a += ["--layers", str(m["model"]["layers"])]
    if m.get("nproc", 1) > 1:
        a += ["--nproc", str(m["nproc"])]
    if m["lane"] == "pretrain" and by.get("shard"):
        a += ["--data", *by["shard"]]
    if m["lane"] == "sft":
        a += ["--sft-records", by["records"][0], "--report", os.path.join(work_dir, "lane_report.json")]
    if m["lane"] == "dpo":
        a += ["--dpo-pairs", by["pairs"][0], "--beta", str(m["optimizer"]["beta"])]
    if by.get("tokenizer") and m["lane"] == "pretrain":
        a += ["--tokenizer", by["tokenizer"][0]]
    if m["expectedOutputs"].get("gguf") and m["lane"] != "dpo":
        a += ["--export-gguf", os.path.join(work_dir, "model.gguf")]
    return a


def receipts(m: dict, work_dir: str, status: str, wall_seconds: float, worker_id: str = "worker.b200.train") -> dict:
    """What goes back: outputs by digest, the last logged step, and the two receipts.  ``status``: succeeded | failed | refused."""
    steps = []
    log = os.path.join(work_dir, "steps.jsonl")
    if os.path.exists(log):
        with open(log) as f:
            steps = [json.loads(x) for x in f if x.strip()]
    report = os.path.join(work_dir, "lane_report.json")
    if not steps and os.path.exists(report):                 # the tuning lane reports its steps in its lane report
        with open(report) as f:
            rep = json.load(f)
        steps = [{"step": r["step"], "loss": r["loss"]} for r in rep.get("stepReceipts", [])]
    last = steps[-1] if steps else {}
    outputs = {}
    if os.path.exists(report):
        outputs["laneReport"] = {"sha256": file_digest(report)[0]}
    gguf = os.path.join(work_dir, "model.gguf")
    if os.path.exists(gguf):
        outputs["gguf"] = {"sha256": file_digest(gguf)[0], "bytes": os.path.getsize(gguf)}
    ck_root = os.path.join(work_dir, "ckpt")
    ck_digest = None
    if os.path.isdir(ck_root):
        for d in sorted(os.listdir(ck_root), reverse=True):
            man = os.path.join(ck_root, d, "manifest.json")
            if os.path.exists(man):
                with open(man) as f:
                    ck_digest = json.load(f).get("checkpointDigestRef")
                outputs["checkpoint"] = {"dir": d, "checkpointDigestRef": ck_digest}
                break
    over = wall_seconds > m["budget"]["maxWallSeconds"]
    evidence = {"manifestDigest": m["manifestDigest"], "outputs": outputs, "lastStep": last.get("step"), "lastLoss": last.get("loss", last.get("pair_loss")),
                "stepsLogged": len(steps), "wallSeconds": round(wall_seconds, 3), "overWallBudget": over}
    tokens = len(steps) * m["batch"]["global"] * m["batch"]["seqLen"]
    return {"evidence": evidence,
            "workerReceipt": mf.worker_receipt(worker_id, "training", m["assignmentId"], "failed" if (over and status == "succeeded") else status, evidence),
            "trainingWorkerReceipt": mf.training_worker_receipt(m["assignmentId"], m["runRef"], f"{m['runRef']}.w0", int(last.get("step") or 0),
                                                                float(last.get("loss", last.get("pair_loss", 0.0)) or 0.0), tokens, ck_digest, None, m["manifestDigest"])}
