"""Artifact digests, release / model manifests, worker and run receipts.

Shapes follow what the reference's consumers read: the release and model-artifact manifests a
node installs from (``psionic.release_manifest.v1``, ``psionic.model_artifact_manifest.v1``:
apps/pylon/docs/2026-06-09-pylon-psionic-ml-connection-audit.md:157-200, 291-306), the training
worker receipt (``openagents.psionic.training_worker_receipt.v0.3``: apps/pylon/src/assignment.ts:
2437-2461), the serving receipt with its ``stages[]`` (inference/openagents-network-adapter.ts:85-133)
and the pipeline-sharded run receipt with its layer-block payout split
(shard-wan-serving-payout-split.ts:25-26, 44-67, 134-194 structural checks, largest-remainder split).
"""
from __future__ import annotations

import hashlib
import json
import os
import time

RELEASE_MANIFEST_VERSION = "psionic.release_manifest.v1"
MODEL_ARTIFACT_MANIFEST_VERSION = "psionic.model_artifact_manifest.v1"
WORKER_RECEIPT_VERSION = "psionic.worker_receipt.v1"
TRAINING_WORKER_RECEIPT_VERSION = "openagents.psionic.training_worker_receipt.v0.3"
SHARDED_RUN_RECEIPT_VERSION = "psionic.serve.pipeline_sharded_run_receipt.v1"
TENSOR_SHARDED_RUN_RECEIPT_VERSION = "psionic.serve.tensor_sharded_run_receipt.v1"


def artifact_digest(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 22), b""):
            h.update(chunk)
    return "sha256:" + h.hexdigest()


def canonical_digest(obj) -> str:
    return "sha256:" + hashlib.sha256(json.dumps(obj, sort_keys=True, separators=(",", ":")).encode()).hexdigest()


def model_artifact_manifest(path: str, architecture: str, quantization: str, chat_template_digest: str | None = None) -> dict:
    m = {"schemaVersion": MODEL_ARTIFACT_MANIFEST_VERSION, "fileName": os.path.basename(path), "sizeBytes": os.path.getsize(path),
         "artifactDigest": artifact_digest(path), "format": "gguf", "architecture": architecture, "quantization": quantization,
         "chatTemplateDigest": chat_template_digest}
    m["manifestDigest"] = canonical_digest(m)
    return m


def release_manifest(version: str, binaries: dict[str, str], models: list[dict]) -> dict:
    """``binaries``: name -> path of a built artefact (the native libraries and the node CLI)."""
    m = {"schemaVersion": RELEASE_MANIFEST_VERSION, "version": version,
         "binaries": [{"name": n, "sizeBytes": os.path.getsize(p), "digest": artifact_digest(p)} for n, p in sorted(binaries.items())],
         "modelArtifacts": [x["manifestDigest"] for x in models]}
    m["manifestDigest"] = canonical_digest(m)
    return m


def verify_manifest(m: dict) -> bool:
    body = {k: v for k, v in m.items() if k != "manifestDigest"}
    return m.get("manifestDigest") == canonical_digest(body)


def serving_receipt(serve_response: dict) -> dict:
    """Gateway-side receipt derived from a serve response (sharded = more than one stage)."""
    return {"servingRunRef": serve_response["servingRunRef"], "servedModel": serve_response["servedModel"],
            "sharded": len(serve_response["stages"]) > 1, "stages": serve_response["stages"],
            "parityMode": serve_response["parityMode"], "parityVerified": serve_response["parityVerified"]}


def clears_paid_traffic(receipt: dict) -> bool:
    """Paid traffic needs verified exact-greedy parity and, when present, a fully passing
    paid-traffic verification bundle (openagents-network-adapter.ts:215-231)."""
    if not (receipt.get("parityMode") == "exact_greedy_parity" and receipt.get("parityVerified") is True):
        return False
    v = receipt.get("paidTrafficVerification")
    if v is None:
        return False
    return bool(v.get("parityPassed") and v.get("canaryPassed") and v.get("replayPassed") and v.get("payoutEligible")
                and not v.get("blockerRefs"))


def worker_receipt(worker_id: str, kind: str, assignment_id: str, status: str, evidence: dict, now_ms: int | None = None) -> dict:
    r = {"schemaVersion": WORKER_RECEIPT_VERSION, "workerId": worker_id, "workerKind": kind, "assignmentId": assignment_id,
         "status": status, "evidenceDigest": canonical_digest(evidence), "emittedAtMs": now_ms if now_ms is not None else int(time.time() * 1000)}
    r["receiptDigest"] = canonical_digest(r)
    return r


def training_worker_receipt(assignment_id: str, run_ref: str, window_ref: str, step: int, loss: float, tokens: int,
                            checkpoint_digest: str | None, base_checkpoint_digest: str | None, config_digest: str,
                            now_ms: int | None = None) -> dict:
    r = {"schemaVersion": TRAINING_WORKER_RECEIPT_VERSION, "assignmentId": assignment_id, "trainingRunRef": run_ref,
         "windowRef": window_ref, "step": step, "loss": loss, "tokensProcessed": tokens, "checkpointDigest": checkpoint_digest,
         "baseCheckpointDigest": base_checkpoint_digest, "trainingConfigDigest": config_digest,
         "emittedAtMs": now_ms if now_ms is not None else int(time.time() * 1000)}
    r["receiptDigest"] = canonical_digest(r)
    return r


# ---------------------------------------------------------------- sharded run receipts
def sharded_run_receipt(model_artifact_digest: str, total_layers: int, stages: list[dict], parity_mode: str = "verified") -> dict:
    if parity_mode not in ("verified", "no_reference", "mismatch"):
        raise ValueError("parityMode must be verified, no_reference or mismatch")
    return {"schemaVersion": SHARDED_RUN_RECEIPT_VERSION, "modelArtifactDigest": model_artifact_digest, "parityMode": parity_mode,
            "stages": stages, "totalLayerCount": total_layers}


def structural_errors(receipt: dict) -> list[str]:
    """More than one stage, GPU resident, contiguous, gap-free, no whole-model stage."""
    errs, total = [], receipt["totalLayerCount"]
    if total <= 0:
        errs.append("totalLayerCount must be a positive integer.")
    if len(receipt["stages"]) < 2:
        errs.append("a sharded run must record more than one serving stage (no single-node split).")
    cursor = 0
    for s in sorted(receipt["stages"], key=lambda s: s["layerStart"]):
        i, a, b = s["stageIndex"], s["layerStart"], s["layerEnd"]
        if not s["gpuResident"]:
            errs.append(f"stage {i} did not hold its layer-block GPU-resident (no whole-model fallback).")
        if a < 0 or b > total:
            errs.append(f"stage {i} layer range [{a}, {b}) is outside [0, {total}).")
        if a >= b:
            errs.append(f"stage {i} has an empty or inverted layer range [{a}, {b}).")
        if a == 0 and b == total and total > 0:
            errs.append(f"stage {i} covers the whole model — that is not a layer-block split.")
        if a > cursor:
            errs.append(f"gap in layer coverage before stage {i}: layers [{cursor}, {a}) unserved.")
        if a < cursor:
            errs.append(f"overlap in layer coverage at stage {i}: layers [{a}, {cursor}) double-served.")
        cursor = max(cursor, b)
    if not errs and cursor != total:
        errs.append(f"layer coverage stops at {cursor} but the model has {total} layers.")
    return errs


def payout_split(receipt: dict, contributor_cut_sats: int) -> list[dict]:
    """Largest-remainder split of the contributor cut by layer-block size."""
    errs = structural_errors(receipt)
    if errs:
        raise ValueError("; ".join(errs))
    if receipt["parityMode"] != "verified":
        raise ValueError("payout needs verified parity")
    stages = sorted(receipt["stages"], key=lambda s: s["stageIndex"])
    counts = [s["layerEnd"] - s["layerStart"] for s in stages]
    total = sum(counts)
    base = []
    for s, n in zip(stages, counts):
        raw = contributor_cut_sats * n
        base.append({"stageIndex": s["stageIndex"], "layerCount": n, "floor": raw // total, "rem": raw - (raw // total) * total,
                     "weightBps": round(n / total * 10000)})
    left = contributor_cut_sats - sum(b["floor"] for b in base)
    bonus = set()
    for b in sorted(base, key=lambda b: (-b["rem"], b["stageIndex"])):
        if left <= 0:
            break
        bonus.add(b["stageIndex"])
        left -= 1
    return [{"stageIndex": b["stageIndex"], "layerCount": b["layerCount"], "weightBps": b["weightBps"],
             "payoutSats": b["floor"] + (1 if b["stageIndex"] in bonus else 0)} for b in base]
