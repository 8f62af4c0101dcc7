"""Checkpoint layout and resume.

A checkpoint is a directory:

    manifest.json          run/window refs, step, world size, ZeRO stage, dtype map, commit term,
                           per-file ``sha256:`` digests, config digest, optimizer-state digest,
                           checkpoint digest (digest of the sorted file digests)
    model-rank{r}.bin      fp32 master-weight shard of rank r
    optim-rank{r}.bin      AdamW first and second moments of rank r's shard (m then v, fp32)

Every file is written under a temporary name and renamed, then read back and re-hashed before the
manifest records it; the manifest itself is written last, so a directory without a manifest is an
aborted save.  ``load`` verifies every digest and re-shards when the world size changed.  The
reference defines the semantics (content-addressed, read back and re-hashed before a window may
seal: training-durable-checkpoint-seal.ts:68-99; candidates carry base-checkpoint, optimizer-state
and config digests: tassadar-gradient-window-regime.ts:15-39; parameter state committed by SHA-256:
cs336-a1-real-gradient-workload.ts:801-809); the file layout is this framework's own.
"""
from __future__ import annotations

import hashlib
import json
import os

import numpy as np
import torch

from ..control import seal as seal_mod

MANIFEST_VERSION = "b200.train.checkpoint_manifest.v1"


def sha256_file(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 22), b""):
            h.update(chunk)
    return "sha256:" + h.hexdigest()


def sha256_json(obj) -> str:
    return "sha256:" + hashlib.sha256(json.dumps(obj, sort_keys=True, separators=(",", ":")).encode()).hexdigest()


def _write_verified(path: str, arr: np.ndarray) -> tuple[str, int]:
    """Temp name + rename, then read back and re-hash."""
    tmp = path + ".tmp"
    data = np.ascontiguousarray(arr).tobytes()
    with open(tmp, "wb") as f:
        f.write(data)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)
    want = "sha256:" + hashlib.sha256(data).hexdigest()
    got = sha256_file(path)
    if got != want:
        raise IOError(f"read-back digest mismatch for {path}")
    return got, len(data)


def save_shard(ckpt_dir: str, rank: int, master: torch.Tensor, m: torch.Tensor, v: torch.Tensor) -> dict:
    """Each rank writes its own two files; returns their manifest entries."""
    os.makedirs(ckpt_dir, exist_ok=True)
    out = {}
    name = f"model-rank{rank}.bin"
    d, n = _write_verified(os.path.join(ckpt_dir, name), master.detach().float().cpu().numpy())
    out[name] = {"digest": d, "bytes": n, "dtype": "f32", "kind": "master_shard", "rank": rank}
    name = f"optim-rank{rank}.bin"
    d, n = _write_verified(os.path.join(ckpt_dir, name), torch.cat((m, v)).detach().float().cpu().numpy())
    out[name] = {"digest": d, "bytes": n, "dtype": "f32", "kind": "adamw_m_v_shard", "rank": rank}
    return out


def write_manifest(ckpt_dir: str, files: dict, *, run_ref: str, window_ref: str, step: int, world_size: int,
                   zero_stage: int, n_total: int, shard: int, term: int, train_config: dict, model_config: dict) -> dict:
    """Rank 0 (the commit authority) writes the manifest once every rank's entries are known."""
    optim_digest = sha256_json(sorted(v["digest"] for k, v in files.items() if k.startswith("optim-")))
    man = {
        "schemaVersion": MANIFEST_VERSION, "runRef": run_ref, "windowRef": window_ref, "step": step,
        "worldSize": world_size, "zeroStage": zero_stage, "nTotal": n_total, "shard": shard, "term": term,
        "dtypeMap": {"master": "f32", "adam_m": "f32", "adam_v": "f32", "working_params": "bf16"},
        "files": files, "trainingConfigDigest": sha256_json(train_config), "modelConfig": model_config,
        "optimizerStateDigest": optim_digest,
        "checkpointDigestRef": sha256_json(sorted(v["digest"] for v in files.values())),
    }
    tmp = os.path.join(ckpt_dir, "manifest.json.tmp")
    with open(tmp, "w") as f:
        json.dump(man, f, indent=1, sort_keys=True)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, os.path.join(ckpt_dir, "manifest.json"))
    return man


def seal_descriptor(man: dict, ckpt_dir: str, replication_factor: int = 1, storage_class: str = "single_host_disk",
                    remote_store_ref: str | None = None) -> seal_mod.DurableCheckpointSeal:
    """The durable-seal descriptor of a saved checkpoint.  A plain local directory is honest about
    what it is (one replica on one disk), so the seal predicate HOLDs until a replicated
    content-addressed store confirms the copy."""
    size = sum(v["bytes"] for v in man["files"].values())
    return seal_mod.DurableCheckpointSeal(
        checkpoint_digest_ref=man["checkpointDigestRef"], replication_factor=replication_factor,
        retrieval_verified=True, size_bytes=size, storage_class=storage_class, window_ref=man["windowRef"],
        remote_checkpoint_store_ref=remote_store_ref,
        remote_checkpoint_object_ref=("objects/" + man["checkpointDigestRef"].split(":")[1]) if remote_store_ref else None,
        readback_rehash_receipt_ref=("receipt.readback." + man["checkpointDigestRef"].split(":")[1][:16]) if remote_store_ref else None)


class CheckpointError(RuntimeError):
    pass


def load_manifest(ckpt_dir: str) -> dict:
    p = os.path.join(ckpt_dir, "manifest.json")
    if not os.path.exists(p):
        raise CheckpointError(f"{ckpt_dir} has no manifest (aborted or missing save)")
    man = json.load(open(p))
    if man.get("schemaVersion") != MANIFEST_VERSION:
        raise CheckpointError("unknown manifest version")
    return man


def verify(ckpt_dir: str) -> dict:
    """Re-hash every file against the manifest; raises on the first mismatch."""
    man = load_manifest(ckpt_dir)
    for name, ent in man["files"].items():
        path = os.path.join(ckpt_dir, name)
        if not os.path.exists(path):
            raise CheckpointError(f"missing shard {name}")
        if sha256_file(path) != ent["digest"]:
            raise CheckpointError(f"digest mismatch for {name}")
    if sha256_json(sorted(v["digest"] for v in man["files"].values())) != man["checkpointDigestRef"]:
        raise CheckpointError("checkpoint digest does not match its files")
    return man


def load_full(ckpt_dir: str) -> tuple[dict, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Verify, then return (manifest, master, m, v) as full flat fp32 tensors."""
    man = verify(ckpt_dir)
    W, sh = man["worldSize"], man["shard"]
    master, m, v = [], [], []
    for r in range(W):
        a = np.fromfile(os.path.join(ckpt_dir, f"model-rank{r}.bin"), dtype=np.float32)
        o = np.fromfile(os.path.join(ckpt_dir, f"optim-rank{r}.bin"), dtype=np.float32)
        if a.size != sh or o.size != 2 * sh:
            raise CheckpointError(f"shard {r} has the wrong size")
        master.append(torch.from_numpy(a))
        m.append(torch.from_numpy(o[:sh].copy()))
        v.append(torch.from_numpy(o[sh:].copy()))
    return man, torch.cat(master), torch.cat(m), torch.cat(v)


def reshard(full: torch.Tensor, n_total_new: int, world_new: int, rank: int) -> torch.Tensor:
    """Slice of a full flat state for ``rank`` of a new world size (zero padded at the tail)."""
    if full.numel() < n_total_new:
        full = torch.cat((full, torch.zeros(n_total_new - full.numel(), dtype=full.dtype)))
    sh = n_total_new // world_new
    return full[rank * sh: (rank + 1) * sh].clone()
