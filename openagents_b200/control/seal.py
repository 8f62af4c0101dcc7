"""Durable checkpoint seal predicate.

A training window may seal on a checkpoint only when the checkpoint is content addressed, lives on a
durable content-addressed storage class, is replicated at least twice, has been read back and
re-hashed, and names its remote store, object and read-back receipt.  Anything else fails toward
HOLD, never toward sealing (reference:
apps/openagents.com/workers/api/src/training-durable-checkpoint-seal.ts:29 digest pattern, :36
replication minimum, :51-66 storage classes, :68-99 descriptor, :140-179 predicate).
"""
from __future__ import annotations

import re
from dataclasses import dataclass

SCHEMA_VERSION = "openagents.training.marathon_operations.durable_checkpoint_seal.v1"
DIGEST_PATTERN = re.compile(r"^sha256:[a-f0-9]{64}$")
PUBLIC_SAFE_REF = re.compile(r"^[A-Za-z0-9][A-Za-z0-9_.:/-]*$")
MIN_DURABLE_REPLICATION_FACTOR = 2

STORAGE_CLASSES = ("content_addressed_object_store", "content_addressed_replicated_blob", "coordinator_memory",
                   "local_scratch", "node_ram", "single_host_disk")
DURABLE_CONTENT_ADDRESSED = frozenset(("content_addressed_object_store", "content_addressed_replicated_blob"))

SEAL = "seal_on_durable_checkpoint"
HOLD = "hold_for_durable_checkpoint"
BLOCKER = "blocker.training.marathon_operations.durable_checkpoint_seal_missing"


def is_public_safe_ref(s) -> bool:
    return isinstance(s, str) and 3 <= len(s.strip()) <= 260 and bool(PUBLIC_SAFE_REF.match(s.strip()))


@dataclass(frozen=True)
class DurableCheckpointSeal:
    checkpoint_digest_ref: str
    replication_factor: int
    retrieval_verified: bool
    size_bytes: int
    storage_class: str
    window_ref: str
    retrieval_proof_ref: str | None = None
    remote_checkpoint_store_ref: str | None = None
    remote_checkpoint_object_ref: str | None = None
    readback_rehash_receipt_ref: str | None = None


@dataclass(frozen=True)
class SealGate:
    decision: str
    durable: bool
    reasons: tuple[str, ...]
    schema_version: str = SCHEMA_VERSION
    blocker_ref: str = BLOCKER


def evaluate(seal: DurableCheckpointSeal) -> SealGate:
    reasons = []
    if not DIGEST_PATTERN.match(seal.checkpoint_digest_ref or ""):
        reasons.append("checkpoint_digest_not_content_addressed")
    if seal.storage_class not in DURABLE_CONTENT_ADDRESSED:
        reasons.append("storage_class_not_durable_content_addressed")
    if seal.replication_factor < MIN_DURABLE_REPLICATION_FACTOR:
        reasons.append("replication_factor_below_durable_minimum")
    if not seal.retrieval_verified:
        reasons.append("checkpoint_retrieval_not_verified")
    if seal.remote_checkpoint_store_ref is None:
        reasons.append("remote_checkpoint_store_missing")
    if seal.remote_checkpoint_object_ref is None:
        reasons.append("remote_checkpoint_object_ref_missing")
    if seal.readback_rehash_receipt_ref is None:
        reasons.append("readback_rehash_receipt_missing")
    ok = not reasons
    return SealGate(SEAL if ok else HOLD, ok, tuple(reasons))


_CAMEL = {"checkpointDigestRef": "checkpoint_digest_ref", "replicationFactor": "replication_factor",
          "retrievalVerified": "retrieval_verified", "sizeBytes": "size_bytes", "storageClass": "storage_class",
          "windowRef": "window_ref", "retrievalProofRef": "retrieval_proof_ref",
          "remoteCheckpointStoreRef": "remote_checkpoint_store_ref",
          "remoteCheckpointObjectRef": "remote_checkpoint_object_ref",
          "readbackRehashReceiptRef": "readback_rehash_receipt_ref"}


def decode(obj) -> DurableCheckpointSeal | None:
    """Decode an untrusted descriptor (camelCase keys as on the wire).  None if malformed."""
    if not isinstance(obj, dict):
        return None
    kw = {}
    for k, v in obj.items():
        if k not in _CAMEL:
            continue
        kw[_CAMEL[k]] = v
    try:
        s = DurableCheckpointSeal(**kw)
    except TypeError:
        return None
    refs = [s.checkpoint_digest_ref, s.window_ref] + [r for r in (s.retrieval_proof_ref, s.remote_checkpoint_store_ref,
                                                                 s.remote_checkpoint_object_ref,
                                                                 s.readback_rehash_receipt_ref) if r is not None]
    if not all(is_public_safe_ref(r) for r in refs):
        return None
    if s.storage_class not in STORAGE_CLASSES:
        return None
    if not (isinstance(s.replication_factor, int) and 0 <= s.replication_factor <= 1000):
        return None
    if not (isinstance(s.size_bytes, int) and 1 <= s.size_bytes <= 1_099_511_627_776):
        return None
    if not isinstance(s.retrieval_verified, bool):
        return None
    return s


def evaluate_untrusted(obj) -> SealGate:
    """A descriptor that does not decode yields HOLD."""
    s = decode(obj)
    if s is None:
        return SealGate(HOLD, False, ("seal_descriptor_malformed",))
    return evaluate(s)
