"""Instruction tuning: an owned chat template, an assistant-token loss mask, a corpus manifest and a lane report with a
resume drill.

The reference publishes one receipt for this lane (apps/openagents.com/workers/api/src/training-post-training-instruct-sft.ts:53-101,
147-210): a chat template with a digest, a corpus manifest (record count, masked and trainable token totals, manifest
digest, rights posture), a generation-mask fixture, a deterministic smoke run under a cosine schedule with a learning-rate
floor in basis points, a resume drill (checkpoint at step k, the remaining steps resumed, per-step receipts compared) and a
report digest.  The training code itself lives upstream; this module is that code for this framework:

* ``render_example`` turns one conversation into token ids and a 0/1 mask that is 1 exactly on the assistant's tokens and
  the end-of-turn marker that closes them, the tokens the model must learn to produce;
* ``build_corpus`` / ``pack`` make a token shard with that mask for the native loader (``data.shards``); the trainer's
  fused cross-entropy ignores masked targets and averages over the rest;
* ``run_lane`` runs the steps, checkpoints at ``checkpoint_at``, resumes a fresh trainer from that checkpoint for the rest
  and reports whether the restored optimizer state is bit-identical and how far the resumed losses are from the
  uninterrupted ones (the trainer's reductions use floating-point atomics, so losses after a resume agree to rounding,
  not to the bit; the report says which of the two was checked).
"""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass, field

import numpy as np

LANE_ID = "b200_instruct_sft_v1"
TEMPLATE = {
    "templateId": "b200_chat_template", "templateVersion": "v1",
    "roles": {"system": "<|system|>", "user": "<|user|>", "assistant": "<|assistant|>"},
    "endOfTurn": "<|end|>", "afterRoleMarker": "\n", "afterEndOfTurn": "\n",
    "trainable": "assistant content and the end-of-turn marker that closes it",
}
SPECIAL_TOKENS = [TEMPLATE["roles"]["system"], TEMPLATE["roles"]["user"], TEMPLATE["roles"]["assistant"], TEMPLATE["endOfTurn"]]
REPORT_SCHEMA = "b200.training.instruct_sft_lane_report.v1"


def _canon(obj) -> bytes:
    return json.dumps(obj, sort_keys=True, separators=(",", ":"), ensure_ascii=False).encode()


def _sha(obj) -> str:
    return "sha256:" + hashlib.sha256(obj if isinstance(obj, (bytes, bytearray)) else _canon(obj)).hexdigest()


def template_digest() -> str:
    return _sha(TEMPLATE)


def render_text(messages) -> str:
    """The conversation as one string (what a server-side chat template would produce for the same roles)."""
    out = []
    for m in messages:
        out.append(TEMPLATE["roles"][m["role"]] + TEMPLATE["afterRoleMarker"] + m["content"] + TEMPLATE["endOfTurn"] + TEMPLATE["afterEndOfTurn"])
    return "".join(out)


def generation_prompt(messages) -> str:
    """Prefix for inference: the conversation so far plus the assistant header."""
    return render_text(messages) + TEMPLATE["roles"]["assistant"] + TEMPLATE["afterRoleMarker"]


def check_messages(messages, where: str = "messages", need_assistant: bool = True) -> None:
    """Raise ``ValueError`` naming ``where`` unless ``messages`` is a list of ``{"role": system|user|assistant|..., "content": str}``."""
    if not isinstance(messages, list) or not messages:
        raise ValueError(f"{where}: must be a non-empty list of messages")
    for i, m in enumerate(messages):
        if not isinstance(m, dict) or m.get("role") not in TEMPLATE["roles"] or not isinstance(m.get("content"), str):
            raise ValueError(f"{where}[{i}]: a message is {{\"role\": one of {', '.join(TEMPLATE['roles'])}, \"content\": text}}")
    if need_assistant and not any(m["role"] == "assistant" and m["content"] for m in messages):
        raise ValueError(f"{where}: an example needs at least one non-empty assistant message")


def load_records(path: str, preference: bool = False) -> list[dict]:
    """The records of a JSON-lines file (blank lines skipped), each checked: ``{"messages": [...]}`` for instruction tuning,
    plus non-empty ``chosen`` and ``rejected`` answers for preference pairs (whose messages are the prompt turns only).  A bad
    line raises ``ValueError`` with the file name and line number."""
    out = []
    with open(path, encoding="utf-8") as f:
        for n, line in enumerate(f, 1):
            if not line.strip():
                continue
            where = f"{path}:{n}"
            try:
                rec = json.loads(line)
            except ValueError as e:
                raise ValueError(f"{where}: not JSON ({e})") from None
            if not isinstance(rec, dict):
                raise ValueError(f"{where}: a record is a JSON object")
            check_messages(rec.get("messages"), f"{where}: messages", need_assistant=not preference)
            if preference:
                for key in ("chosen", "rejected"):
                    if not isinstance(rec.get(key), str) or not rec[key].strip():
                        raise ValueError(f"{where}: {key} must be a non-empty string")
            out.append(rec)
    if not out:
        raise ValueError(f"{path}: no records")
    return out


def render_example(messages, tokenizer) -> tuple[list[int], list[int]]:
    """Token ids and the loss mask (1 = trainable).  ``tokenizer.encode`` must map the four markers to single ids
    (``data.bpe.ByteBpe`` with ``special=SPECIAL_TOKENS`` does)."""
    check_messages(messages, "example")
    ids: list[int] = []
    mask: list[int] = []
    for m in messages:
        role, content = m.get("role"), m.get("content")
        if role not in TEMPLATE["roles"] or not isinstance(content, str):
            raise ValueError(f"bad message: role {role!r}")
        head = tokenizer.encode(TEMPLATE["roles"][role] + TEMPLATE["afterRoleMarker"])
        body = tokenizer.encode(content)
        end = tokenizer.encode(TEMPLATE["endOfTurn"])
        tail = tokenizer.encode(TEMPLATE["afterEndOfTurn"])
        if len(end) != 1:
            raise ValueError("the tokenizer does not know the end-of-turn marker as one token")
        train = 1 if role == "assistant" else 0
        ids += head + body + end + tail
        mask += [0] * len(head) + [train] * len(body) + [train] + [0] * len(tail)
    return ids, mask


def generation_mask_fixture(messages, tokenizer) -> list[dict]:
    """One row per token: its text and whether it is trained on (for reading a mask by eye and for golden tests)."""
    ids, mask = render_example(messages, tokenizer)
    return [{"id": i, "text": tokenizer.decode([i]), "trainable": bool(m)} for i, m in zip(ids, mask)]


@dataclass
class SftCorpus:
    ids: np.ndarray
    mask: np.ndarray
    manifest: dict
    example_offsets: list[int] = field(default_factory=list)


def build_corpus(records, tokenizer, dataset_identity: str, rights_posture: str = "repo_owned_example_text") -> SftCorpus:
    """``records``: iterable of ``{"messages": [...]}``.  Examples are concatenated in order; the manifest commits to the
    template, the records and the token totals."""
    all_ids, all_mask, offsets, digests = [], [], [], []
    n = 0
    for rec in records:
        if not isinstance(rec, dict):
            raise ValueError(f"record {n}: a record is an object with messages")
        ids, mask = render_example(rec.get("messages"), tokenizer)
        offsets.append(len(all_ids))
        all_ids += ids
        all_mask += mask
        digests.append(_sha([{"role": m["role"], "content": m["content"]} for m in rec["messages"]]))
        n += 1
    if n == 0:
        raise ValueError("empty corpus")
    trainable = int(sum(all_mask))
    manifest = {"datasetIdentity": dataset_identity, "recordCount": n, "rightsPosture": rights_posture,
                "totalTrainableTokens": trainable, "totalMaskedTokens": len(all_ids) - trainable,
                "template": {"templateId": TEMPLATE["templateId"], "templateVersion": TEMPLATE["templateVersion"], "templateDigest": template_digest()},
                "recordDigests": digests, "tokenDigest": _sha(np.asarray(all_ids, dtype=np.int64).tobytes())}
    manifest["manifestDigest"] = _sha(manifest)
    return SftCorpus(np.asarray(all_ids, dtype=np.int64), np.asarray(all_mask, dtype=np.uint8), manifest, offsets)


def pack(corpus: SftCorpus, path, repeat: int = 1) -> dict:
    """Write the corpus as one masked token shard (``repeat`` > 1 tiles a tiny corpus so that it fills a batch)."""
    from ..data import write_token_shard
    return write_token_shard(path, np.tile(corpus.ids, repeat), np.tile(corpus.mask, repeat))


def cosine_lr(step: int, total_steps: int, lr: float, ratio_bps: int = 1000, warmup_steps: int = 0) -> float:
    """Cosine annealing from ``lr`` to ``lr * ratio_bps / 10000`` (the trainer's own schedule has the same shape with a
    floor of 1000 bps)."""
    import math
    if warmup_steps and step < warmup_steps:
        return lr * (step + 1) / warmup_steps
    t = min(1.0, (step - warmup_steps) / max(1, total_steps - warmup_steps))
    floor = ratio_bps / 10000.0
    return lr * (floor + (1.0 - floor) * 0.5 * (1.0 + math.cos(math.pi * t)))


def _state_digest(trainer) -> str:
    h = hashlib.sha256()
    for name in ("master", "m", "v"):
        t = getattr(trainer, name, None)
        if t is not None:
            h.update(t.detach().float().cpu().numpy().tobytes())
    return "sha256:" + h.hexdigest()


def _run_steps(trainer, loader, n: int, device):
    recs = []
    for _ in range(n):
        tok, tgt, n_valid, batch = loader.next()
        tok, tgt = tok.to(device, non_blocking=True), tgt.to(device, non_blocking=True)
        loss = float(trainer.train_step(tok, tgt, n_valid if n_valid < tok.numel() else None))
        recs.append({"step": int(trainer.step_count), "batch": batch, "trainableTokens": n_valid, "loss": loss})
    return recs


def run_lane(make_trainer, make_loader, steps: int, checkpoint_at: int, ckpt_dir: str, corpus_manifest: dict, device="cpu",
             run_id: str = "b200-instruct-sft-smoke", loss_tolerance: float = 5e-3, on_finished=None) -> dict:
    """``make_trainer()`` -> an object with ``train_step(tokens, targets, n_valid)``, ``step_count``, ``save_checkpoint(dir)``,
    ``load_checkpoint(dir)`` and the flat state tensors ``master`` / ``m`` / ``v``; ``make_loader(start_batch)`` -> a
    ``data.BatchLoader``.  ``on_finished(trainer)`` is called with the trainer of the uninterrupted run after its last step
    (export the tuned weights there).  Returns the lane report."""
    if not 0 < checkpoint_at < steps:
        raise ValueError("checkpoint_at must lie inside the run")
    tr = make_trainer()
    ld = make_loader(0)
    first = _run_steps(tr, ld, checkpoint_at, device)
    tr.save_checkpoint(ckpt_dir)
    at_save = _state_digest(tr)
    rest = _run_steps(tr, ld, steps - checkpoint_at, device)
    ld.close()
    straight = first + rest
    if on_finished is not None:
        on_finished(tr)
    del tr, ld                                  # the first trainer's device memory is free before the second is built
    # the drill: a fresh trainer, the checkpoint, the same stream from the same batch
    tr2 = make_trainer()
    tr2.load_checkpoint(ckpt_dir)
    at_load = _state_digest(tr2)
    ld2 = make_loader(checkpoint_at)
    resumed = _run_steps(tr2, ld2, steps - checkpoint_at, device)
    ld2.close()
    diffs = [abs(a["loss"] - b["loss"]) for a, b in zip(rest, resumed)]
    same_stream = all(a["batch"] == b["batch"] and a["trainableTokens"] == b["trainableTokens"] and a["step"] == b["step"] for a, b in zip(rest, resumed))
    losses = [r["loss"] for r in straight]
    report = {
        "schema": REPORT_SCHEMA, "laneId": LANE_ID, "runId": run_id, "completedSteps": steps, "schedulerKind": "cosine_annealing",
        "learningRateRatioBps": 1000, "corpus": {k: corpus_manifest[k] for k in ("datasetIdentity", "recordCount", "rightsPosture", "totalTrainableTokens",
                                                                                   "totalMaskedTokens", "manifestDigest")},
        "template": corpus_manifest["template"], "stepReceipts": straight, "firstLoss": losses[0], "lastLoss": losses[-1],
        "lossImproved": losses[-1] < losses[0],
        "resumeDrill": {"checkpointAtStep": checkpoint_at, "resumedSteps": steps - checkpoint_at, "restoredStateBitExact": at_save == at_load,
                        "sameBatchesAfterResume": same_stream, "postResumeLossMaxAbsDiff": max(diffs) if diffs else 0.0,
                        "postResumeLossesAgree": bool(diffs) and max(diffs) <= loss_tolerance, "lossTolerance": loss_tolerance,
                        "postResumeLossesBitExact": all(d == 0.0 for d in diffs)},
        "paidDispatchState": "not_dispatched",
    }
    report["reportDigest"] = _sha({k: v for k, v in report.items() if k != "stepReceipts"} | {"losses": [round(x, 4) for x in losses]})
    return report
