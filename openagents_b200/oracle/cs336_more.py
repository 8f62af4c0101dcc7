"""CS336 A3 (IsoFLOP sweep cell), A4 (data refinery stages) and A5 (rollouts and reward grading) as CPU
workloads: seeded, deterministic, digest-committed; public-safe outputs (counts, losses, digests, refs).

All randomness is mulberry32 seeded by FNV-1a of a scope string, so that a re-run of a sampled cell
reproduces its digest exactly (the ``deterministic_recompute`` verification class depends on it).

Reference: apps/openagents.com/workers/api/src/cs336-a3-sweep-workload.ts:1-23 (cell definition),
:35-47 (defaults), :141 ``planCs336A3SweepGrid``, :249 ``runCs336A3SweepCell``;
cs336-a4-refinery-workload.ts:111 ``buildCs336A4SyntheticCorpus``, :513 ``runCs336A4RefineryStage``
(PII masking, exact line dedup, Gopher rules, MinHash with 8 bands x 2 rows, 3-token shingles,
Jaccard 0.7); cs336-a5-rollout-workload.ts:222 ``runCs336A5RolloutBatch``, :334
``gradeCs336A5Rollouts`` (group-normalised advantages).
"""
from __future__ import annotations

import hashlib
import json
import math
import re

import numpy as np

from .cs336 import mulberry32

VOCAB = 256
PARAMS_PER_RANK = 2 * VOCAB
EVAL_UNITS = 2048
LEARNING_RATE = 0.3
FLOPS_PER_PARAM_UNIT = 6
DEFAULT_BUDGETS = (300_000_000, 600_000_000, 1_200_000_000, 2_400_000_000)
A3_WORKLOAD_REF = "workload.cs336_a3.seeded_factored_bigram_lm.v1"
A4_WORKLOAD_REF = "workload.cs336_a4.seeded_synthetic_refinery.v1"
A5_WORKLOAD_REF = "workload.cs336_a5.seeded_rollout_and_reference_grading.v1"
A5_TASKSET_REF = "dataset.cs336_a5.bounded_synthetic_math_tasks.v1"


def fnv1a32(text: str) -> int:
    h = 0x811C9DC5
    data = text.encode("utf-16-le", "surrogatepass")
    for i in range(0, len(data), 2):
        h ^= data[i] | (data[i + 1] << 8)
        h = (h * 0x01000193) & 0xFFFFFFFF
    return h


def seeded_random(scope: str):
    return mulberry32(fnv1a32(scope))


def sha256_json(obj) -> str:
    return hashlib.sha256(json.dumps(obj, separators=(",", ":"), ensure_ascii=False).encode()).hexdigest()


# ---------------------------------------------------------------- A3
def plan_sweep_grid(budgets=DEFAULT_BUDGETS, cells_per_budget: int = 6, params_min: int = 1024, params_max: int = 65536) -> list[dict]:
    """Geometric N spacing inside the bounds per compute budget, D = C / (6 N); each planned N is realised
    as the nearest whole factor rank so that a real model can be trained at that point."""
    if not budgets or any(b <= 0 for b in budgets):
        raise ValueError("sweep budgets must be positive")
    if cells_per_budget < 3:
        raise ValueError("a sweep needs at least 3 cells per budget")
    if params_min <= 0 or params_max <= params_min:
        raise ValueError("parameter bounds are invalid")
    lo, hi = math.log(params_min), math.log(params_max)
    cells = []
    for bi, C in enumerate(budgets):
        for i in range(cells_per_budget):
            planned = math.exp(lo + i / (cells_per_budget - 1) * (hi - lo))
            rank = max(1, int(math.floor(planned / PARAMS_PER_RANK + 0.5)))
            n = rank * PARAMS_PER_RANK
            cells.append({"budgetIndex": bi, "cellIndex": len(cells) + 1, "computeBudgetFlops": C, "parameterCount": n,
                          "plannedParameterCount": planned, "rank": rank,
                          "tokenCount": int(math.floor(C / (FLOPS_PER_PARAM_UNIT * n) + 0.5))})
    return cells


def _stream(scope: str):
    """Bigram mixture: two affine successor maps (45 % and 30 %) plus uniform noise."""
    rnd = seeded_random(scope)
    cur = int(rnd() * VOCAB)

    def nxt():
        nonlocal cur
        prev, draw = cur, rnd()
        if draw < 0.45:
            cur = (3 * prev + 11) % VOCAB
        elif draw < 0.75:
            cur = (5 * prev + 29) % VOCAB
        else:
            cur = int(rnd() * VOCAB)
        return prev, cur
    return nxt


def _eval_loss(I: np.ndarray, O: np.ndarray, scope: str) -> float:
    nxt = _stream(scope)
    pairs = np.array([nxt() for _ in range(EVAL_UNITS)])
    logits = I[pairs[:, 0]] @ O.T
    m = logits.max(axis=1, keepdims=True)
    lse = np.log(np.exp(logits - m).sum(axis=1)) + m[:, 0]
    return float((lse - logits[np.arange(EVAL_UNITS), pairs[:, 1]]).mean())


def run_sweep_cell(compute_budget_flops: float, rank: int, shard_digest_hex: str, max_tokens: int | None = None) -> dict:
    """One real bounded training run: a rank-``rank`` factorised bigram model (input and output factor
    tables of 256 rows) trained by single-pass SGD (lr 0.3) over D = C / (6 N) stream units, then scored
    by held-out cross-entropy.  ``max_tokens`` bounds the run for tests (it is part of the digest)."""
    if not (compute_budget_flops > 0 and math.isfinite(compute_budget_flops)):
        raise ValueError("cell compute budget must be positive")
    if not (isinstance(rank, int) and rank >= 1):
        raise ValueError("cell rank must be a positive integer")
    n_params = rank * PARAMS_PER_RANK
    tokens = int(math.floor(compute_budget_flops / (FLOPS_PER_PARAM_UNIT * n_params) + 0.5))
    trained = tokens if max_tokens is None else min(tokens, max_tokens)
    rnd = seeded_random(f"cs336_a3.init.{shard_digest_hex}.{rank}.{compute_budget_flops}")
    I, O = np.empty((VOCAB, rank)), np.empty((VOCAB, rank))
    fi, fo = I.reshape(-1), O.reshape(-1)
    for i in range(fi.size):
        fi[i] = (rnd() - 0.5) * 0.2
        fo[i] = (rnd() - 0.5) * 0.2
    eval_scope = f"cs336_a3.eval.{shard_digest_hex}"
    initial = _eval_loss(I, O, eval_scope)
    nxt = _stream(f"cs336_a3.train.{shard_digest_hex}")
    for _ in range(trained):
        ctx, tgt = nxt()
        x = I[ctx].copy()
        logits = O @ x
        p = np.exp(logits - logits.max())
        err = p / p.sum()
        err[tgt] -= 1.0
        grad_ctx = err @ O                      # with the output factors as they were before this step
        O -= LEARNING_RATE * np.outer(err, x)
        I[ctx] -= LEARNING_RATE * grad_ctx
    final = _eval_loss(I, O, eval_scope)
    # the committed body (:352-363): losses with 17 significant digits; a run cut short for a test also commits to where it stopped
    body = {"computeBudgetFlops": compute_budget_flops, "finalLoss": format(final, ".17g"), "initialLoss": format(initial, ".17g"),
            "parameterCount": n_params, "rank": rank, "shardDigestHex": shard_digest_hex, "tokenCount": tokens}
    if max_tokens is not None:
        body["trainedDataUnits"] = trained
    body["workloadRef"] = A3_WORKLOAD_REF
    return {**body, "trainedDataUnits": trained, "finalLoss": final, "initialLoss": initial, "outputDigestHex": sha256_json(body)}


# ---------------------------------------------------------------- A4
TOPICS = ("the harbor ledger reconciled every settled invoice", "a seeded model trained one bounded pass over synthetic tokens",
          "the validator recomputed the digest and the verdicts matched", "quality rules filtered the document before it reached the corpus",
          "duplicate lines were removed before the shard was committed", "the contributor device returned counts digests and refs only")
BOILERPLATE = "shared boilerplate footer line for the synthetic corpus"
MINHASH_BANDS, MINHASH_ROWS, SHINGLE, NEAR_DUP_JACCARD = 8, 2, 3, 0.7
STAGES = ("pii_masking", "exact_line_dedup", "gopher_rules", "minhash_dedup")
_EMAIL = re.compile(r"[A-Za-z0-9._%+-]+@[A-Za-z0-9.-]+\.[A-Za-z]{2,}")
_PHONE = re.compile(r"\b\d{3}-\d{4}\b")
_IPV4 = re.compile(r"\b(?:\d{1,3}\.){3}\d{1,3}\b")


def build_synthetic_corpus(shard_digest_hex: str, document_count: int = 64, lines_per_document: int = 6) -> list[dict]:
    """Every fourth document repeats its predecessor except for the last line (a near duplicate); some lines
    carry fake contact details, some are symbol soup, the last line of every document is boilerplate."""
    if document_count < 4 or lines_per_document < 2:
        raise ValueError("corpus needs at least 4 documents of at least 2 lines")
    rnd = seeded_random(f"cs336_a4.corpus.{shard_digest_hex}")
    docs = []
    for di in range(document_count):
        near = docs[-1] if di % 4 == 3 and docs else None
        lines = []
        for li in range(lines_per_document):
            if near is not None and li < lines_per_document - 1:
                lines.append(near["lines"][li])
            elif li == lines_per_document - 1:
                lines.append(BOILERPLATE)
            else:
                topic = TOPICS[int(rnd() * len(TOPICS))]
                draw = rnd()
                if draw < 0.18:
                    lines.append(f"contact user{di}@example.invalid or call 555-0{100 + di:03d} from 192.0.2.{di % 254}")
                elif draw < 0.3:
                    lines.append("### $$$ %% @@ ^^ && ** (( )) -- ++ == ~~ ## !!")
                else:
                    lines.append(f"{topic} number {di}.{li}")
        docs.append({"documentRef": f"doc.cs336_a4.{di}", "lines": lines})
    return docs


def pii_masking(docs) -> tuple[list[str], dict]:
    n = {"maskedEmails": 0, "maskedIpv4": 0, "maskedPhones": 0}
    out = []
    for d in docs:
        for line in d["lines"]:
            line, k = _EMAIL.subn("[EMAIL]", line); n["maskedEmails"] += k
            line, k = _IPV4.subn("[IPV4]", line); n["maskedIpv4"] += k
            line, k = _PHONE.subn("[PHONE]", line); n["maskedPhones"] += k
            out.append(line)
    n["maskedTotal"] = n["maskedEmails"] + n["maskedIpv4"] + n["maskedPhones"]
    return out, n


def exact_line_dedup(docs) -> tuple[list[str], dict]:
    seen, kept, total = set(), [], 0
    for d in docs:
        for line in d["lines"]:
            total += 1
            if line not in seen:
                seen.add(line)
                kept.append(line)
    return kept, {"inputLines": total, "removedLines": total - len(kept), "uniqueLines": len(kept)}


def gopher_verdict(text: str) -> str | None:
    chars = list(text)
    words = [w for w in re.split(r"\s+", text) if w]
    if len(words) < 3:
        return "too_few_words"
    if (sum(c.isascii() and c.isalpha() for c in chars) / len(chars) if chars else 0) < 0.6:
        return "low_alpha_ratio"
    if chars and sum(c in "#$%^&*()-+=~!" for c in chars) / len(chars) > 0.1:
        return "symbol_heavy"
    return None


def gopher_rules(docs) -> tuple[list[str], dict]:
    kept, rej = [], {"too_few_words": 0, "low_alpha_ratio": 0, "symbol_heavy": 0}
    for d in docs:
        v = gopher_verdict(" ".join(d["lines"]))
        if v is None:
            kept.append(d["documentRef"])
        else:
            rej[v] += 1
    return kept, {"inputDocuments": len(docs), "keptDocuments": len(kept), "rejectedLowAlphaRatio": rej["low_alpha_ratio"],
                  "rejectedSymbolHeavy": rej["symbol_heavy"], "rejectedTooFewWords": rej["too_few_words"]}


def _shingles(doc) -> set[int]:
    toks = [t for t in re.split(r"[^a-z0-9]+", " ".join(doc["lines"]).lower()) if t]
    s = {fnv1a32(" ".join(toks[i:i + SHINGLE])) for i in range(len(toks) - SHINGLE + 1)}
    if not s and toks:
        s.add(fnv1a32(" ".join(toks)))
    return s


def _jaccard(a: set, b: set) -> float:
    if not a and not b:
        return 1.0
    inter = len(a & b)
    return inter / (len(a) + len(b) - inter)


def minhash_dedup(docs, shard_digest_hex: str) -> tuple[list[str], dict]:
    """Banded MinHash finds candidate pairs; a pair is merged only when its exact Jaccard over 3-token
    shingles reaches 0.7; each cluster keeps its lowest-numbered document."""
    P = MINHASH_BANDS * MINHASH_ROWS
    rnd = seeded_random(f"cs336_a4.minhash.{shard_digest_hex}")
    seeds = [(int(rnd() * 0xFFFFFFFF) & 0xFFFFFFFF) | 1 for _ in range(P)]
    sets = [_shingles(d) for d in docs]
    sigs = []
    for s in sets:
        sig = [0xFFFFFFFF] * P
        for sh in s:
            for i in range(P):
                h = ((sh ^ seeds[i]) * 0x01000193) & 0xFFFFFFFF
                if h < sig[i]:
                    sig[i] = h
        sigs.append(sig)
    parent = list(range(len(docs)))

    def find(x):
        while parent[x] != x:
            parent[x] = parent[parent[x]]
            x = parent[x]
        return x

    pairs = 0
    for band in range(MINHASH_BANDS):
        buckets: dict[tuple, list[int]] = {}
        for di, sig in enumerate(sigs):
            buckets.setdefault(tuple(sig[band * MINHASH_ROWS:(band + 1) * MINHASH_ROWS]), []).append(di)
        for bucket in buckets.values():
            for i, a in enumerate(bucket):
                for b in bucket[i + 1:]:
                    ra, rb = find(a), find(b)
                    if ra != rb and _jaccard(sets[a], sets[b]) >= NEAR_DUP_JACCARD:
                        parent[max(ra, rb)] = min(ra, rb)
                        pairs += 1
    kept = [docs[i]["documentRef"] for i in range(len(docs)) if find(i) == i]
    return kept, {"confirmedNearDuplicatePairs": pairs, "inputDocuments": len(docs), "keptDocuments": len(kept),
                  "nearDuplicateClusters": len({find(i) for i in range(len(docs))}), "removedDocuments": len(docs) - len(kept)}


def run_refinery_stage(stage: str, shard_digest_hex: str, document_count: int = 64, lines_per_document: int = 6) -> dict:
    if stage not in STAGES:
        raise ValueError(f"unknown refinery stage {stage!r}")
    docs = build_synthetic_corpus(shard_digest_hex, document_count, lines_per_document)
    body, stats = {"pii_masking": pii_masking, "exact_line_dedup": exact_line_dedup, "gopher_rules": gopher_rules,
                   "minhash_dedup": lambda d: minhash_dedup(d, shard_digest_hex)}[stage](docs)
    digest = sha256_json({"output": body, "shardDigestHex": shard_digest_hex, "stage": stage, "stats": stats, "workloadRef": A4_WORKLOAD_REF})
    return {"stage": stage, "inputDocumentCount": len(docs), "stats": stats, "outputDigestHex": digest, "workloadRef": A4_WORKLOAD_REF}


# ---------------------------------------------------------------- A5
_TEMPLATES = (
    (lambda a, b, c: (a + b) * c, "A crate holds {a} parts plus {b} spares. With {c} crates total, how many parts are there?"),
    (lambda a, b, c: a * b - c, "Each of {a} shelves holds {b} units. After removing {c} units, how many remain?"),
    (lambda a, b, c: a + b * c, "A ledger starts at {a} entries and gains {b} entries on each of {c} days. How many entries result?"),
    (lambda a, b, c: a * c + b * c, "A route makes {c} trips carrying {a} boxes and {b} bags each trip. How many items move in total?"),
)
ADVANTAGE_EPS = 1e-6


def build_tasks(shard_digest_hex: str, split_ref: str, task_count: int = 32) -> list[dict]:
    if task_count < 4:
        raise ValueError("a task set needs at least 4 tasks")
    rnd = seeded_random(f"cs336_a5.tasks.{shard_digest_hex}.{split_ref}")
    tasks = []
    for i in range(task_count):
        fn, text = _TEMPLATES[int(rnd() * len(_TEMPLATES))]
        a, b, c = 2 + int(rnd() * 18), 2 + int(rnd() * 18), 2 + int(rnd() * 8)
        tasks.append({"difficulty": rnd(), "referenceValue": fn(a, b, c), "taskRef": f"task.cs336_a5.{split_ref}.{i}",
                      "taskText": text.format(a=a, b=b, c=c)})
    return tasks


def sample_rollout(seed_scope: str, task: dict, rollout_index: int) -> dict:
    rnd = seeded_random(f"{seed_scope}.{task['taskRef']}.{rollout_index}")
    correct = rnd() < 0.35 + 0.5 * task["difficulty"]
    malformed = rnd() < 0.05
    off = (1 + int(rnd() * 3)) * (-1 if rnd() < 0.5 else 1)
    value = task["referenceValue"] if correct else task["referenceValue"] + off
    line = f"Working through the quantities step by step gives {value}."
    text = f"{line}\nThe final value is {value}" if malformed else f"{line}\n#### {value}"
    return {"completionText": text, "rolloutIndex": rollout_index, "taskRef": task["taskRef"]}


def run_rollout_batch(shard_digest_hex: str, split_ref: str, task_count: int = 32, rollouts_per_task: int = 4) -> dict:
    if rollouts_per_task < 2:
        raise ValueError("rollout batches need at least 2 rollouts per task")
    tasks = build_tasks(shard_digest_hex, split_ref, task_count)
    scope = f"cs336_a5.rollout.{shard_digest_hex}.{split_ref}"
    rollouts = [sample_rollout(scope, t, i) for t in tasks for i in range(rollouts_per_task)]
    digest = sha256_json({"rollouts": rollouts, "shardDigestHex": shard_digest_hex, "splitRef": split_ref,
                          "taskSetDatasetRef": A5_TASKSET_REF, "workloadRef": A5_WORKLOAD_REF})
    return {"rollouts": rollouts, "tasks": tasks, "splitRef": split_ref, "outputDigestHex": digest,
            "stats": {"meanCompletionChars": round(sum(len(r["completionText"]) for r in rollouts) / len(rollouts)),
                      "rolloutCount": len(rollouts), "rolloutsPerTask": rollouts_per_task, "taskCount": len(tasks)}}


_FINAL = re.compile(r"^####\s*(-?[\d,]+)\s*$", re.M)


def parse_final_value(text: str) -> int | None:
    m = _FINAL.findall(text)
    if not m:
        return None
    try:
        v = int(m[-1].replace(",", ""))
    except ValueError:
        return None
    return v if abs(v) <= 2 ** 53 - 1 else None


def grade_rollouts(rollouts: list[dict], tasks: list[dict], split_ref: str) -> dict:
    """Reward 1 for a parsed final value equal to the reference, else 0; advantages are the rewards
    normalised inside each task's group (zero for a group without variance)."""
    if not rollouts:
        raise ValueError("grading needs at least one rollout")
    ref = {t["taskRef"]: t["referenceValue"] for t in tasks}
    groups: dict[str, list[int]] = {}
    correct = unparseable = 0
    for r in rollouts:
        if r["taskRef"] not in ref:
            raise ValueError("grading saw a rollout for an unknown task ref")
        v = parse_final_value(r["completionText"])
        unparseable += v is None
        reward = int(v is not None and v == ref[r["taskRef"]])
        correct += reward
        groups.setdefault(r["taskRef"], []).append(reward)
    graded, zero_var = [], 0
    for task_ref in sorted(groups):
        rw = groups[task_ref]
        mean = sum(rw) / len(rw)
        std = math.sqrt(sum((x - mean) ** 2 for x in rw) / len(rw))
        zero_var += std == 0
        graded.append({"advantages": [f"{0 if std == 0 else (x - mean) / (std + ADVANTAGE_EPS):.6f}" for x in rw], "rewards": rw, "taskRef": task_ref})
    acc = correct / len(rollouts)
    digest = sha256_json({"accuracyBp": round(acc * 10000), "correctCount": correct, "gradedGroups": graded,
                          "gradedRolloutCount": len(rollouts), "inputRolloutDigestHex": sha256_json(rollouts), "splitRef": split_ref,
                          "unparseableCount": unparseable, "workloadRef": A5_WORKLOAD_REF})
    return {"accuracy": acc, "outputDigestHex": digest, "splitRef": split_ref, "gradedGroups": graded,
            "stats": {"accuracyBp": round(acc * 10000), "correctCount": correct, "gradedRolloutCount": len(rollouts),
                      "groupCount": len(graded), "unparseableCount": unparseable, "zeroVarianceGroupCount": zero_var}}


def eval_suite_summary(gradings: list[dict], split_ref: str, verified_digests: list[str]) -> dict:
    if not gradings:
        raise ValueError("an eval suite summary needs at least one grading result")
    n = sum(g["stats"]["gradedRolloutCount"] for g in gradings)
    c = sum(g["stats"]["correctCount"] for g in gradings)
    v = sum(g["stats"]["gradedRolloutCount"] for g in gradings if g["outputDigestHex"] in verified_digests)
    return {"metric": "accuracy", "sampleCount": n, "score": c / n if n else 0, "splitRef": split_ref, "taskSetRef": "math",
            "verifiedSampleCount": v}
