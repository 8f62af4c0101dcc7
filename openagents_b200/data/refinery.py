"""Text refinery: the four deterministic stages run as a pipeline over real documents.

The reference's A4 workload defines the stages one at a time over a synthetic corpus (PII masking, exact line
de-duplication, Gopher-style quality rules, MinHash near-duplicate removal;
apps/openagents.com/workers/api/src/cs336-a4-refinery-workload.ts:111, :513; restated in ``oracle.cs336_more``) and
its continuation audit calls them the seed of an owned data refinery (docs/2026-06-10-cs336-distributed-homework-continuation-audit.md:280-295).
``refine`` chains the same stage functions: mask contact details in every line, drop lines that occur more than
``max_line_repeats`` times across the corpus (boilerplate), drop documents the quality rules reject, drop near
duplicates (each cluster keeps its first document).  The report carries every stage's counters and a digest of the output.
"""
from __future__ import annotations

import hashlib
import json

from ..oracle import cs336_more as a4

STAGES = ("pii_masking", "exact_line_dedup", "gopher_rules", "minhash_dedup")


def documents_from_texts(texts, prefix: str = "doc") -> list[dict]:
    return [{"documentRef": f"{prefix}.{i}", "lines": [ln for ln in t.splitlines() if ln.strip()]} for i, t in enumerate(texts)]


def refine(docs: list[dict], stages=STAGES, seed: str = "refinery", max_line_repeats: int = 1) -> tuple[list[dict], dict]:
    """``docs``: ``{"documentRef", "lines"}``.  Returns the surviving documents (lines possibly masked or removed) and the
    report.  ``max_line_repeats``: a line may occur this many times over the whole corpus; further copies are dropped
    (1 = every line once, the reference stage's rule)."""
    unknown = [s for s in stages if s not in STAGES]
    if unknown:
        raise ValueError(f"unknown stages {unknown}")
    docs = [{"documentRef": d["documentRef"], "lines": list(d["lines"])} for d in docs]
    report = {"inputDocuments": len(docs), "inputLines": sum(len(d["lines"]) for d in docs), "stages": []}
    for stage in stages:
        if stage == "pii_masking":
            flat, stats = a4.pii_masking(docs)
            at = 0
            for d in docs:
                d["lines"] = flat[at: at + len(d["lines"])]
                at += len(d["lines"])
        elif stage == "exact_line_dedup":
            seen: dict[str, int] = {}
            removed = 0
            for d in docs:
                kept = []
                for ln in d["lines"]:
                    n = seen.get(ln, 0)
                    seen[ln] = n + 1
                    if n < max_line_repeats:
                        kept.append(ln)
                    else:
                        removed += 1
                d["lines"] = kept
            stats = {"removedLines": removed, "uniqueLines": len(seen)}
            docs = [d for d in docs if d["lines"]]
        elif stage == "gopher_rules":
            keep, stats = a4.gopher_rules(docs)
            keep = set(keep)
            docs = [d for d in docs if d["documentRef"] in keep]
        else:
            keep, stats = a4.minhash_dedup(docs, seed)
            keep = set(keep)
            docs = [d for d in docs if d["documentRef"] in keep]
        report["stages"].append({"stage": stage, "stats": stats, "documentsAfter": len(docs)})
    report["outputDocuments"] = len(docs)
    report["outputLines"] = sum(len(d["lines"]) for d in docs)
    report["outputDigest"] = "sha256:" + hashlib.sha256(json.dumps([[d["documentRef"], d["lines"]] for d in docs], separators=(",", ":")).encode()).hexdigest()
    return docs, report
