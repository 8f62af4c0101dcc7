"""Serving traces -> supervised examples.

The reference names trace-to-training conversion beside the tokenizer and the refinery as the jobs of its upstream data
crate (``psionic-data``), and its data-market plan sells redacted conversation bundles
(docs/2026-06-10-cs336-distributed-homework-continuation-audit.md:286-295).  A trace here is what an OpenAI-compatible
server sees: the request's ``messages`` (and ``tools``), the ``response`` it produced and, optionally, an ``outcome`` label
from whoever consumed it.  ``traces_to_records`` keeps a trace only when the answer finished normally and was not
rejected, folds tool calls and tool results into the template's three roles, masks contact details in every message,
drops exact duplicates, and reports why each dropped trace was dropped.  The records feed ``train.sft.build_corpus``.
"""
from __future__ import annotations

import hashlib
import json

from ..oracle import cs336_more as a4

DROP_REASONS = ("rejected_outcome", "unfinished_answer", "empty_answer", "malformed", "duplicate", "too_long")


def _mask(text: str) -> tuple[str, int]:
    lines, stats = a4.pii_masking([{"documentRef": "m", "lines": text.split("\n")}])
    return "\n".join(lines), stats["maskedTotal"]


def _fold(message: dict) -> dict | None:
    """One OpenAI message -> a system / user / assistant message of the training template."""
    role, content = message.get("role"), message.get("content")
    if isinstance(content, list):                                        # content parts: keep the text parts
        content = "".join(p.get("text", "") for p in content if isinstance(p, dict) and p.get("type") == "text")
    content = content or ""
    if role in ("system", "developer"):
        return {"role": "system", "content": content}
    if role == "user":
        return {"role": "user", "content": content}
    if role == "tool":                                                   # a tool result is input the model reads
        return {"role": "user", "content": f"[tool result {message.get('tool_call_id', '')}]\n{content}".strip()}
    if role == "assistant":
        calls = message.get("tool_calls") or []
        if calls:
            rendered = [json.dumps({"name": c["function"]["name"], "arguments": json.loads(c["function"].get("arguments") or "{}")}, sort_keys=True)
                        for c in calls]
            content = (content + "\n" if content else "") + "\n".join(f"[tool call] {r}" for r in rendered)
        return {"role": "assistant", "content": content}
    return None


def trace_to_record(trace: dict) -> tuple[dict | None, str | None, int]:
    """(record, drop reason, masked spans)."""
    try:
        if trace.get("outcome") in ("rejected", "failed", "refused"):
            return None, "rejected_outcome", 0
        choice = trace["response"]["choices"][0]
        if choice.get("finish_reason") not in ("stop", "tool_calls"):
            return None, "unfinished_answer", 0
        msgs = [_fold(m) for m in list(trace["messages"]) + [choice["message"]]]
        if any(m is None for m in msgs):
            return None, "malformed", 0
    except (KeyError, IndexError, TypeError, ValueError):
        return None, "malformed", 0
    if not msgs[-1]["content"].strip():
        return None, "empty_answer", 0
    masked = 0
    out = []
    for m in msgs:
        text, k = _mask(m["content"])
        masked += k
        if out and out[-1]["role"] == m["role"]:                         # consecutive tool results / system notes merge
            out[-1]["content"] += "\n" + text
        else:
            out.append({"role": m["role"], "content": text})
    return {"messages": out}, None, masked


def traces_to_records(traces, max_chars: int = 200_000) -> tuple[list[dict], dict]:
    records, seen = [], set()
    drops = {r: 0 for r in DROP_REASONS}
    masked = 0
    for t in traces:
        rec, why, k = trace_to_record(t)
        if rec is not None and sum(len(m["content"]) for m in rec["messages"]) > max_chars:
            rec, why = None, "too_long"
        if rec is not None:
            key = hashlib.sha256(json.dumps(rec, sort_keys=True).encode()).hexdigest()
            if key in seen:
                rec, why = None, "duplicate"
            else:
                seen.add(key)
        if rec is None:
            drops[why] += 1
            continue
        masked += k
        records.append(rec)
    n = len(records) + sum(drops.values())
    return records, {"inputTraces": n, "records": len(records), "dropped": drops, "maskedSpans": masked,
                     "recordsDigest": "sha256:" + hashlib.sha256(json.dumps(records, sort_keys=True).encode()).hexdigest()}
