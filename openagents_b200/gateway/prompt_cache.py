"""Prefix-cache-friendly prompt layout and cache-affinity keys.

A KV prefix cache only hits when two prompts share their leading tokens, so everything stable
(acceptance contract, identity, tool schemas, stable policy, other system text) goes first in a fixed
order and everything volatile keeps its own order after it.  The stable prefix is hashed (FNV-1a 32
over UTF-16 code units, the same function the serving engine's callers use to key sessions) so two
requests can be compared without their text.

Reference: inference/prompt-prefix-cache.ts:1-45 (rule), :194 ``assembleStablePromptLayout``, :324
``deriveCacheAffinityKey``, :361 ``sessionAffinityParams``; ``hashCacheAffinityKey`` in
inference/khala-telemetry.ts.
"""
from __future__ import annotations

import json

STABLE_ORDINAL = {"acceptanceContract": 0, "identity": 1, "toolSchemas": 2, "stablePolicy": 3, "otherSystem": 4}
SESSION_AFFINITY_PARAM = "x-session-affinity"
OPENAI_USER_PARAM = "user"


def _fnv1a32_utf16(text: str) -> int:
    h = 0x811C9DC5
    data = text.encode("utf-16-le", "surrogatepass")
    for i in range(0, len(data), 2):
        h ^= data[i] | (data[i + 1] << 8)
        h = (h * 0x01000193) & 0xFFFFFFFF
    return h


def hash_stable_prefix(text: str) -> str:
    return f"prefix:fnv1a32:{_fnv1a32_utf16(text):08x}"


def hash_cache_affinity_key(raw_key: str) -> str:
    return f"cacheaff:fnv1a32:{_fnv1a32_utf16(raw_key):08x}"


def assemble_stable_prompt_layout(tagged: list) -> dict:
    """``tagged``: list of ``(message, stable_kind_or_None)``; a message is ``{"role", "content"}``.
    Stable blocks sort by their kind's ordinal (ties keep input order), volatile messages follow in
    input order."""
    entries, vol = [], 0
    for idx, (msg, kind) in enumerate(tagged):
        if kind is not None:
            entries.append((STABLE_ORDINAL[kind], idx, msg, "stable"))
        elif msg.get("role") == "system":
            entries.append((STABLE_ORDINAL["otherSystem"], idx, msg, "stable"))
        else:
            entries.append((1000 + vol, idx, msg, "volatile"))
            vol += 1
    entries.sort(key=lambda e: (e[0], e[1]))
    prefix = "".join(f"{m['role']}:{m['content']}" for _, _, m, st in entries if st == "stable")
    return {"messages": [m for _, _, m, _ in entries],
            "classified": [{"message": m, "stability": st, "stableOrdinal": o} for o, _, m, st in entries],
            "stablePrefixText": prefix, "stablePrefixHash": hash_stable_prefix(prefix)}


def canonical_json(value) -> str:
    """JSON with object keys sorted at every depth, no spaces."""
    if isinstance(value, dict):
        return "{" + ",".join(f"{json.dumps(k)}:{canonical_json(value[k])}" for k in sorted(value)) + "}"
    if isinstance(value, (list, tuple)):
        return "[" + ",".join(canonical_json(v) for v in value) + "]"
    return json.dumps(value, ensure_ascii=False)


def serialize_tool_schemas(tools: list) -> str:
    """Tool list in name order, canonical JSON per tool: the same tool set always yields the same text."""
    def name(t):
        if isinstance(t, dict):
            if isinstance(t.get("name"), str):
                return t["name"]
            fn = t.get("function")
            if isinstance(fn, dict) and isinstance(fn.get("name"), str):
                return fn["name"]
        return canonical_json(t)

    return "\n".join(canonical_json(t) for t in sorted(tools, key=name))


def derive_cache_affinity_key(account: str, session: str | None = None, codebase: str | None = None) -> str:
    return "".join((f"acct={account}", f"sess={session or ''}", f"code={codebase or ''}"))


def session_affinity_params(affinity_value: str) -> dict:
    return {OPENAI_USER_PARAM: affinity_value, SESSION_AFFINITY_PARAM: affinity_value}


def reconcile_usage_tokens(prompt: int, completion: int, total: int, cached_prompt: int | None = None) -> dict:
    un = max(0, total - (prompt + completion))
    return {"promptTokens": prompt, "completionTokens": completion, "totalTokens": total, "cachedPromptTokens": cached_prompt,
            "unaccountedTokens": un, "hasUnaccountedTokens": un > 0}
