"""The attach-only client a node runtime uses against a local model server: doctor, smoke, and a completion with a tool loop.

The reference's node runtime attached to an already running local server and never started one
(apps/pylon/docs/2026-06-09-pylon-qwen35-local-inference-roadmap.md: base-URL resolution :216-217, the health contract
:232-236, model-row admission :281-296, the tool loop and its receipts :352-364; its commands were ``backend psionic doctor`` and
``backend psionic smoke``, apps/pylon/packages/runtime/src/cli.ts:136-141, 311-354).  The same three operations against this
package's server:

* ``doctor``: ``GET /health`` must name an accepted execution engine and list ``/v1/chat/completions``; ``GET /v1/models`` rows are
  admitted only with a verified artifact digest or a public-safe manifest ref;
* ``smoke``: one short greedy completion on an admitted model, with its usage counts;
* ``complete``: lower a provider-neutral request to OpenAI chat messages and function tools, run the tool loop (streamed
  ``delta.tool_calls`` are re-assembled), and emit a content-redacted transcript (roles, lengths, SHA-256 of each message) plus
  one receipt per tool call; prompts, answers and tool arguments never leave the node in those records.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import re
import sys
import urllib.error
import urllib.parse
import urllib.request

from ..utils.cli import cli_entry
from .tools import LlmRequest, ToolCallDeltaAssembler, parse_sse, run_tool_loop

DEFAULT_BASE_URL = "http://127.0.0.1:8080/v1"
BASE_URL_ENV = ("PYLON_PSIONIC_BASE_URL", "PROBE_PSIONIC_BASE_URL")
ACCEPTED_ENGINES = ("psionic", "b200")
_DIGEST = re.compile(r"^sha256:[0-9a-f]{64}$")
_SAFE_REF = re.compile(r"^[A-Za-z0-9][A-Za-z0-9_.:/-]{2,200}$")


def resolve_base_url(flag: str | None = None, env=None) -> str:
    """Command line first, then the two environment variables in order, then the default."""
    env = os.environ if env is None else env
    for v in (flag, *[env.get(k) for k in BASE_URL_ENV]):
        if isinstance(v, str) and v.strip():
            return v.strip().rstrip("/")
    return DEFAULT_BASE_URL


def admit_model_row(row: dict) -> dict:
    digest, manifest = row.get("artifact_digest"), row.get("manifest_ref")
    ok_digest = isinstance(digest, str) and bool(_DIGEST.match(digest))
    ok_manifest = isinstance(manifest, str) and bool(_SAFE_REF.match(manifest)) and "/Users/" not in manifest and "/home/" not in manifest
    blockers = [] if (ok_digest or ok_manifest) else ["blocker.model_row.no_verified_artifact_digest_or_manifest_ref"]
    return {"id": row.get("id"), "admitted": not blockers, "blockerRefs": blockers, "artifactDigest": digest if ok_digest else None,
            "manifestRef": manifest if ok_manifest else None}


class AttachClient:
    def __init__(self, base_url: str | None = None, api_key: str | None = None, opener=urllib.request.urlopen, timeout_s: float = 120.0):
        self.base_url, self.api_key, self.opener, self.timeout_s = resolve_base_url(base_url), api_key, opener, timeout_s

    def _root(self) -> str:
        return self.base_url[:-3] if self.base_url.endswith("/v1") else self.base_url

    def _request(self, url: str, body: dict | None = None):
        headers = {"Content-Type": "application/json", **({"Authorization": f"Bearer {self.api_key}"} if self.api_key else {})}
        req = urllib.request.Request(url, data=None if body is None else json.dumps(body).encode(), headers=headers, method="GET" if body is None else "POST")
        return self.opener(req, timeout=self.timeout_s)

    def _json(self, url: str, body: dict | None = None) -> dict:
        with self._request(url, body) as r:
            return json.loads(r.read())

    # ---- session turns (the routes the local foundation-model bridge of the reference exposes:
    # packages/apple-fm-runtime/native/foundation-bridge/Sources/foundation-bridge/main.swift:472-494)
    def create_session(self, model: str | None = None, instructions: str | None = None) -> str:
        body = {k: v for k, v in (("model", model), ("instructions", instructions)) if v is not None}
        return self._json(self._root() + "/v1/sessions", body)["id"]

    def stream_turn(self, session_id: str, prompt: str, **options):
        """Yields ``("snapshot", text_so_far)`` as the answer grows, then ``("completed", {output, model, usage, ...})``.
        A failure after the stream began arrives as an ``error`` event and is raised here."""
        url = self._root() + f"/v1/sessions/{urllib.parse.quote(session_id, safe='')}/responses/stream"
        event = None
        with self._request(url, {"prompt": prompt, **options}) as r:
            for line in r:
                line = line.decode().rstrip("\r\n")
                if line.startswith("event: "):
                    event = line[7:]
                elif line.startswith("data: ") and event:
                    data = json.loads(line[6:])
                    if event == "snapshot":
                        yield ("snapshot", data["content"])
                    elif event == "completed":
                        yield ("completed", data)
                    elif event == "error":
                        raise RuntimeError(data.get("message") or "the turn failed")
                    event = None

    def doctor(self) -> dict:
        blockers, engine, endpoints, rows = [], None, [], []
        try:
            h = self._json(self._root() + "/health")
            engine, endpoints = h.get("execution_engine"), list(h.get("endpoints") or [])
            if engine not in ACCEPTED_ENGINES:
                blockers.append("blocker.attach.execution_engine_not_accepted")
            if "/v1/chat/completions" not in endpoints:
                blockers.append("blocker.attach.chat_completions_not_listed")
            rows = [admit_model_row(m) for m in self._json(self.base_url + "/models").get("data", [])]
            if not any(r["admitted"] for r in rows):
                blockers.append("blocker.attach.no_admitted_model")
        except (urllib.error.URLError, OSError, ValueError) as e:
            blockers.append("blocker.attach.server_unreachable")
            return {"ok": False, "baseUrl": self.base_url, "blockerRefs": blockers, "detail": f"{type(e).__name__}", "executionEngine": None, "endpoints": [], "models": []}
        return {"ok": not blockers, "baseUrl": self.base_url, "blockerRefs": blockers, "executionEngine": engine, "endpoints": endpoints, "models": rows}

    def smoke(self, model: str | None = None) -> dict:
        d = self.doctor()
        if not d["ok"]:
            return {"ok": False, "blockerRefs": d["blockerRefs"]}
        model = model or next(r["id"] for r in d["models"] if r["admitted"])
        if not any(r["id"] == model and r["admitted"] for r in d["models"]):
            return {"ok": False, "blockerRefs": ["blocker.attach.model_not_admitted"]}
        r = self._json(self.base_url + "/chat/completions", {"model": model, "messages": [{"role": "user", "content": "Reply with one word."}], "max_tokens": 4, "temperature": 0})
        u = r.get("usage") or {}
        ok = r.get("object") == "chat.completion" and isinstance(u.get("completion_tokens"), int) and u["completion_tokens"] >= 1
        return {"ok": ok, "model": model, "finishReason": r["choices"][0].get("finish_reason"), "usage": {k: u.get(k) for k in ("prompt_tokens", "completion_tokens", "total_tokens")},
                "blockerRefs": [] if ok else ["blocker.attach.smoke_completion_malformed"]}

    def _complete_once(self, body: dict, stream: bool) -> dict:
        if not stream:
            return self._json(self.base_url + "/chat/completions", body)
        asm, finish, usage = ToolCallDeltaAssembler(), None, None
        with self._request(self.base_url + "/chat/completions", {**body, "stream": True}) as r:
            for chunk in parse_sse(r):
                for ch in chunk.get("choices", []):
                    asm.feed(ch.get("delta") or {})
                    finish = ch.get("finish_reason") or finish
                usage = chunk.get("usage") or usage
        msg = {"role": "assistant", "content": asm.content or None}
        calls = asm.result()
        if calls:
            msg["tool_calls"] = calls
        return {"object": "chat.completion", "choices": [{"index": 0, "message": msg, "finish_reason": finish}], "usage": usage}

    def complete(self, request: LlmRequest, tool_impls: dict | None = None, max_steps: int = 8, stream: bool = False) -> dict:
        """Returns the final message, the number of round trips, a redacted transcript and one receipt per tool call."""
        usage_total = {"prompt_tokens": 0, "completion_tokens": 0}

        def once(body):
            r = self._complete_once(body, stream)
            for k in usage_total:
                usage_total[k] += int((r.get("usage") or {}).get(k) or 0)
            return r
        out = run_tool_loop(once, request, tool_impls or {}, max_steps)

        def digest(x) -> str:
            return "sha256:" + hashlib.sha256((x if isinstance(x, str) else json.dumps(x, sort_keys=True)).encode()).hexdigest()
        transcript, receipts = [], []
        for m in out["transcript"]:
            content = m.get("content") or ""
            transcript.append({"role": m["role"], "contentChars": len(content), "contentDigest": digest(content), "toolCalls": len(m.get("tool_calls") or [])})
            for c in m.get("tool_calls") or []:
                receipts.append({"toolCallRef": f"toolcall.{(c.get('id') or 'call')}", "tool": c["function"]["name"], "argumentsDigest": digest(c["function"]["arguments"] or "{}"),
                                 "resultDigest": None})
        results = {m["tool_call_id"]: m for m in out["transcript"] if m.get("role") == "tool"}
        for r in receipts:
            res = results.get(r["toolCallRef"][len("toolcall."):])
            if res is not None:
                r["resultDigest"] = digest(res["content"])
                r["failed"] = res["content"].startswith('{"error"')
        return {"message": out["message"], "steps": out["steps"], "usage": {**usage_total, "total_tokens": sum(usage_total.values())},
                "redactedTranscript": transcript, "toolCallReceipts": receipts}


@cli_entry("b200-attach")
def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m openagents_b200.serve.attach_client")
    ap.add_argument("command", choices=["doctor", "smoke"])
    ap.add_argument("--base-url", default=None)
    ap.add_argument("--api-key", default=None)
    ap.add_argument("--model", default=None)
    a = ap.parse_args(argv)
    c = AttachClient(a.base_url, a.api_key)
    out = c.doctor() if a.command == "doctor" else c.smoke(a.model)
    print(json.dumps(out))
    return 0 if out["ok"] else 3


if __name__ == "__main__":
    sys.exit(main())
