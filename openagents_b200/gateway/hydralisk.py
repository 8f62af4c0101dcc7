"""OpenAI-compatible adapter to owner-run serving hosts, and the replica pool in front of several of them.

The reference's Hydralisk lane talks to vLLM hosts over the OpenAI chat-completions API but stays receipt-first:
a non-streaming answer without terminal usage is an error, and a streamed answer must carry usage in its last
frames (inference/hydralisk-adapter.ts:1-8).  The pool keeps per-replica routing state (health, warmth, in-flight
count and cap, queue depth, last 429, observed TTFT and tokens/s), ranks eligible replicas, honours a
cache-affinity hint, and applies one of three saturation policies (:44-79, 107-117).  Selection and saturation
logic live in ``evidence.py`` (``select_replica`` / ``dispatch_to_pool`` / ``route_admission``); this module adds
the HTTP client and the stateful pool adapter that plugs into the provider registry.

The server of this package (``serve/server.py``) speaks the same API, so a pool of its instances is the
"Psionic replicas behind one gateway id" deployment; ``tests/test_hydralisk.py`` runs the adapter against it.
"""
from __future__ import annotations

import json
import threading
import time
import urllib.error
import urllib.request

from . import prompt_cache as pc
from .evidence import default_saturation_policy, dispatch_to_pool, replica_state, route_admission
from .fabric import InferenceAdapterError, InferenceRequest, InferenceResult, InferenceUsage, classify_status

_PASS = ("max_tokens", "temperature", "top_p", "top_k", "stop", "seed", "tools", "tool_choice", "user")


def _usage(u) -> InferenceUsage | None:
    if not isinstance(u, dict):
        return None
    p, c = u.get("prompt_tokens"), u.get("completion_tokens")
    if not isinstance(p, int) or not isinstance(c, int) or p < 0 or c < 0:
        return None
    t = u.get("total_tokens")
    cached = (u.get("prompt_tokens_details") or {}).get("cached_tokens") if isinstance(u.get("prompt_tokens_details"), dict) else None
    return InferenceUsage(p, c, t if isinstance(t, int) else p + c, cached if isinstance(cached, int) else None)


class HydraliskAdapter:
    """One host.  ``opener`` is ``urllib.request.urlopen``-shaped and injectable."""

    def __init__(self, id: str, api_key: str, base_url: str, opener=urllib.request.urlopen, upstream_model: str | None = None,
                 timeout_s: float = 120.0):
        self.id, self._key, self.base_url, self.opener = id, api_key, base_url.rstrip("/"), opener
        self.upstream_model, self.timeout_s = upstream_model, timeout_s

    def _body(self, request: InferenceRequest, stream: bool) -> dict:
        body = {"model": self.upstream_model or request.model, "messages": [dict(m) for m in request.messages], "stream": stream}
        for k in _PASS:
            if k in request.passthrough_params:
                body[k] = request.passthrough_params[k]
        if stream:
            body["stream_options"] = {"include_usage": True}
        return body

    def _open(self, body: dict):
        req = urllib.request.Request(self.base_url + "/chat/completions", data=json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json", "Authorization": f"Bearer {self._key}"})
        try:
            return self.opener(req, timeout=self.timeout_s)
        except urllib.error.HTTPError as e:
            kind, retryable = classify_status(e.code)
            raise InferenceAdapterError(self.id, kind, f"upstream answered HTTP {e.code}", retryable, e.code)
        except (urllib.error.URLError, OSError) as e:
            raise InferenceAdapterError(self.id, "transport_error", str(e), True)

    def complete(self, request: InferenceRequest) -> InferenceResult:
        with self._open(self._body(request, False)) as r:
            raw = r.read().decode()
        try:
            obj = json.loads(raw)
            choice = obj["choices"][0]
            content = choice["message"].get("content") or ""
        except (ValueError, KeyError, IndexError, TypeError, AttributeError):
            raise InferenceAdapterError(self.id, "malformed_response", "upstream answer is not an OpenAI chat completion", True)
        usage = _usage(obj.get("usage"))
        if usage is None:          # receipt-first: an answer that cannot be metered is not delivered
            raise InferenceAdapterError(self.id, "usage_missing", "upstream answer carries no terminal usage", False)
        return InferenceResult(content, choice.get("finish_reason") or "stop", obj.get("model") or request.model, usage)

    def stream(self, request: InferenceRequest):
        """Yields ``("delta", text)`` items, then one ``("done", InferenceResult)`` whose usage comes from the stream's
        terminal frames.  A stream that ends without usage raises after the deltas."""
        usage, finish, served, parts = None, None, None, []
        with self._open(self._body(request, True)) as r:
            for line in r:
                line = line.decode().strip() if isinstance(line, bytes) else line.strip()
                if not line.startswith("data:"):
                    continue
                data = line[5:].strip()
                if data == "[DONE]":
                    break
                try:
                    obj = json.loads(data)
                except ValueError:
                    continue
                served = obj.get("model") or served
                usage = _usage(obj.get("usage")) or usage
                for ch in obj.get("choices") or []:
                    text = (ch.get("delta") or {}).get("content")
                    if text:
                        parts.append(text)
                        yield ("delta", text)
                    finish = ch.get("finish_reason") or finish
        if usage is None:
            raise InferenceAdapterError(self.id, "usage_missing", "stream ended without terminal usage", False)
        yield ("done", InferenceResult("".join(parts), finish or "stop", served or request.model, usage))


class HydraliskPoolAdapter:
    """Several replicas behind one adapter id.  ``replicas``: list of dicts with ``adapter`` (a ``HydraliskAdapter``),
    ``replicaId``, ``maxInflight`` and optional ``benchmarkReserved`` / ``draining`` / ``region``.  ``affinity_oracle``
    maps a session-affinity value to the replica that last served it (default: this pool's own memory of it);
    ``routing_state_oracle(replica_id)`` may override health and the like from outside telemetry."""

    def __init__(self, id: str, replicas: list[dict], affinity_oracle=None, routing_state_oracle=None, saturation_policy: str | None = None,
                 max_queue_wait_ms: float = 250, sleep=None, now_ms=lambda: int(time.time() * 1000)):
        self.id, self.replicas = id, {r["replicaId"]: r for r in replicas}
        self.order = [r["replicaId"] for r in replicas]
        self.affinity_oracle, self.routing_state_oracle = affinity_oracle, routing_state_oracle
        self.saturation_policy, self.max_queue_wait_ms, self.sleep, self.now_ms = saturation_policy, max_queue_wait_ms, sleep, now_ms
        self.lock = threading.Lock()
        self.live = {rid: {"inflight": 0, "warm": "unknown", "warmAt": None, "last429": None, "ttft": None, "tps": None, "health": "healthy",
                           "errors": 0} for rid in self.order}
        self.affinity: dict[str, str] = {}
        self.max_affinity_entries = 100_000        # sessions remembered; the least recently used tenth goes when it is full
        self.last_route: dict | None = None

    def states(self) -> list[dict]:
        out = []
        with self.lock:
            for rid in self.order:
                cfg, lv = self.replicas[rid], self.live[rid]
                s = replica_state(rid, lv["health"], lv["warm"], lv["inflight"], cfg.get("maxInflight", 1), 0, lv["ttft"], lv["tps"], lv["warmAt"],
                                  bool(cfg.get("benchmarkReserved")), bool(cfg.get("draining")), cfg.get("region"))
                over = self.routing_state_oracle(rid) if self.routing_state_oracle else None
                if over:
                    for k in ("health", "warmState", "queueDepth", "observedTtftMs", "observedTps", "inflightCount", "maxInflight",
                              "benchmarkReserved", "draining", "region", "warmAtEpochMs"):
                        if over.get(k) is not None:
                            s[k] = over[k]
                out.append(s)
        return out

    def route_admission(self) -> dict:
        return route_admission(self.states())

    def _run(self, request: InferenceRequest, affinity: str | None):
        def run(rid):
            lv = self.live[rid]
            with self.lock:
                lv["inflight"] += 1
            t0 = self.now_ms()
            try:
                res = self.replicas[rid]["adapter"].complete(request)
            except InferenceAdapterError as e:
                with self.lock:
                    lv["errors"] += 1
                    if e.http_status == 429:
                        lv["last429"] = self.now_ms()
                    elif e.retryable:              # two transport / 5xx failures in a row take the replica out of rotation
                        lv["health"] = "unhealthy" if lv["errors"] >= 2 else "degraded"
                raise InferenceAdapterError(self.id, e.kind, f"{rid}: {e.reason}", e.retryable, e.http_status)
            finally:
                with self.lock:
                    lv["inflight"] -= 1
            dt = max(1, self.now_ms() - t0)
            with self.lock:
                lv.update(errors=0, health="healthy", warm="warm", warmAt=self.now_ms(), ttft=dt,
                          tps=1000.0 * res.usage.completion_tokens / dt)
                if affinity:
                    self.affinity.pop(affinity, None)            # re-insert: the map is kept in order of last use
                    self.affinity[affinity] = rid
                    if len(self.affinity) > self.max_affinity_entries:
                        for k in list(self.affinity)[: self.max_affinity_entries // 10]:
                            del self.affinity[k]
            return res
        return run

    def complete(self, request: InferenceRequest) -> InferenceResult:
        affinity = request.passthrough_params.get(pc.SESSION_AFFINITY_PARAM) or request.passthrough_params.get(pc.OPENAI_USER_PARAM)
        hint = None
        if affinity:
            hint = self.affinity_oracle(affinity) if self.affinity_oracle else self.affinity.get(affinity)
        policy = self.saturation_policy or default_saturation_policy(request.stream)
        res, route = dispatch_to_pool(self.states, self._run(request, affinity), policy, self.max_queue_wait_ms, self.sleep, hint, self.id)
        self.last_route = route
        return res
