"""``b200-serve``: OpenAI-compatible model server.

    python -m openagents_b200.serve.server -m model.gguf --backend cuda --host 127.0.0.1 --port 8080

Flags and routes follow the reference's description of its model server
(apps/pylon/docs/2026-06-09-pylon-qwen35-local-inference-roadmap.md:137-160, 232-236):
``-m`` (repeatable), ``--backend cpu|cuda``, ``--host``, ``--port``, ``--reasoning-budget``,
``--mesh-coordination enabled|disabled``; ``GET /health`` (reports ``execution_engine`` and the
endpoints), ``GET /v1/models``, ``POST /v1/chat/completions`` (streaming and not), ``POST
/v1/responses`` (with ``previous_response_id`` replay), ``GET /psionic/management/status``; plus
``/v1/sessions`` in the shape of the one in-tree local model server with session semantics
(packages/apple-fm-runtime/native/foundation-bridge/Sources/foundation-bridge/main.swift:472-494)
and a Prometheus ``/metrics``.  ``POST /v1/serve`` answers the gateway's serve wire contract
(apps/openagents.com/workers/api/src/inference/psionic-fabric-serve.ts:116-164) including the
exact-greedy parity check: the request is decoded a second time on the same engine and the two
token streams must be identical.
"""
from __future__ import annotations

import argparse
import hashlib
import hmac
import json
import os
import queue
import threading
import time
import urllib.parse
import uuid
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

from .. import ENGINE_NAME, __version__
from ..gateway.observability import ChatTraceEmitter, RateMonitorConfig, ServedTokensLedger, ServingRateMonitor
from ..utils.cli import cli_entry
from ..utils.nvtx import nvtx_range
from ..utils.telemetry import Histogram
from . import request_schema as schema
from . import tools as tooling
from .generation import (CHAT_TEMPLATE_DIGEST, ByteTokenizer, Request, RequestRejected, Scheduler,
                         render_chat, tokenizer_from_metadata)

ENDPOINTS = ["/health", "/v1/models", "/v1/completions", "/v1/chat/completions", "/v1/responses", "/v1/sessions", "/v1/sessions/{id}/responses",
             "/v1/sessions/{id}/responses/stream", "/v1/serve",
             "/psionic/management/status", "/metrics"]


class ServedModel:
    """One model, one engine, ONE scheduling thread.  HTTP handlers never run the engine: they ``submit`` (a short
    critical section) and wait on the request's completion event or token queue, so requests that arrive while
    others are decoding join the same decode batch (continuous batching across connections)."""

    def __init__(self, model_id: str, backend, artifact_digest: str | None, tokenizer=None, max_num_seqs: int = 64,
                 prefill_chunk: int = 2048, chat_template: str | None = None, speculation=None):
        self.id, self.backend, self.artifact_digest = model_id, backend, artifact_digest
        self.tok = tokenizer or ByteTokenizer(backend.cfg.vocab)
        self.chat_template = chat_template          # a GGUF chat template admitted by the digest allowlist, or None
        self.sched = Scheduler(backend, self.tok, max_num_seqs=max_num_seqs, prefill_chunk=prefill_chunk, speculation=speculation)
        self.cv = threading.Condition()              # guards the scheduler and the backend
        self.waiters = 0                             # handler threads that want the lock (see _loop)
        self._wl = threading.Lock()
        self.created = int(time.time())
        self.closed = False
        self.thread = threading.Thread(target=self._loop, name=f"sched-{model_id}", daemon=True)
        self.thread.start()

    # `lock` is what guards direct backend calls made outside the scheduling loop (closing a session's sequence)
    @property
    def lock(self):
        return self.cv

    def _loop(self):
        while True:
            with self.cv:
                while not self.closed and not self.sched.has_work:
                    self.cv.wait()
                if self.closed:
                    return
                try:
                    with nvtx_range("scheduler.step"):
                        self.sched.step()
                except Exception as e:      # noqa: BLE001 - this thread is the only one that runs the engine: it must outlive any step
                    self.sched.fail_all(e)
                # Python locks are not fair: a loop that re-takes the lock at once can starve the handler threads that
                # want to enqueue, and their requests would miss the running batch.  While any handler is waiting, give
                # the lock away (bounded: a few milliseconds per step at most).
                for _ in range(8):
                    if not self.waiters:
                        break
                    self.cv.wait(timeout=0.001)

    def close(self):
        with self.cv:
            self.closed = True
            self.cv.notify_all()
        self.thread.join(timeout=5)

    def submit(self, prompt_ids, params, seq_id=None, keep=False, on_token=None, on_done=None, history=None) -> Request:
        with self._wl:
            self.waiters += 1
        try:
            with self.cv:
                r = self.sched.submit(prompt_ids, params, seq_id=seq_id, keep_sequence=keep, on_token=on_token, on_done=on_done,
                                      history=history)
                self.cv.notify_all()
        finally:
            with self._wl:
                self.waiters -= 1
        return r

    _score_ids = 1 << 50

    def token_logprobs(self, context_ids, output_ids) -> list[float]:
        """Natural-log probability of each generated token given everything before it: one extra forward over
        ``context + output`` in a sequence of its own, between two scheduler steps (the ``logprobs`` option of a completed,
        non-streamed request)."""
        if not getattr(self.backend, "supports_score", False):
            raise RequestRejected(f"the {self.backend.name} backend cannot report log-probabilities")
        if not output_ids:
            return []
        ctx, out = list(context_ids), list(output_ids)
        feed = ctx + out[:-1]
        targets = [-1] * (len(ctx) - 1) + out
        with self._wl:
            self.waiters += 1
            ServedModel._score_ids += 1
            sid = ServedModel._score_ids
        try:
            with self.cv:
                cached = self.backend.begin(sid, feed)
                try:
                    if cached:
                        self.backend.truncate(sid, 0)
                    lp = self.backend.score(sid, feed, targets)
                finally:
                    self.backend.end(sid)
        finally:
            with self._wl:
                self.waiters -= 1
        return lp[len(ctx) - 1:]

    def generate(self, prompt_ids, params, seq_id=None, keep=False, on_token=None, history=None) -> Request:
        """Blocking completion.  ``on_token`` is called on THIS thread (tokens cross from the scheduling thread through
        a queue), so a slow client socket never stalls the decode loop."""
        q: queue.SimpleQueue = queue.SimpleQueue()
        r = self.submit(prompt_ids, params, seq_id=seq_id, keep=keep, on_token=q.put, on_done=lambda _r: q.put(None),
                        history=history)
        while True:
            tok = q.get()
            if tok is None:
                break
            if on_token:
                try:
                    on_token(tok)
                except (BrokenPipeError, ConnectionError, OSError):      # client went away: stop generating for it
                    with self.cv:
                        self.sched.cancel(r)
                    on_token = None
        if r.finish_reason == "error" and r.error is not None:
            raise r.error
        return r


class Session:
    def __init__(self, sid: str, model: ServedModel):
        self.id, self.model = sid, model
        self.seq_id: int | None = None
        self.tokens: list[int] = []       # everything the sequence's KV covers, plus the pending tail
        self.pending: list[int] = []      # generated tokens whose K/V have not been written yet
        self.responses: list[str] = []
        self.instructions: str | None = None   # a system message that opens the session's first turn
        self.created = time.time()
        self.last_used = self.created
        self.busy = 0                          # turns in flight; a busy session is never evicted


class ServerState:
    def __init__(self, models: list[ServedModel], reasoning_budget: int = 0, mesh_coordination: str = "disabled"):
        self.models = {m.id: m for m in models}
        self.default = models[0]
        self.sessions: dict[str, Session] = {}
        self.responses: dict[str, tuple[str, str]] = {}     # response id -> (session id, text)
        # an idle session pins the KV pages of its conversation: sessions are dropped after ``session_ttl_s`` without a turn, the
        # least recently used ones beyond ``max_sessions``, and as many idle ones as it takes when the KV pool runs out
        self.max_sessions = int(os.environ.get("B200_SERVE_MAX_SESSIONS", "1024"))
        self.session_ttl_s = float(os.environ.get("B200_SERVE_SESSION_TTL_S", "1800"))
        self.sessions_evicted = 0
        self._sess_lock = threading.Lock()
        self.reasoning_budget, self.mesh_coordination = reasoning_budget, mesh_coordination
        self.started = time.time()
        self.allow_shutdown = False
        self.api_key: str | None = None      # when set, every POST route wants "Authorization: Bearer <key>"
        self.ttft = Histogram([0.005, 0.01, 0.025, 0.05, 0.1, 0.25, 0.5, 1, 2.5, 5, 10])
        self.itl = Histogram([0.0005, 0.001, 0.002, 0.005, 0.01, 0.02, 0.05, 0.1, 0.25])
        self.lock = threading.Lock()
        # served-token ledger (one idempotent row per completed request), rate monitor over it, opt-in trace emitter
        self.ledger = ServedTokensLedger(os.environ.get("B200_SERVED_TOKENS_LEDGER") or None)
        self.rate_monitor = ServingRateMonitor(self.ledger, RateMonitorConfig.from_env())
        self.traces = ChatTraceEmitter(enabled=os.environ.get("B200_CHAT_TRACE_EMIT", "false").lower() == "true")

    def model(self, name: str | None) -> ServedModel:
        if not name:
            return self.default
        if name not in self.models:
            raise KeyError(name)
        return self.models[name]

    # ---- sessions
    def add_session(self, s: Session) -> Session:
        self.reap_sessions()
        with self._sess_lock:
            self.sessions[s.id] = s
        return s

    def drop_session(self, sid: str) -> Session | None:
        """Forget a session and give its sequence (its KV pages) back; its response ids stop resolving."""
        with self._sess_lock:
            s = self.sessions.pop(sid, None)
            if s is None:
                return None
            for rid in s.responses:
                self.responses.pop(rid, None)
        if s.seq_id is not None:
            with s.model.lock:
                try:
                    s.model.backend.end(s.seq_id)
                except Exception:      # noqa: BLE001 - the sequence may already be gone (a failed turn closed it)
                    pass
            s.seq_id = None
        return s

    def reap_sessions(self, need_room: bool = False, now: float | None = None) -> int:
        """Drop expired sessions and the least recently used ones beyond the cap; with ``need_room`` (the KV pool ran out) also the
        least recently used idle half of what is left.  Returns how many were dropped."""
        now = time.time() if now is None else now
        with self._sess_lock:
            idle = sorted((s for s in self.sessions.values() if not s.busy), key=lambda s: s.last_used)
            victims = [s for s in idle if now - s.last_used > self.session_ttl_s]
            rest = [s for s in idle if s not in victims]
            over = len(self.sessions) - len(victims) - self.max_sessions + 1
            if over > 0:
                victims += rest[:over]
                rest = rest[over:]
            if need_room and rest:
                victims += rest[:max(1, len(rest) // 2)]
        n = sum(1 for s in victims if self.drop_session(s.id) is not None)
        self.sessions_evicted += n
        return n

    # ---- one completion, with or without a session
    def complete(self, model: ServedModel, messages: list[dict], body: dict, session: Session | None = None,
                 on_token=None) -> tuple[Request, dict]:
        """Runs the completion.  When the KV pool is exhausted, idle sessions are evicted; the request itself is tried once more
        if nothing of it has been seen yet (no token streamed, no earlier turns whose KV the failure just gave up)."""
        if session is not None:
            with self._sess_lock:
                session.busy += 1
                session.last_used = time.time()
        fresh = session is None or session.seq_id is None
        emitted = [0]

        def counted(t):
            emitted[0] += 1
            if on_token:
                on_token(t)
        try:
            try:
                return self._complete(model, messages, body, session, counted)
            except MemoryError:
                if self.reap_sessions(need_room=True) == 0 or not fresh or emitted[0]:
                    raise
                return self._complete(model, messages, body, session, counted)
        finally:
            if session is not None:
                with self._sess_lock:
                    session.busy -= 1
                    session.last_used = time.time()

    def _complete(self, model: ServedModel, messages: list[dict], body: dict, session: Session | None = None,
                  on_token=None) -> tuple[Request, dict]:
        params = schema.sampling_params(body)
        tok = model.tok
        toks = getattr(tok, "tokens", None)

        def special(i):
            return toks[i] if toks is not None and isinstance(i, int) and 0 <= i < len(toks) else ""
        ids = tok.encode(render_chat(messages, model.chat_template, bos_token=special(getattr(tok, "bos_id", None)),
                                     eos_token=special(getattr(tok, "eos_id", None)), tools=schema.tools(body) or None,
                                     **schema.template_kwargs(body)))
        with nvtx_range("serve.complete"):
            if session is None:
                r = model.generate(ids, params, on_token=on_token)
            else:
                feed = session.pending + ids
                try:
                    if session.seq_id is None:
                        r = model.generate(feed, params, keep=True, on_token=on_token)
                        session.seq_id = r.seq_id
                    else:
                        r = model.generate(feed, params, seq_id=session.seq_id, keep=True, on_token=on_token,
                                           history=session.tokens)
                except RequestRejected:
                    raise
                except Exception:
                    # a turn that opened the sequence had it closed by the scheduler; a continued sequence is still open and is
                    # closed here, so that the forgotten conversation does not keep its KV pages
                    if session.seq_id is not None:
                        with model.lock:
                            try:
                                model.backend.end(session.seq_id)
                            except Exception:      # noqa: BLE001
                                pass
                    session.seq_id, session.tokens, session.pending = None, [], []
                    raise
                session.tokens += feed + r.output[:-1] if r.output else feed
                session.pending = r.output[-1:] if r.output else []
        usage = {"prompt_tokens": len(ids), "completion_tokens": len(r.output), "total_tokens": len(ids) + len(r.output),
                 "prompt_tokens_details": {"cached_tokens": r.cached_prompt_tokens}}
        if model.sched.speculation is not None:      # disclosed per request, in the gateway's speculation-metadata shape
            from ..gateway.metadata import speculation_metadata
            usage["speculation"] = speculation_metadata(model.sched.speculation.mode, active=r.spec_proposed > 0,
                                                        proposed=r.spec_proposed, accepted=r.spec_accepted)
        self.ledger.record(r.request_id + "." + uuid.uuid4().hex[:8], model.id, len(ids), len(r.output),
                           account_ref=str(body.get("user") or "account.anonymous"), adapter_id=ENGINE_NAME,
                           demand_kind=str(body.get("demand_kind") or "unlabeled"))
        self.rate_monitor.lane_heartbeat(True)
        trace = self.traces.emit(messages, model.tok.decode(r.output), opted_in=bool(body.get("emit_trace")))
        if trace.get("emitted"):
            usage["trace"] = trace["path"]
        with self.lock:
            if r.ttft_s is not None:
                self.ttft.observe(r.ttft_s)
            if r.t_done and r.t_first_token and len(r.output) > 1:
                self.itl.observe((r.t_done - r.t_first_token) / (len(r.output) - 1))
        return r, usage

    def serve_contract(self, model: ServedModel, body: dict) -> dict:
        """The gateway's serve request: greedy decode twice on this engine; parity = same tokens."""
        msgs = schema.messages(body.get("messages"))
        if not isinstance(body.get("passthroughParams"), (dict, type(None))):
            raise schema.BadRequest("passthroughParams must be an object")
        pp = dict(body.get("passthroughParams") or {})
        schema.common(pp)
        pp["temperature"] = 0.0
        r1, usage = self.complete(model, msgs, pp)
        parity = False
        if body.get("requireExactGreedyParity", True):
            r2, _ = self.complete(model, msgs, pp)
            parity = r1.output == r2.output
        topo = model.backend.topology()
        run_ref = "serve." + hashlib.sha256(json.dumps([model.id, msgs, r1.output]).encode()).hexdigest()[:24]
        return {"content": model.tok.decode(r1.output), "finishReason": r1.finish_reason or "stop",
                "usage": {"promptTokens": usage["prompt_tokens"], "completionTokens": usage["completion_tokens"],
                          "totalTokens": usage["total_tokens"], "cachedPromptTokens": r1.cached_prompt_tokens},
                "servedModel": model.id, "servingRunRef": run_ref, "stages": topo["stages"],
                "parityMode": "exact_greedy_parity" if body.get("requireExactGreedyParity", True) else "none",
                "parityVerified": parity,
                "tokenHash": "sha256:" + hashlib.sha256(json.dumps(r1.output).encode()).hexdigest()}

    def status(self) -> dict:
        return {"execution_engine": ENGINE_NAME, "version": __version__, "uptime_s": round(time.time() - self.started, 1),
                "mesh_coordination": self.mesh_coordination, "reasoning_budget": self.reasoning_budget,
                "models": [{"id": m.id, "backend": m.backend.name, "architecture": m.backend.cfg.arch,
                            "artifact_digest": m.artifact_digest, "kv": m.backend.kv_stats(),
                            "topology": m.backend.topology(), "scheduler": dict(m.sched.stats),
                            "levers": {"max_num_seqs": m.sched.max_num_seqs, "prefix_caching": True, "chunked_prefill": True,
                                       "prefill_chunk": m.sched.prefill_chunk,
                                       "speculation": m.sched.speculation.mode if m.sched.speculation else "none",
                                       "speculation_acceptance_rate": m.sched.speculation_acceptance_rate}} for m in self.models.values()],
                "sessions": len(self.sessions), "sessions_evicted": self.sessions_evicted, "tokens_served": self.ledger.public_projection(),
                "serving_rate": self.rate_monitor.tick()["classification"]}

    def metrics_text(self) -> str:
        out = []
        for m in self.models.values():
            s, lab = m.sched.stats, f'{{model="{m.id}"}}'
            out += [f"b200_requests_total{lab} {s['requests']}", f"b200_prompt_tokens_total{lab} {s['prompt_tokens']}",
                    f"b200_completion_tokens_total{lab} {s['completion_tokens']}",
                    f"b200_prefix_cache_hit_tokens_total{lab} {s['cached_prompt_tokens']}",
                    f"b200_decode_steps_total{lab} {s['steps']}",
                    f"b200_decode_batch_size_avg{lab} {s['batch_size_sum'] / s['steps'] if s['steps'] else 0}",
                    f"b200_request_errors_total{lab} {s['errors']}", f"b200_requests_rejected_total{lab} {s['rejected']}",
                    f"b200_sampled_ids_d2h_bytes_total{lab} {s['d2h_bytes']}"]
            for k, v in m.backend.kv_stats().items():
                out.append(f"b200_kv_{k}{lab} {v}")
        out.append(f"b200_tokens_served_total {self.ledger.total()}")
        out += [f"b200_sessions {len(self.sessions)}", f"b200_sessions_evicted_total {self.sessions_evicted}"]
        out += self.ttft.prometheus("b200_ttft_seconds") + self.itl.prometheus("b200_inter_token_latency_seconds")
        return "\n".join(out) + "\n"


def make_handler(state: ServerState):
    class H(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"

        def log_message(self, *a):
            pass

        def _json(self, code: int, obj):
            data = json.dumps(obj).encode()
            self.send_response(code)
            self.send_header("Content-Type", "application/json")
            self.send_header("Content-Length", str(len(data)))
            self.end_headers()
            self.wfile.write(data)

        def _err(self, code: int, msg: str, kind: str = "invalid_request_error"):
            self._json(code, {"error": {"message": msg, "type": kind}})

        def _body(self):
            try:
                n = int(self.headers.get("Content-Length") or 0)
            except ValueError:
                return None
            if n < 0:
                return None
            raw = self.rfile.read(n) if n else b"{}"
            try:
                obj = json.loads(raw)
            except ValueError:            # malformed JSON, or bytes that are not UTF-8
                return None
            return obj if isinstance(obj, dict) else None

        def do_GET(self):
            path = self.path.split("?")[0]
            if path == "/health":
                return self._json(200, {"status": "ok", "execution_engine": ENGINE_NAME, "endpoints": ENDPOINTS,
                                        "models": list(state.models)})
            if path == "/v1/models":
                return self._json(200, {"object": "list", "data": [
                    {"id": m.id, "object": "model", "created": m.created, "owned_by": ENGINE_NAME,
                     "artifact_digest": m.artifact_digest, "architecture": m.backend.cfg.arch,
                     "chat_template_digest": CHAT_TEMPLATE_DIGEST, "context_length": m.backend.cfg.context}
                    for m in state.models.values()]})
            if path == "/psionic/management/status":
                return self._json(200, state.status())
            if path == "/metrics":
                data = state.metrics_text().encode()
                self.send_response(200)
                self.send_header("Content-Type", "text/plain; version=0.0.4")
                self.send_header("Content-Length", str(len(data)))
                self.end_headers()
                return self.wfile.write(data)
            if path == "/v1/sessions":
                return self._json(200, {"sessions": [{"id": s.id, "model": s.model.id, "tokens": len(s.tokens),
                                                      "responses": s.responses} for s in state.sessions.values()]})
            self._err(404, f"no route {path}", "not_found")

        def do_DELETE(self):
            parts = self.path.strip("/").split("/")
            if len(parts) == 3 and parts[:2] == ["v1", "sessions"]:
                s = state.drop_session(urllib.parse.unquote(parts[2]))
                if s is not None:
                    return self._json(200, {"deleted": s.id})
            self._err(404, "no such session", "not_found")

        def do_POST(self):
            path = self.path.split("?")[0]
            body = self._body()
            if body is None:
                return self._err(400, "request body must be a JSON object")
            self._streaming = False
            if state.api_key and not hmac.compare_digest((self.headers.get("Authorization") or "").encode(), f"Bearer {state.api_key}".encode()):
                return self._err(401, "send Authorization: Bearer <the server's API key>", "invalid_api_key")
            try:
                return self._post(path, body)
            except Exception as e:      # noqa: BLE001 - a handler that raises would close the connection without an answer
                if not self._streaming:
                    return self._err(500, f"{type(e).__name__}: {e}", "engine_error")
                self.close_connection = True      # the event stream has begun: all that is left is to end it
                return None

        def _post(self, path, body):
            if path == "/admin/shutdown":          # only with --allow-shutdown: lets a launcher or a test stop all ranks cleanly
                if not state.allow_shutdown:
                    return self._err(404, "not found", "not_found")
                self._json(200, {"stopping": True})
                threading.Thread(target=self.server.shutdown, daemon=True).start()
                return None
            try:
                schema.common(body)
                model = state.model(body.get("model"))
            except schema.BadRequest as e:
                return self._err(400, str(e))
            except KeyError:
                return self._err(404, f"model {body.get('model')!r} is not served", "model_not_found")
            try:
                if path == "/v1/chat/completions":
                    return self._chat(model, body)
                if path == "/v1/completions":
                    return self._completions(model, body)
                if path == "/v1/responses":
                    return self._responses(model, body)
                if path == "/v1/serve":
                    return self._json(200, state.serve_contract(model, body))
                if path == "/v1/sessions":
                    s = Session("sess-" + uuid.uuid4().hex[:16], model)
                    s.instructions = schema.string(body, "instructions")
                    state.add_session(s)
                    return self._json(200, {"id": s.id, "model": model.id, "session": {"id": s.id}})
                parts = path.strip("/").split("/")
                if len(parts) in (4, 5) and parts[:2] == ["v1", "sessions"] and parts[3] == "responses" and parts[4:] in ([], ["stream"]):
                    s = state.sessions.get(urllib.parse.unquote(parts[2]))
                    if s is None:
                        return self._err(404, "no such session", "not_found")
                    if body.get("messages"):
                        msgs = body["messages"]
                    elif body.get("prompt") is not None:           # the shape of a session turn on the local attach path
                        msgs = [{"role": "user", "content": schema.string(body, "prompt")}]
                    else:
                        msgs = self._input_messages(body)
                    if s.instructions and not s.tokens and not s.pending:      # the session's instructions open its first turn
                        msgs = [{"role": "system", "content": s.instructions}] + list(msgs)
                    if parts[4:] == ["stream"]:
                        return self._session_stream(s, msgs, body)
                    r, usage = state.complete(s.model, msgs, body, session=s)
                    rid = "resp-" + uuid.uuid4().hex[:16]
                    s.responses.append(rid)
                    return self._json(200, {"id": rid, "session": s.id, "output_text": s.model.tok.decode(r.output),
                                            "usage": usage})
            except schema.BadRequest as e:
                return self._err(400, str(e))
            except RequestRejected as e:
                return self._err(400, str(e), "context_length_exceeded")
            except MemoryError as e:
                return self._err(503, str(e), "kv_cache_exhausted")
            except Exception as e:      # surface engine errors as a typed, non-retryable failure
                if self._streaming:
                    raise
                return self._err(500, f"{type(e).__name__}: {e}", "engine_error")
            self._err(404, f"no route {path}", "not_found")

        @staticmethod
        def _input_messages(body):
            """``input`` of the responses routes: a string (one user turn) or a list of messages."""
            inp = body.get("input")
            if isinstance(inp, list):
                return schema.messages(inp, "input")
            if inp is None or isinstance(inp, str):
                return [{"role": "user", "content": inp or ""}]
            raise schema.BadRequest("input must be a string or a list of messages")

        def _session_stream(self, sess, msgs, body):
            """One session turn as server-sent events: a ``snapshot`` event per step whose ``content`` is the answer so far (it
            grows toward the final text; the last one carries ``finish_reason``), then one ``completed`` event with the output, the
            model and the usage.  Sent as it is generated (chunked transfer)."""
            self._streaming = True
            self.send_response(200)
            self.send_header("Content-Type", "text/event-stream; charset=utf-8")
            self.send_header("Cache-Control", "no-cache")
            self.send_header("Transfer-Encoding", "chunked")
            self.end_headers()

            def frame(event, obj):
                data = f"event: {event}\ndata: {json.dumps(obj)}\n\n".encode()
                self.wfile.write(f"{len(data):x}\r\n".encode() + data + b"\r\n")
                self.wfile.flush()

            out: list[int] = []
            sent = [0, ""]                          # snapshots sent, text of the last one

            def on_token(t):
                out.append(t)
                text = sess.model.tok.decode(out)
                if text and not text.endswith("\ufffd") and text != sent[1]:      # hold back incomplete UTF-8 sequences
                    frame("snapshot", {"sequence": sent[0], "content": text, "output": text, "finish_reason": None})
                    sent[0], sent[1] = sent[0] + 1, text

            try:
                r, usage = state.complete(sess.model, msgs, body, session=sess, on_token=on_token)
            except Exception as e:      # noqa: BLE001 - the stream has begun: the failure is its last event
                frame("error", {"error": "generation_failed", "message": f"{type(e).__name__}: {e}"})
                self.wfile.write(b"0\r\n\r\n")
                return
            text = sess.model.tok.decode(r.output)
            frame("snapshot", {"sequence": sent[0], "content": text, "output": text, "finish_reason": r.finish_reason or "stop"})
            rid = "resp-" + uuid.uuid4().hex[:16]
            sess.responses.append(rid)
            frame("completed", {"id": rid, "session": sess.id, "output": text, "content": text, "model": sess.model.id, "usage": usage})
            self.wfile.write(b"0\r\n\r\n")

        def _completions(self, model, body):
            """Text completion on a raw prompt (no chat template): ``prompt`` is a string or a list of token ids; ``echo`` returns
            the prompt in front of the completion; ``logprobs`` (any value but null / false) adds the tokens, their log-probabilities
            (the first prompt token has none) and text offsets; ``max_tokens: 0`` with ``echo`` scores a text without generating,
            which is how evaluation harnesses compute log-likelihoods.  Not streamed."""
            prompt = body.get("prompt")
            if isinstance(prompt, list) and len(prompt) == 1 and isinstance(prompt[0], (str, list)):
                prompt = prompt[0]
            if isinstance(prompt, str):
                ids = model.tok.encode(prompt)
            elif isinstance(prompt, list) and prompt and all(isinstance(t, int) and 0 <= t < model.backend.cfg.vocab for t in prompt):
                ids = list(prompt)
            else:
                return self._err(400, "prompt must be a non-empty string or a list of token ids (one prompt per request)")
            if not ids:
                return self._err(400, "the prompt is empty")
            if body.get("stream"):
                return self._err(400, "text completions are not streamed; use /v1/chat/completions")
            echo, want_lp = schema.boolean(body, "echo"), body.get("logprobs") not in (None, False)
            n_new = schema.integer(body, "max_tokens", 0)
            n_new = 16 if n_new is None else n_new
            if n_new == 0 and not echo:
                return self._err(400, "max_tokens must be positive (0 is allowed together with echo)")
            out, finish = [], "length"
            if n_new > 0:
                params = schema.sampling_params(body, max_tokens=n_new)
                r = model.generate(ids, params)
                out, finish = list(r.output), r.finish_reason or "stop"
            shown = (ids if echo else []) + out
            choice = {"index": 0, "text": model.tok.decode(shown), "finish_reason": finish, "logprobs": None}
            if want_lp:
                scored = ids + out
                lps = model.token_logprobs(scored[:1], scored[1:]) if len(scored) > 1 else []
                lps = [None] + lps                                     # nothing precedes the first token
                lps = lps if echo else lps[len(ids):]
                pieces = [model.tok.decode([t]) for t in shown]
                offsets, at = [], 0
                for piece in pieces:
                    offsets.append(at)
                    at += len(piece)
                choice["logprobs"] = {"tokens": pieces, "token_ids": shown, "token_logprobs": lps, "text_offset": offsets, "top_logprobs": None}
            usage = {"prompt_tokens": len(ids), "completion_tokens": len(out), "total_tokens": len(ids) + len(out)}
            state.ledger.record("cmpl." + uuid.uuid4().hex[:12], model.id, len(ids), len(out), account_ref=str(body.get("user") or "account.anonymous"),
                                adapter_id=ENGINE_NAME, demand_kind=str(body.get("demand_kind") or "unlabeled"))
            self._json(200, {"id": "cmpl-" + uuid.uuid4().hex[:24], "object": "text_completion", "created": int(time.time()), "model": model.id,
                             "choices": [choice], "usage": usage})

        def _chat(self, model, body):
            msgs = schema.messages(body.get("messages"))
            tools = schema.tools(body)
            try:
                mode, fname = tooling.normalize_tool_choice(body.get("tool_choice"), tools)
            except tooling.ToolCallError as e:
                return self._err(400, str(e), e.kind)
            tool_msg = tooling.render_tools_system_message(tools, mode, fname)
            if tool_msg is not None:         # stable position: ahead of the conversation, after other system text
                head = [m for m in msgs if m.get("role") == "system"]
                msgs = head + [{"role": "system", "content": tool_msg["content"]}] + [m for m in msgs if m.get("role") != "system"]
            msgs = [{"role": m["role"], "content": m.get("content") if isinstance(m.get("content"), str) else
                     json.dumps(m.get("tool_calls") or m.get("content") or "")} for m in msgs]
            cid = "chatcmpl-" + uuid.uuid4().hex[:24]
            created = int(time.time())
            want_lp = bool(body.get("logprobs"))
            if want_lp and (body.get("stream") or int(body.get("top_logprobs") or 0) > 0):
                return self._err(400, "logprobs are reported for non-streamed completions, for the chosen tokens only (top_logprobs must be 0)")
            if body.get("stream"):
                self._streaming = True
                self.send_response(200)
                self.send_header("Content-Type", "text/event-stream")
                self.send_header("Cache-Control", "no-cache")
                self.send_header("Transfer-Encoding", "chunked")
                self.end_headers()

                def chunk(obj):
                    data = ("data: " + (obj if isinstance(obj, str) else json.dumps(obj)) + "\n\n").encode()
                    self.wfile.write(f"{len(data):x}\r\n".encode() + data + b"\r\n")
                    self.wfile.flush()

                base = {"id": cid, "object": "chat.completion.chunk", "created": created, "model": model.id}
                chunk({**base, "choices": [{"index": 0, "delta": {"role": "assistant"}, "finish_reason": None}]})
                pending: list[int] = []
                splitter = tooling.ToolCallStreamSplitter(tools) if mode != "none" else None

                def emit(text):
                    for d in (splitter.feed(text) if splitter else [{"content": text}]):
                        chunk({**base, "choices": [{"index": 0, "delta": d, "finish_reason": None}]})

                def on_token(t):
                    pending.append(t)
                    text = model.tok.decode(pending)
                    if text and not text.endswith("\ufffd"):       # hold back incomplete UTF-8 sequences
                        emit(text)
                        pending.clear()

                r, usage = state.complete(model, msgs, body, on_token=on_token)
                finish = r.finish_reason
                if pending:                  # bytes held back as an incomplete UTF-8 sequence: the answer ends here, send them
                    tail = model.tok.decode(pending)
                    pending.clear()
                    if tail:
                        emit(tail)
                if splitter:
                    for d in splitter.flush():
                        chunk({**base, "choices": [{"index": 0, "delta": d, "finish_reason": None}]})
                    if splitter.n_calls:
                        finish = "tool_calls"
                chunk({**base, "choices": [{"index": 0, "delta": {}, "finish_reason": finish}], "usage": usage})
                chunk("[DONE]")
                self.wfile.write(b"0\r\n\r\n")
                return
            r, usage = state.complete(model, msgs, body)
            text = model.tok.decode(r.output)
            try:
                msg, finish = tooling.finish_with_tools(text, tools, mode, fname)
            except tooling.ToolCallError as e:
                return self._err(422, str(e), e.kind)
            if finish == "stop":
                finish = r.finish_reason
            choice = {"index": 0, "message": msg, "finish_reason": finish}
            if want_lp:
                try:
                    lps = model.token_logprobs(list(r.history) + list(r.prompt), r.output)
                except RequestRejected as e:
                    return self._err(400, str(e))
                dec = getattr(model.tok, "decode_bytes", None)
                choice["logprobs"] = {"content": [{"token": model.tok.decode([t]), "logprob": lp,
                                                   "bytes": list(dec([t])) if dec else list(model.tok.decode([t]).encode()), "top_logprobs": []}
                                                  for t, lp in zip(r.output, lps)]}
            self._json(200, {"id": cid, "object": "chat.completion", "created": created, "model": model.id,
                             "choices": [choice], "usage": usage,
                             "timings": {"ttft_ms": None if r.ttft_s is None else round(r.ttft_s * 1e3, 3),
                                         "predicted_per_second": (len(r.output) - 1) / (r.t_done - r.t_first_token)
                                         if r.t_done and r.t_first_token and len(r.output) > 1 and r.t_done > r.t_first_token else None}})

        def _responses(self, model, body):
            msgs = self._input_messages(body) if body.get("input") is not None or body.get("messages") is None else body["messages"]
            prev = body.get("previous_response_id")
            if prev is not None:
                sess = state.sessions.get(state.responses[prev][0]) if prev in state.responses else None
                if sess is None:
                    return self._err(404, f"previous_response_id {prev!r} is unknown or its conversation has expired", "not_found")
            else:
                sess = state.add_session(Session("sess-" + uuid.uuid4().hex[:16], model))
            r, usage = state.complete(sess.model, msgs, body, session=sess)
            rid = "resp-" + uuid.uuid4().hex[:16]
            text = sess.model.tok.decode(r.output)
            state.responses[rid] = (sess.id, text)
            sess.responses.append(rid)
            self._json(200, {"id": rid, "object": "response", "model": sess.model.id, "previous_response_id": prev,
                             "status": "completed", "output_text": text,
                             "output": [{"type": "message", "role": "assistant", "content": [{"type": "output_text", "text": text}]}],
                             "usage": {"input_tokens": usage["prompt_tokens"], "output_tokens": usage["completion_tokens"],
                                       "total_tokens": usage["total_tokens"],
                                       "input_tokens_details": {"cached_tokens": r.cached_prompt_tokens}}})

    return H


def load_tokenizer(path: str, vocab_size: int):
    """Tokenizer and chat template of a GGUF file.  The template is used only when its digest is on the allowlist of
    ``control.node_bridge`` (a template is code that runs on every request); otherwise the built-in template applies."""
    from ..control.node_bridge import template_admitted
    from ..gguf import GGUFFile
    meta = {k: v for k, v in GGUFFile(path).metadata.items() if k.startswith("tokenizer.")}
    tok = tokenizer_from_metadata(meta, vocab_size)
    tpl = meta.get("tokenizer.chat_template")
    return tok, (tpl if isinstance(tpl, str) and template_admitted(tpl) else None)


def build_state(model_paths: list[str], backend: str = "cuda", max_num_seqs: int = 64, kv_page_size: int = 16,
                max_ctx: int = 4096, reasoning_budget: int = 0, mesh_coordination: str = "disabled",
                device="cuda:0", tp_rank: int = 0, tp_world: int = 1, ep_rank: int = 0, ep_world: int = 1, comm=None,
                control_group=None, speculation=None) -> ServerState:
    """``tp_world`` / ``ep_world`` > 1: this process is rank 0 of a tensor- or expert-parallel group whose other ranks
    run ``serve.distributed.follower_loop``; every engine call is first announced to them over ``control_group``."""
    from ..receipts.manifests import artifact_digest
    from .backend import open_backend
    if backend not in ("cpu", "cuda"):
        raise ValueError("--backend accepts cpu or cuda")
    if kv_page_size != 16:
        raise ValueError("the paged KV cache uses 16-token pages")
    models = []
    for p in model_paths:
        b = open_backend(p, backend, device, max_num_seqs=max_num_seqs, max_ctx=max_ctx, tp_rank=tp_rank,
                         tp_world=tp_world, comm=comm, ep_rank=ep_rank, ep_world=ep_world)
        if max(tp_world, ep_world) > 1:
            from .distributed import LeaderBackend
            b = LeaderBackend(b, control_group)
        mid = p.rsplit("/", 1)[-1].removesuffix(".gguf")
        tok, tpl = load_tokenizer(p, b.cfg.vocab)
        models.append(ServedModel(mid, b, artifact_digest(p), tokenizer=tok, max_num_seqs=max_num_seqs, chat_template=tpl,
                                  speculation=speculation))
    return ServerState(models, reasoning_budget, mesh_coordination)


class _Server(ThreadingHTTPServer):
    # the default listen backlog of 5 resets connections when a few dozen clients connect in the same instant
    request_queue_size = 1024

    def handle_error(self, request, client_address):
        """A client that goes away mid-request is routine, not a traceback on stderr; anything else is still reported."""
        import sys
        if isinstance(sys.exc_info()[1], (ConnectionError, TimeoutError)):
            return
        super().handle_error(request, client_address)


def serve(state: ServerState, host: str = "127.0.0.1", port: int = 8080) -> ThreadingHTTPServer:
    httpd = _Server((host, port), make_handler(state))
    httpd.daemon_threads = True
    return httpd


def _flag_env(name: str, default):
    """Flags are decoded once: the command line wins, then ``B200_SERVE_<FLAG>`` from the environment, then the default."""
    v = os.environ.get("B200_SERVE_" + name.upper().replace("-", "_"))
    return type(default)(v) if v is not None and default is not None else (v if v is not None else default)


def parse_args(argv=None):
    ap = argparse.ArgumentParser(prog="b200-serve")
    ap.add_argument("-m", "--model", action="append", required=True)
    ap.add_argument("--backend", default=_flag_env("backend", "cuda"), choices=["cpu", "cuda"])
    ap.add_argument("--host", default=_flag_env("host", "127.0.0.1"))
    ap.add_argument("--port", type=int, default=_flag_env("port", 8080))
    ap.add_argument("--reasoning-budget", type=int, default=_flag_env("reasoning-budget", 0))
    ap.add_argument("--mesh-coordination", default=_flag_env("mesh-coordination", "disabled"), choices=["enabled", "disabled"])
    ap.add_argument("--tp", type=int, default=_flag_env("tp", 1), help="tensor-parallel ranks (one GPU each)")
    ap.add_argument("--ep", type=int, default=_flag_env("ep", 1), help="expert-parallel ranks (models with experts)")
    ap.add_argument("--kv-page-size", type=int, default=_flag_env("kv-page-size", 16))
    ap.add_argument("--max-num-seqs", type=int, default=_flag_env("max-num-seqs", 64))
    ap.add_argument("--max-ctx", type=int, default=_flag_env("max-ctx", 4096))
    ap.add_argument("--speculation", default=_flag_env("speculation", "none"), choices=["none", "n_gram"],
                    help="low-batch speculative decoding: n-gram drafts verified in one forward (greedy requests only)")
    ap.add_argument("--speculation-max-batch", type=int, default=_flag_env("speculation-max-batch", 4))
    ap.add_argument("--api-key", default=os.environ.get("B200_API_KEY"),
                    help="require 'Authorization: Bearer <key>' on every POST route (default: $B200_API_KEY; unset = open, for loopback use)")
    ap.add_argument("--allow-shutdown", action="store_true", help="accept POST /admin/shutdown (stops every rank between steps)")
    a = ap.parse_args(argv)
    if a.tp > 1 and a.ep > 1:
        ap.error("--tp and --ep cannot be combined")
    if max(a.tp, a.ep) > 1 and a.backend != "cuda":
        ap.error("--tp / --ep need --backend cuda")
    return a


def run_server(a, **parallel):
    spec = None
    if getattr(a, "speculation", "none") == "n_gram":
        from .generation import SpeculationConfig
        spec = SpeculationConfig(max_batch=a.speculation_max_batch)
    state = build_state(a.model, a.backend, a.max_num_seqs, a.kv_page_size, a.max_ctx, a.reasoning_budget, a.mesh_coordination,
                        speculation=spec, **parallel)
    state.allow_shutdown = bool(getattr(a, "allow_shutdown", False))
    state.api_key = getattr(a, "api_key", None) or None
    httpd = serve(state, a.host, a.port)
    print(json.dumps({"event": "listening", "host": a.host, "port": httpd.server_address[1], "models": list(state.models),
                      "execution_engine": ENGINE_NAME, "tp": a.tp, "ep": a.ep}), flush=True)
    try:
        httpd.serve_forever()
    except KeyboardInterrupt:
        pass
    finally:
        for m in state.models.values():
            m.close()


@cli_entry("b200-serve")
def main(argv=None):
    a = parse_args(argv)
    if max(a.tp, a.ep) > 1:
        from .distributed import launch_ranks
        return launch_ranks(a)
    run_server(a)


if __name__ == "__main__":
    main()
