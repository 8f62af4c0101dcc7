"""The gateway's chat-completions route: the request path from an API key to a metered, receipted answer.

Order of work for ``POST /v1/chat/completions`` (the reference's ``handleChatCompletions``,
inference/chat-completions-routes.ts:2550, wired at index.ts:16272):

1. authenticate the bearer key; 2. fair share: a key may hold only so many requests in flight;
3. decode and validate the body; 4. model gating (the key's allowed models); 5. stable-first prompt
layout and the cache-affinity hash; 6. lane plan from the router; 7. dispatch with overflow across the
registered adapters; 8. re-frame the answer (JSON, or server-sent events for ``stream``); 9. meter the
usage against the pricing table and the key's balance; 10. build the telemetry record and return the
compact telemetry block on the response.

Caller-funded requests (``x-openagents-provider`` / ``x-openagents-provider-key`` headers, or a provider key attached
to the account) go to an adapter built for that key, are never debited and are acknowledged in the
``x-openagents-byok`` response header (chat-completions-routes.ts:221-223, 254-312, 2786-2812); the billing
disclosure on the receipt says which of receipt-backed / zero-charge / no-debit applied (:1533-1553).  Model gating
comes from a table (``ModelGate``): premium models need an entitled key, internal models an allow-listed account, and a
model nobody can serve is refused before any spend check (:2586-2600, 3019-3025).  With ``platform_funded=False`` only
caller-funded or no-meter traffic is dispatched (:3043-3065).  Every answered request lands in the served-token ledger.

Adapters here: ``LocalEngineAdapter`` answers from an in-process ``ServerState`` (this engine, whole-model
lane) and produces the serving receipt with exact-greedy parity itself; the ``openagents-network`` adapter
from ``fabric`` does the same over HTTP to a node.
"""
from __future__ import annotations

import json
import threading
import time
import uuid

from ..serve import request_schema as schema
from . import prompt_cache as pc
from . import request_telemetry as rt
from .fabric import InferenceAdapterError, InferenceRequest, InferenceResult, InferenceUsage, ProviderRegistry, normalize_serve_response
from .metadata import engine_quantization
from .router import PricingTable, dispatch_with_overflow, select_adapter_plan


class GatewayError(Exception):
    def __init__(self, status: int, code: str, message: str):
        super().__init__(message)
        self.status, self.code, self.message = status, code, message

    def body(self) -> dict:
        return {"error": {"message": self.message, "type": self.code, "code": self.code}}


class ApiKey:
    def __init__(self, key: str, account: str, balance_msat: int = 0, allowed_models: tuple | None = None, max_inflight: int = 4,
                 byok: dict | None = None, premium: bool = False, no_meter: bool = False):
        self.key, self.account, self.balance_msat, self.allowed_models = key, account, balance_msat, allowed_models
        self.max_inflight, self.inflight, self.byok = max_inflight, 0, byok or {}
        self.premium, self.no_meter = premium, no_meter      # entitled to premium models; operator-owned capacity, never debited


BYOK_PROVIDER_HEADER = "x-openagents-provider"
BYOK_PROVIDER_KEY_HEADER = "x-openagents-provider-key"
BYOK_ACK_HEADER = "x-openagents-byok"
BYOK_PROVIDERS = ("openrouter",)


class ByokState:
    """``absent`` | ``accepted`` (provider, api_key, source = request | account) | ``invalid`` (reason)."""

    def __init__(self, tag: str, provider: str | None = None, api_key: str | None = None, source: str | None = None, reason: str | None = None):
        self.tag, self.provider, self.api_key, self.source, self.reason = tag, provider, api_key, source, reason

    def __repr__(self):        # the key never reaches a log line
        return f"ByokState({self.tag}, provider={self.provider}, source={self.source})"


def _key_shape_ok(raw) -> bool:
    return isinstance(raw, str) and 8 <= len(raw.strip()) <= 512 and raw.strip() == raw and not any(c.isspace() or c == "," for c in raw)


def resolve_byok(headers: dict | None) -> ByokState:
    """Per-request caller funding from the two headers (names compared case-insensitively)."""
    h = {str(k).lower(): v for k, v in (headers or {}).items()}
    provider = (h.get(BYOK_PROVIDER_HEADER) or "").strip().lower()
    raw = h.get(BYOK_PROVIDER_KEY_HEADER)
    if not provider and raw is None:
        return ByokState("absent")
    if provider not in BYOK_PROVIDERS:
        return ByokState("invalid", reason=f"Only {BYOK_PROVIDER_HEADER}: {' | '.join(BYOK_PROVIDERS)} is supported for BYOK.")
    if not _key_shape_ok(raw):
        return ByokState("invalid", reason=f"{BYOK_PROVIDER_KEY_HEADER} must be a single valid API key value.")
    return ByokState("accepted", provider, raw, "request")


def byok_response_headers(state: ByokState, routed: bool) -> dict:
    if state.tag == "absent":
        return {}
    return {BYOK_ACK_HEADER: "invalid" if state.tag == "invalid" else ("routed" if routed else "accepted")}


class ModelGate:
    """One row of the model gating table."""

    def __init__(self, model: str, premium: bool = False, internal_only: bool = False, servable: bool = True, alias_of: str | None = None):
        self.model, self.premium, self.internal_only, self.servable, self.alias_of = model, premium, internal_only, servable, alias_of


def billing_disclosure(zero_charge: bool, receipt_ref: str | None, byok: bool) -> dict:
    if zero_charge:
        return {"mode": "zero_charge", "receipt_required": False}
    if receipt_ref is not None:
        return {"mode": "receipt_backed", "receipt_required": True}
    if byok:
        return {"mode": "no_debit", "reason": "caller_provider_key", "receipt_required": False}
    return {"mode": "no_debit", "reason": "operator_exempt_or_unmetered", "receipt_required": False}


class LocalEngineAdapter:
    """Serves from an in-process ``openagents_b200.serve.server.ServerState``."""

    def __init__(self, state, adapter_id: str = "openagents-network", model_alias: dict | None = None):
        self.id, self.state, self.alias = adapter_id, state, model_alias or {}

    def complete(self, request: InferenceRequest):
        try:
            model = self.state.model(self.alias.get(request.model, request.model))
        except KeyError:
            raise InferenceAdapterError(self.id, "request_rejected", f"model {request.model!r} is not served here", False, 404)
        try:
            greedy = float(request.passthrough_params.get("temperature") or 0.0) == 0.0
            raw = self.state.serve_contract(model, {"messages": [dict(m) for m in request.messages],
                                                    "passthroughParams": dict(request.passthrough_params),
                                                    "requireExactGreedyParity": greedy})
        except (ValueError, TypeError) as e:        # a request the engine refuses (too long for the context, a mistyped option)
            raise InferenceAdapterError(self.id, "request_rejected", str(e), False, 400)
        except MemoryError as e:
            raise InferenceAdapterError(self.id, "service_overloaded", str(e), True, 503)
        serve = normalize_serve_response(raw)
        if serve is None:
            raise InferenceAdapterError(self.id, "malformed_response", "engine returned a malformed serve response")
        if greedy and not serve["parityVerified"]:
            raise InferenceAdapterError(self.id, "fabric_parity_unverified", "greedy decode was not reproducible")
        result = InferenceResult(serve["content"], serve["finishReason"], serve["servedModel"], serve["usage"])
        receipt = {k: serve[k] for k in ("servingRunRef", "servedModel", "stages", "parityMode", "parityVerified")}
        receipt["sharded"] = len(serve["stages"]) > 1
        return result, receipt


class ChatGateway:
    def __init__(self, registry: ProviderRegistry, keys: list[ApiKey], pricing: PricingTable | None = None, plan=None, now=time.time,
                 sleep=lambda ms: None, default_price_msat_per_token: tuple[int, int] = (1, 4), gates: list[ModelGate] | None = None,
                 internal_accounts: tuple = (), byok_adapter_factory=None, resolve_account_byok=None, ledger=None,
                 platform_funded: bool = True):
        """``gates``: the model gating table (a model without a row is not gated).  ``byok_adapter_factory(provider,
        api_key)`` builds the adapter a caller-funded request is sent to; ``resolve_account_byok(account)`` returns
        ``(provider, api_key)`` for an account with an attached provider key, or None.  ``ledger``: a
        ``ServedTokensLedger``.  ``platform_funded=False``: only caller-funded or no-meter keys are served."""
        self.registry, self.pricing, self.plan, self.now, self.sleep = registry, pricing, plan, now, sleep
        self.keys = {k.key: k for k in keys}
        self.default_price = default_price_msat_per_token
        self.lock = threading.Lock()
        self.telemetry: list[dict] = []                      # the most recent records (at most ``telemetry_keep``)
        self.telemetry_keep = 10_000
        self.route_totals: dict[str, list[int]] = {}         # route -> [requests, prompt tokens, completion tokens, msat], since start
        self.gates = {g.model: g for g in (gates or [])}
        self.internal_accounts = frozenset(internal_accounts)
        self.byok_adapter_factory, self.resolve_account_byok = byok_adapter_factory, resolve_account_byok
        self.ledger, self.platform_funded = ledger, platform_funded

    # ---- steps
    def authenticate(self, authorization: str | None) -> ApiKey:
        if not authorization or not authorization.lower().startswith("bearer "):
            raise GatewayError(401, "missing_api_key", "send Authorization: Bearer <key>")
        k = self.keys.get(authorization[7:].strip())
        if k is None:
            raise GatewayError(401, "invalid_api_key", "unknown API key")
        return k

    @staticmethod
    def decode_body(body) -> dict:
        if isinstance(body, (bytes, str)):
            try:
                body = json.loads(body)
            except json.JSONDecodeError:
                raise GatewayError(400, "invalid_json", "request body is not JSON")
        if not isinstance(body, dict):
            raise GatewayError(400, "invalid_request", "request body must be an object")
        if not isinstance(body.get("model"), str) or not body["model"].strip():
            raise GatewayError(400, "invalid_request", "model is required")
        msgs = body.get("messages")
        if not isinstance(msgs, list) or not msgs or not all(isinstance(m, dict) and isinstance(m.get("role"), str) and isinstance(m.get("content"), str) for m in msgs):
            raise GatewayError(400, "invalid_request", "messages must be a non-empty list of {role, content}")
        mt = body.get("max_tokens")
        if mt is not None and not (isinstance(mt, int) and not isinstance(mt, bool) and 1 <= mt <= 131072):
            raise GatewayError(400, "invalid_request", "max_tokens out of range")
        try:                             # the checks the model server applies, applied before any lane is tried
            schema.sampling_fields(body)
            schema.boolean(body, "stream")
            schema.tools(body)
            schema.string(body, "user")
        except schema.BadRequest as e:
            raise GatewayError(400, "invalid_request", str(e))
        for m in msgs:
            if m.get("stable_kind") is not None and not (isinstance(m["stable_kind"], str) and m["stable_kind"] in pc.STABLE_ORDINAL):
                raise GatewayError(400, "invalid_request", f"stable_kind must be one of {', '.join(pc.STABLE_ORDINAL)}")
        return body

    def price_msat(self, model: str, usage: InferenceUsage) -> int:
        e = self.pricing.lookup(model) if self.pricing else None
        if e is not None:     # USD per million tokens -> msat at a fixed planning rate of 1 USD = 1,000,000 msat
            return int(round(usage.prompt_tokens * e.input_usd_per_mtok + usage.completion_tokens * e.output_usd_per_mtok))
        pi, po = self.default_price
        return usage.prompt_tokens * pi + usage.completion_tokens * po

    # ---- the route
    def handle(self, authorization: str | None, body, session: str | None = None, headers: dict | None = None) -> tuple[int, dict | list[str]]:
        """Returns (status, JSON object) or, for ``stream``, (200, list of SSE frames)."""
        status, _, out = self.handle_with_headers(authorization, body, session, headers)
        return status, out

    def handle_with_headers(self, authorization: str | None, body, session: str | None = None, headers: dict | None = None):
        """As ``handle`` plus the response headers (the caller-funding acknowledgement)."""
        t0 = self.now()
        byok = ByokState("absent")
        try:
            key = self.authenticate(authorization)
            byok = resolve_byok(headers)
            if byok.tag == "invalid":
                return 400, byok_response_headers(byok, False), {"error": {"message": byok.reason, "type": "invalid_byok_provider_key",
                                                                           "code": "invalid_byok_provider_key"}}
            if byok.tag == "absent":       # request headers win and stay ephemeral; else a key attached to the account
                attached = None
                if self.resolve_account_byok is not None:
                    try:
                        attached = self.resolve_account_byok(key.account)
                    except Exception:      # noqa: BLE001 - a failing lookup means "no attached key", never a failed request
                        attached = None
                if attached is None and key.byok.get("provider") and key.byok.get("api_key"):
                    attached = (key.byok["provider"], key.byok["api_key"])
                if attached is not None and attached[0] in BYOK_PROVIDERS and _key_shape_ok(attached[1]):
                    byok = ByokState("accepted", attached[0], attached[1], "account")
            with self.lock:
                if key.inflight >= key.max_inflight:
                    raise GatewayError(429, "fair_share_exceeded", "too many requests in flight for this key")
                key.inflight += 1
            try:
                status, out = self._handle(key, body, session, t0, byok)
                return status, byok_response_headers(byok, status == 200), out
            finally:
                with self.lock:
                    key.inflight -= 1
        except GatewayError as e:
            return e.status, byok_response_headers(byok, False), e.body()

    def gate(self, key: ApiKey, model: str) -> str:
        """Model gating: returns the model id to route (aliases resolved) or raises.  Servability comes first: a model
        nobody can serve is never the caller's balance or allow-list problem."""
        g = self.gates.get(model)
        if g is not None and g.alias_of:
            model, g = g.alias_of, self.gates.get(g.alias_of)
        if g is not None and not g.servable:
            raise GatewayError(503, "model_unavailable", f"{model!r} has no serving lane right now")
        if key.allowed_models is not None and model not in key.allowed_models:
            raise GatewayError(403, "model_not_allowed", f"this key may not use {model!r}")
        if g is not None and g.internal_only and key.account not in self.internal_accounts:
            raise GatewayError(403, "model_not_allowed", f"{model!r} is limited to internal accounts")
        if g is not None and g.premium and not (key.premium or key.account in self.internal_accounts):
            raise GatewayError(403, "premium_model_requires_entitlement", f"{model!r} needs a premium entitlement")
        return model

    def _handle(self, key: ApiKey, body, session, t0, byok: ByokState | None = None):
        byok = byok or ByokState("absent")
        body = self.decode_body(body)
        requested = body["model"].strip()
        model = self.gate(key, requested)
        caller_paid = byok.tag == "accepted"
        if not caller_paid and not key.no_meter:
            if not self.platform_funded:
                raise GatewayError(503, "platform_funding_unavailable",
                                   "Platform-funded inference is unavailable. Configure a supported BYOK provider account.")
            if key.balance_msat <= 0:
                raise GatewayError(402, "insufficient_balance", "the key has no balance")
        layout = pc.assemble_stable_prompt_layout([(m, m.get("stable_kind")) for m in body["messages"]])
        messages = tuple({"role": m["role"], "content": m["content"]} for m in layout["messages"])
        affinity_raw = pc.derive_cache_affinity_key(key.account, session)
        passthrough = {k: body[k] for k in ("max_tokens", "temperature", "top_p", "top_k", "stop", "seed") if k in body}
        passthrough.update(pc.session_affinity_params(pc.hash_cache_affinity_key(affinity_raw)))
        request = InferenceRequest(model, messages, bool(body.get("stream")), passthrough)
        plan = self.plan(model) if self.plan else select_adapter_plan(model, self.pricing)
        events = []
        t_dispatch = self.now()
        registry = self.registry
        if caller_paid:                  # the caller's own provider account answers; no overflow onto platform capacity
            if self.byok_adapter_factory is None:
                raise GatewayError(503, "byok_provider_unavailable", f"no adapter is configured for provider {byok.provider!r}")
            adapter = self.byok_adapter_factory(byok.provider, byok.api_key)
            registry = ProviderRegistry()
            registry.register(adapter)
            plan = [adapter.id]
        try:
            d = dispatch_with_overflow(request, lambda a, r: a.complete(r), registry, plan=plan, sleep=self.sleep, telemetry=events.append)
        except InferenceAdapterError as e:
            status = e.http_status if e.http_status in (400, 404, 429) else (503 if e.retryable else 502)
            raise GatewayError(status, e.kind, e.reason)
        t_done = self.now()
        out = d.value if isinstance(d.value, tuple) else (d.value, {})      # an external adapter returns the bare result
        result, receipt = out[0], out[1]
        paid = out[2] if len(out) > 2 else None
        price = self.price_msat(result.served_model if self.pricing and self.pricing.lookup(result.served_model) else model, result.usage)
        debited = not caller_paid and not key.no_meter
        if debited:
            with self.lock:
                key.balance_msat -= price
        else:
            price = 0
        rid = "chatcmpl-" + uuid.uuid4().hex[:24]
        receipt_ref = f"receipt.inference.{rid}" if debited and price > 0 else None
        billing = billing_disclosure(zero_charge=debited and price == 0, receipt_ref=receipt_ref, byok=caller_paid)
        if self.ledger is not None:      # the ledger is a projection of the answer: it never fails the request
            try:
                self.ledger.record(rid, model, result.usage.prompt_tokens, result.usage.completion_tokens, account_ref=key.account,
                                   adapter_id=d.adapter_id, demand_kind="internal" if key.account in self.internal_accounts else "external",
                                   served_model=result.served_model)
            except Exception:            # noqa: BLE001
                pass
        record = rt.build_record(
            request_id=rid, requested_model=model, served_model=result.served_model, route=d.adapter_id, provider=d.adapter_id,
            request_class="interactive_stream" if request.stream else "async_job", prompt_tokens=result.usage.prompt_tokens,
            completion_tokens=result.usage.completion_tokens, total_tokens=result.usage.total_tokens,
            cached_input_tokens=result.usage.cached_prompt_tokens, total_wall_clock_ms=(t_done - t0) * 1000,
            provider_time_ms=(t_done - t_dispatch) * 1000, gateway_overhead_ms=(t_dispatch - t0) * 1000,
            cache_affinity_key_raw=affinity_raw, fallback_reason=d.fallback_reason, price_msat=price,
            verification_class="exact_trace_replay" if receipt.get("parityVerified") else "unverified",
            executed_verdict="passed" if receipt.get("parityVerified") else "not_executed",
            quantization=None, speculation={"mode": "none"}, settlement_state="not_applicable")
        if d.adapter_id == "openagents-network":
            record["quantization"] = engine_quantization("Q4_K") if "q4" in result.served_model.lower() else record["quantization"]
        with self.lock:
            self.telemetry.append(record)
            if len(self.telemetry) > 2 * self.telemetry_keep:
                del self.telemetry[: len(self.telemetry) - self.telemetry_keep]
            tot = self.route_totals.setdefault(d.adapter_id, [0, 0, 0, 0])
            tot[0] += 1
            tot[1] += result.usage.prompt_tokens
            tot[2] += result.usage.completion_tokens
            tot[3] += price
        usage = {"prompt_tokens": result.usage.prompt_tokens, "completion_tokens": result.usage.completion_tokens,
                 "total_tokens": result.usage.total_tokens}
        if result.usage.cached_prompt_tokens is not None:
            usage["prompt_tokens_details"] = {"cached_tokens": result.usage.cached_prompt_tokens}
        ext = {"telemetry": rt.block_from_record(record, f"telemetry.{rid}"), "receipt": receipt, "route": d.adapter_id,
               "overflow_count": d.overflow_count, "stable_prefix_hash": layout["stablePrefixHash"], "price_msat": price,
               "clears_paid_traffic": paid, "billing": billing, "receipt_ref": receipt_ref,
               "requested_model": requested}
        created = int(t_done)
        if request.stream:
            frames = []
            head = {"id": rid, "object": "chat.completion.chunk", "created": created, "model": result.served_model}
            frames.append("data: " + json.dumps({**head, "choices": [{"index": 0, "delta": {"role": "assistant"}, "finish_reason": None}]}) + "\n\n")
            text = result.content
            for i in range(0, len(text), 16):        # the upstream answer is re-framed into OpenAI delta chunks
                frames.append("data: " + json.dumps({**head, "choices": [{"index": 0, "delta": {"content": text[i:i + 16]}, "finish_reason": None}]}) + "\n\n")
            frames.append("data: " + json.dumps({**head, "choices": [{"index": 0, "delta": {}, "finish_reason": result.finish_reason}], "usage": usage,
                                                 "openagents": ext}) + "\n\n")
            frames.append("data: [DONE]\n\n")
            return 200, frames
        return 200, {"id": rid, "object": "chat.completion", "created": created, "model": result.served_model,
                     "choices": [{"index": 0, "message": {"role": "assistant", "content": result.content}, "finish_reason": result.finish_reason}],
                     "usage": usage, "openagents": ext}

    def models(self) -> dict:
        return {"object": "list", "data": [{"id": i, "object": "model", "owned_by": "openagents"} for i in self.registry.ids()]}

    def quote(self, model: str, prompt_tokens: int, max_tokens: int) -> dict:
        """``/v1/quote``: worst-case price of a request."""
        return {"model": model, "maxPriceMsat": self.price_msat(model, InferenceUsage(prompt_tokens, max_tokens, prompt_tokens + max_tokens))}
