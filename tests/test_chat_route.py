"""The gateway's chat-completions route end to end on CPU: key -> fair share -> plan -> overflow -> local engine -> metering -> telemetry."""
import json

import pytest

from openagents_b200.gateway import chat_route as cr
from openagents_b200.gateway import fabric as fb
from openagents_b200.gateway import router as rt
from openagents_b200.models.config import TINY_LLAMA
from openagents_b200.models.weights import PLAN_Q8_0, random_weights, save_gguf
from openagents_b200.receipts import manifests as mf
from openagents_b200.serve.backend import CpuBackend
from openagents_b200.serve.server import ServedModel, ServerState


@pytest.fixture(scope="module")
def state(tmp_path_factory):
    cfg = TINY_LLAMA.with_(vocab=512, d_model=64, n_heads=2, n_kv_heads=1, head_dim=32, ffn=128)
    p = str(tmp_path_factory.mktemp("m") / "tiny.gguf")
    save_gguf(p, cfg, random_weights(cfg, 0), PLAN_Q8_0)
    return ServerState([ServedModel("tiny", CpuBackend.from_gguf(p), mf.artifact_digest(p), max_num_seqs=4)])


class _Failing:
    def __init__(self, id, err):
        self.id, self.err, self.calls = id, err, 0

    def complete(self, request):
        self.calls += 1
        raise self.err


def _gateway(state, keys=None, fireworks_error=None):
    reg = fb.ProviderRegistry()
    fw = _Failing(rt.FIREWORKS, fireworks_error or fb.InferenceAdapterError(rt.FIREWORKS, "rate_limited", "429", True, 429))
    reg.register(fw)
    reg.register(cr.LocalEngineAdapter(state, model_alias={"qwen-tiny": "tiny"}))
    keys = keys or [cr.ApiKey("k1", "acct1", balance_msat=10_000, max_inflight=1), cr.ApiKey("k2", "acct2", 10_000, allowed_models=("other",)),
                    cr.ApiKey("k3", "acct3", 0)]
    return cr.ChatGateway(reg, keys), fw


BODY = {"model": "qwen-tiny", "messages": [{"role": "user", "content": "hello"}, {"role": "system", "content": "be brief"}], "max_tokens": 8}


def test_route_overflows_to_local_engine_and_meters(state):
    gw, fw = _gateway(state)
    status, out = gw.handle("Bearer k1", json.dumps(BODY), session="s1")
    assert status == 200 and out["object"] == "chat.completion" and out["choices"][0]["message"]["role"] == "assistant"
    ext = out["openagents"]
    assert fw.calls == 1 and ext["route"] == "openagents-network" and ext["overflow_count"] == 1
    assert ext["receipt"]["parityVerified"] is True and ext["receipt"]["sharded"] is False
    u = out["usage"]
    assert u["completion_tokens"] == 8 and ext["price_msat"] == u["prompt_tokens"] * 1 + 8 * 4
    assert gw.keys["k1"].balance_msat == 10_000 - ext["price_msat"] and gw.keys["k1"].inflight == 0
    rec = gw.telemetry[-1]
    assert rec["fallbackReason"] == "rate_limited" and rec["verificationClass"] == "exact_trace_replay" and rec["executedVerdict"] == "passed"
    assert rec["cacheAffinityKeyHash"].startswith("cacheaff:fnv1a32:") and ext["telemetry"]["detailRef"].startswith("telemetry.chatcmpl-")
    assert ext["stable_prefix_hash"].startswith("prefix:fnv1a32:")
    # same request again: same content (greedy) and the stable prefix hash is unchanged
    _, out2 = gw.handle("Bearer k1", BODY)
    assert out2["choices"][0]["message"]["content"] == out["choices"][0]["message"]["content"]
    assert out2["openagents"]["stable_prefix_hash"] == ext["stable_prefix_hash"]


def test_stream_is_reframed_as_sse(state):
    gw, _ = _gateway(state)
    status, frames = gw.handle("Bearer k1", dict(BODY, stream=True))
    assert status == 200 and frames[-1] == "data: [DONE]\n\n" and all(f.startswith("data: ") and f.endswith("\n\n") for f in frames)
    chunks = [json.loads(f[6:]) for f in frames[:-1]]
    assert chunks[0]["choices"][0]["delta"] == {"role": "assistant"} and chunks[-1]["choices"][0]["finish_reason"] in ("length", "stop")
    text = "".join(c["choices"][0]["delta"].get("content", "") for c in chunks)
    _, plain = gw.handle("Bearer k1", BODY)
    assert text == plain["choices"][0]["message"]["content"] and chunks[-1]["usage"]["completion_tokens"] == 8


def test_refusals(state):
    gw, fw = _gateway(state)
    assert gw.handle(None, BODY)[0] == 401 and gw.handle("Bearer nope", BODY)[1]["error"]["code"] == "invalid_api_key"
    assert gw.handle("Bearer k2", BODY)[1]["error"]["code"] == "model_not_allowed"
    assert gw.handle("Bearer k3", BODY)[0] == 402
    assert gw.handle("Bearer k1", "{not json")[1]["error"]["code"] == "invalid_json"
    assert gw.handle("Bearer k1", {"model": "qwen-tiny", "messages": []})[0] == 400
    assert gw.handle("Bearer k1", dict(BODY, max_tokens=0))[0] == 400
    gw.keys["k1"].inflight = 1
    assert gw.handle("Bearer k1", BODY) == (429, {"error": {"message": "too many requests in flight for this key", "type": "fair_share_exceeded", "code": "fair_share_exceeded"}})
    gw.keys["k1"].inflight = 0
    # a non-retryable failure on the first lane surfaces instead of overflowing
    gw2, fw2 = _gateway(state, fireworks_error=fb.InferenceAdapterError(rt.FIREWORKS, "request_rejected", "bad request", False, 400))
    status, out = gw2.handle("Bearer k1", BODY)
    assert status == 400 and out["error"]["code"] == "request_rejected" and gw2.keys["k1"].balance_msat == 10_000
    # an unknown model on every lane
    status, out = gw.handle("Bearer k1", dict(BODY, model="qwen-unknown"))
    assert status in (404, 502, 503) and gw.keys["k1"].inflight == 0
    assert gw.quote("qwen-tiny", 100, 50) == {"model": "qwen-tiny", "maxPriceMsat": 300} and rt.FIREWORKS in [m["id"] for m in gw.models()["data"]]


class _Echo:
    """An external provider reached with the caller's own key."""

    def __init__(self, provider, api_key):
        self.id, self.api_key, self.calls = f"byok-{provider}", api_key, 0

    def complete(self, request):
        self.calls += 1
        return fb.InferenceResult("echo:" + request.messages[-1]["content"], "stop", request.model, fb.InferenceUsage(5, 3, 8))


def test_caller_funded_request_is_routed_not_debited_and_acknowledged(state):
    from openagents_b200.gateway.observability import ServedTokensLedger
    made = []

    def factory(provider, api_key):
        made.append(_Echo(provider, api_key))
        return made[-1]

    reg = fb.ProviderRegistry()
    reg.register(cr.LocalEngineAdapter(state, model_alias={"qwen-tiny": "tiny"}))
    ledger = ServedTokensLedger()
    gw = cr.ChatGateway(reg, [cr.ApiKey("k", "acct", 0)], byok_adapter_factory=factory, ledger=ledger, platform_funded=False)
    hdr = {"X-OpenAgents-Provider": "OpenRouter", "x-openagents-provider-key": "sk-or-0123456789abcdef"}
    status, rh, out = gw.handle_with_headers("Bearer k", BODY, headers=hdr)
    assert status == 200 and rh == {cr.BYOK_ACK_HEADER: "routed"} and made[0].calls == 1 and made[0].api_key == "sk-or-0123456789abcdef"
    ext = out["openagents"]
    assert ext["route"] == "byok-openrouter" and ext["price_msat"] == 0 and gw.keys["k"].balance_msat == 0
    assert ext["billing"] == {"mode": "no_debit", "reason": "caller_provider_key", "receipt_required": False} and ext["receipt_ref"] is None
    assert ledger.total() == 8 and list(ledger.rows.values())[0]["adapterId"] == "byok-openrouter"
    assert "sk-or" not in repr(cr.resolve_byok(hdr))                                   # the key never prints
    # unsupported provider / malformed key: 400 with the acknowledgement header, nothing dispatched
    for bad in ({"x-openagents-provider": "acme", "x-openagents-provider-key": "sk-or-0123456789abcdef"},
                {"x-openagents-provider": "openrouter", "x-openagents-provider-key": "two keys"},
                {"x-openagents-provider-key": "sk-or-0123456789abcdef"}):
        status, rh, out = gw.handle_with_headers("Bearer k", BODY, headers=bad)
        assert status == 400 and rh == {cr.BYOK_ACK_HEADER: "invalid"} and out["error"]["code"] == "invalid_byok_provider_key"
    assert len(made) == 1
    # without caller funding the platform does not pay
    status, rh, out = gw.handle_with_headers("Bearer k", BODY)
    assert status == 503 and out["error"]["code"] == "platform_funding_unavailable" and rh == {}
    # a key attached to the account is used when the request carries none; request headers win over it
    gw.resolve_account_byok = lambda account: ("openrouter", "sk-or-attached-000000") if account == "acct" else None
    status, rh, out = gw.handle_with_headers("Bearer k", BODY)
    assert status == 200 and rh == {cr.BYOK_ACK_HEADER: "routed"} and made[-1].api_key == "sk-or-attached-000000"
    status, rh, out = gw.handle_with_headers("Bearer k", BODY, headers=hdr)
    assert made[-1].api_key == "sk-or-0123456789abcdef"
    # a resolver that throws means "no attached key"
    def boom(account):
        raise RuntimeError("db down")
    gw.resolve_account_byok = boom
    assert gw.handle("Bearer k", BODY)[0] == 503


def test_model_gating_table_and_billing_modes(state):
    from openagents_b200.gateway.observability import ServedTokensLedger
    reg = fb.ProviderRegistry()
    reg.register(cr.LocalEngineAdapter(state, model_alias={"qwen-tiny": "tiny", "qwen-pro": "tiny", "qwen-lab": "tiny"}))
    gates = [cr.ModelGate("qwen-pro", premium=True), cr.ModelGate("qwen-lab", internal_only=True), cr.ModelGate("qwen-dead", servable=False),
             cr.ModelGate("qwen-latest", alias_of="qwen-pro")]
    ledger = ServedTokensLedger()
    keys = [cr.ApiKey("plain", "a1", 10_000), cr.ApiKey("prem", "a2", 10_000, premium=True), cr.ApiKey("ops", "ops1", 0, no_meter=True),
            cr.ApiKey("broke", "a3", 0)]
    gw = cr.ChatGateway(reg, keys, gates=gates, internal_accounts=("ops1",), ledger=ledger, plan=lambda m: ["openagents-network"])
    body = lambda m: {**BODY, "model": m}
    assert gw.handle("Bearer plain", body("qwen-pro"))[1]["error"]["code"] == "premium_model_requires_entitlement"
    assert gw.handle("Bearer plain", body("qwen-latest"))[1]["error"]["code"] == "premium_model_requires_entitlement"      # alias resolves first
    assert gw.handle("Bearer plain", body("qwen-lab"))[1]["error"]["code"] == "model_not_allowed"
    # servability is checked before balance: a dead model is a 503 even for a key without balance
    assert gw.handle("Bearer broke", body("qwen-dead")) [0] == 503
    assert gw.handle("Bearer broke", body("qwen-tiny"))[1]["error"]["code"] == "insufficient_balance"
    status, out = gw.handle("Bearer prem", body("qwen-latest"))
    assert status == 200 and out["openagents"]["requested_model"] == "qwen-latest"
    assert out["openagents"]["billing"] == {"mode": "receipt_backed", "receipt_required": True}
    assert out["openagents"]["receipt_ref"].startswith("receipt.inference.chatcmpl-")
    # operator-owned capacity: internal account, never debited, demand labelled internal in the ledger
    status, out = gw.handle("Bearer ops", body("qwen-lab"))
    assert status == 200 and out["openagents"]["billing"]["reason"] == "operator_exempt_or_unmetered" and out["openagents"]["price_msat"] == 0
    kinds = sorted(r["demandKind"] for r in ledger.rows.values())
    assert kinds == ["external", "internal"]
    # a model without a row is not gated
    assert gw.handle("Bearer plain", body("qwen-tiny"))[0] == 200


def test_gateway_reaches_a_live_model_server_across_the_process_boundary(tmp_path):
    """The whole serving call stack with the hop that is a process boundary in production: gateway route -> lane plan ->
    admitted network adapter (registration + heartbeat + payout snapshot) -> serve wire contract over the HTTP transport with a
    bearer token -> this package's model server (``/v1/serve``: tokenize, prefill, decode, a second greedy decode for parity) ->
    normalised response, stage-count and parity gates, receipt, metering.  A node that stops heart-beating is refused before
    any request leaves."""
    import threading
    import time
    from datetime import datetime, timezone
    from openagents_b200.serve.server import serve
    cfg = TINY_LLAMA.with_(vocab=512, d_model=64, n_heads=2, n_kv_heads=1, head_dim=32, ffn=128)
    p = str(tmp_path / "tiny.gguf")
    save_gguf(p, cfg, random_weights(cfg, 0), PLAN_Q8_0)
    live = ServerState([ServedModel("qwen-tiny", CpuBackend.from_gguf(p), mf.artifact_digest(p), max_num_seqs=4)])
    httpd = serve(live, "127.0.0.1", 0)
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    try:
        now = [time.time()]
        hb = [datetime.fromtimestamp(now[0], timezone.utc).strftime("%Y-%m-%dT%H:%M:%SZ")]
        snap = lambda: fb.ServingSnapshot("pylon.b200.1", "active", ("capability.serve.qwen-tiny",), ("lane.openagents-network",), hb[0], "healthy", True, "spark.target.1")
        transport = fb.make_http_transport(f"http://127.0.0.1:{httpd.server_address[1]}/v1/serve", "node-bearer-token")
        adapter = fb.OpenAgentsNetworkAdapter(dispatch=fb.dispatch_psionic_serve(transport),
                                              admission=lambda: fb.decide_admission(snap(), "capability.serve.qwen-tiny", int(now[0] * 1000)))
        reg = fb.ProviderRegistry()
        reg.register(_Failing(rt.FIREWORKS, fb.InferenceAdapterError(rt.FIREWORKS, "rate_limited", "429", True, 429)))
        reg.register(adapter)
        gw = cr.ChatGateway(reg, [cr.ApiKey("k1", "acct1", balance_msat=10_000)])
        status, out = gw.handle("Bearer k1", json.dumps(BODY))
        assert status == 200, out
        ext = out["openagents"]
        assert ext["route"] == "openagents-network" and ext["receipt"]["parityVerified"] is True and ext["receipt"]["sharded"] is False
        assert out["usage"]["completion_tokens"] == 8 and gw.keys["k1"].balance_msat == 10_000 - ext["price_msat"]
        stats = live.model("qwen-tiny").sched.stats
        assert stats["requests"] >= 2                                  # the answer and its parity replay ran on the server
        # the node goes quiet: the admission gate refuses before dispatch, nothing reaches the server, the caller gets a typed failure
        served_before = stats["requests"]
        now[0] += 600
        status, out = gw.handle("Bearer k1", json.dumps(BODY))
        assert status >= 400 and "heartbeat_stale" in json.dumps(out)
        assert live.model("qwen-tiny").sched.stats["requests"] == served_before
    finally:
        httpd.shutdown()


@pytest.mark.parametrize("patch,needle", [
    ({"temperature": True}, "temperature"), ({"temperature": [1]}, "temperature"), ({"top_p": 2}, "top_p"), ({"top_k": 3.5}, "top_k"),
    ({"seed": "x"}, "seed"), ({"stop": 0}, "stop"), ({"stop": [[]]}, "stop"), ({"stream": 1e9}, "stream"), ({"tools": 3.5}, "tools"),
    ({"user": [[]]}, "user"), ({"max_tokens": True}, "max_tokens"), ({"max_tokens": 0}, "max_tokens"),
    ({"messages": [{"role": "user", "content": "hi", "stable_kind": False}]}, "stable_kind"),
    ({"messages": [{"role": "user", "content": "hi", "stable_kind": "nope"}]}, "stable_kind"),
])
def test_mistyped_options_are_refused_at_the_gateway_before_any_lane(state, patch, needle):
    gw, fw = _gateway(state)
    before = gw.keys["k1"].balance_msat
    status, out = gw.handle("Bearer k1", json.dumps({**BODY, **patch}))
    assert status == 400 and out["error"]["code"] == "invalid_request" and needle in out["error"]["message"], out
    assert fw.calls == 0 and gw.keys["k1"].balance_msat == before and gw.keys["k1"].inflight == 0


def test_engine_refusal_reaches_the_caller_as_a_400_not_an_exception(state):
    """A request the gateway's own checks pass but the engine refuses (longer than its context window) comes back from the
    in-process adapter as a typed, non-retryable 400."""
    gw, _ = _gateway(state)
    long_text = "word " * 6000
    status, out = gw.handle("Bearer k1", json.dumps({**BODY, "messages": [{"role": "user", "content": long_text}]}))
    assert status == 400 and out["error"]["code"] == "request_rejected" and "context" in out["error"]["message"], out
    assert gw.keys["k1"].inflight == 0


def test_gateway_memory_is_bounded_while_its_counters_stay_exact(state):
    gw, _ = _gateway(state, keys=[cr.ApiKey("k1", "acct1", balance_msat=10**9, max_inflight=4)])
    gw.telemetry_keep = 3
    for _ in range(8):
        assert gw.handle("Bearer k1", json.dumps({**BODY, "max_tokens": 1}))[0] == 200
    assert 3 <= len(gw.telemetry) <= 6                                     # trimmed in blocks, never beyond twice the window
    n, prompt, completion, msat = gw.route_totals["openagents-network"]
    assert n == 8 and completion == 8 and prompt > 0 and msat == 10**9 - gw.keys["k1"].balance_msat
