"""The gateway as its own HTTP process in front of a model server: key -> plan -> serve wire contract over HTTP (bearer-protected
node) -> metering; streaming; refusals; the configuration loader."""
import json
import subprocess
import sys
import threading
import urllib.error
import urllib.request

import pytest

from openagents_b200.gateway import server as gs
from openagents_b200.models.config import TINY_LLAMA
from openagents_b200.models.weights import PLAN_Q8_0, random_weights, save_gguf
from openagents_b200.receipts import manifests as mf
from openagents_b200.serve.backend import CpuBackend
from openagents_b200.serve.server import ServedModel, ServerState, serve as serve_model


def _call(url, body=None, key=None, raw=None, headers=None):
    data = raw if raw is not None else (json.dumps(body).encode() if body is not None else None)
    h = {"Content-Type": "application/json", **(headers or {})}
    if key:
        h["Authorization"] = f"Bearer {key}"
    try:
        with urllib.request.urlopen(urllib.request.Request(url, data=data, headers=h), timeout=60) as r:
            return r.status, r.read(), dict(r.headers)
    except urllib.error.HTTPError as e:
        return e.code, e.read(), dict(e.headers)


@pytest.fixture(scope="module")
def stack(tmp_path_factory):
    d = tmp_path_factory.mktemp("gw")
    cfg = TINY_LLAMA.with_(vocab=512, d_model=64, n_heads=2, n_kv_heads=1, head_dim=32, ffn=128)
    p = str(d / "tiny.gguf")
    save_gguf(p, cfg, random_weights(cfg, 0), PLAN_Q8_0)
    node_state = ServerState([ServedModel("tiny", CpuBackend.from_gguf(p), mf.artifact_digest(p), max_num_seqs=4)])
    node_state.api_key = "node-secret"
    node = serve_model(node_state, "127.0.0.1", 0)
    threading.Thread(target=node.serve_forever, daemon=True).start()
    node_url = f"http://127.0.0.1:{node.server_address[1]}"
    config = {"keys": [{"key": "sk-a", "account": "acct.a", "balance_msat": 50_000, "max_inflight": 2},
                       {"key": "sk-broke", "account": "acct.b", "balance_msat": 0},
                       {"key": "sk-narrow", "account": "acct.c", "balance_msat": 1000, "allowed_models": ["other"]}],
              "nodes": [{"id": "hydralisk", "kind": "openai", "endpoint": "http://127.0.0.1:9/v1", "bearer": "x", "timeout_s": 2},
                        {"id": "openagents-network", "kind": "serve", "endpoint": node_url, "bearer": "node-secret"}],
              "plans": {"*": ["hydralisk", "openagents-network"]},
              "gates": [{"model": "fast", "alias_of": "tiny"}, {"model": "gone", "servable": False}],
              "ledger": str(d / "ledger.jsonl"), "admin_key": "adm"}
    gw = gs.build_gateway(config)
    httpd = gs.serve(gw, "127.0.0.1", 0, config["admin_key"])
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    yield f"http://127.0.0.1:{httpd.server_address[1]}", gw, node_state, node_url, config, d
    httpd.shutdown()
    node.shutdown()


BODY = {"model": "tiny", "messages": [{"role": "user", "content": "hello"}], "max_tokens": 6}


def test_request_crosses_two_process_boundaries_and_is_metered(stack):
    base, gw, node_state, node_url, _, _ = stack
    code, raw, _ = _call(node_url + "/v1/serve", BODY)                         # the node itself refuses a caller without its key
    assert code == 401 and json.loads(raw)["error"]["type"] == "invalid_api_key"
    before = gw.keys["sk-a"].balance_msat
    code, raw, _ = _call(base + "/v1/chat/completions", BODY, key="sk-a")
    out = json.loads(raw)
    assert code == 200, out
    ext = out["openagents"]
    # the first adapter of the plan is unreachable: the request overflowed onto the node, which answered with a verified receipt
    assert ext["route"] == "openagents-network" and ext["overflow_count"] == 1 and ext["receipt"]["parityVerified"] is True
    assert out["usage"]["completion_tokens"] == 6 and out["choices"][0]["message"]["role"] == "assistant"
    assert gw.keys["sk-a"].balance_msat == before - ext["price_msat"] and ext["price_msat"] > 0 and ext["billing"]["mode"] == "receipt_backed"
    assert node_state.model("tiny").sched.stats["requests"] >= 2                # the answer and its parity replay
    code, raw, _ = _call(base + "/v1/chat/completions", {**BODY, "model": "fast"}, key="sk-a")      # an alias from the gating table
    assert code == 200 and json.loads(raw)["openagents"]["requested_model"] == "fast"
    code, raw, _ = _call(base + "/metrics")
    text = raw.decode()
    assert 'b200_gateway_requests_total{route="openagents-network"} 2' in text and "b200_gateway_tokens_served_total" in text
    code, raw, _ = _call(base + "/admin/telemetry", key="adm")
    assert code == 200 and len(json.loads(raw)["records"]) == 2
    assert _call(base + "/admin/telemetry", key="sk-a")[0] == 404 and _call(base + "/admin/telemetry")[0] == 404


def test_stream_is_served_as_event_stream(stack):
    base = stack[0]
    code, raw, headers = _call(base + "/v1/chat/completions", {**BODY, "stream": True}, key="sk-a")
    assert code == 200 and headers["Content-Type"] == "text/event-stream"
    frames = [f[6:] for f in raw.decode().split("\n\n") if f.startswith("data: ")]
    assert frames[-1] == "[DONE]" and json.loads(frames[0])["choices"][0]["delta"] == {"role": "assistant"}
    last = json.loads(frames[-2])
    assert last["usage"]["completion_tokens"] == 6 and last["openagents"]["route"] == "openagents-network"
    text = "".join(json.loads(f)["choices"][0]["delta"].get("content", "") for f in frames[1:-2])
    code, raw, _ = _call(base + "/v1/chat/completions", BODY, key="sk-a")
    assert text == json.loads(raw)["choices"][0]["message"]["content"]           # greedy: the streamed text is the same answer


@pytest.mark.parametrize("key,body,raw,status,kind", [
    (None, BODY, None, 401, "missing_api_key"),
    ("sk-nope", BODY, None, 401, "invalid_api_key"),
    ("sk-broke", BODY, None, 402, "insufficient_balance"),
    ("sk-narrow", BODY, None, 403, "model_not_allowed"),
    ("sk-a", {**BODY, "model": "gone"}, None, 503, "model_unavailable"),
    ("sk-a", {**BODY, "messages": []}, None, 400, "invalid_request"),
    ("sk-a", {**BODY, "max_tokens": "six"}, None, 400, "invalid_request"),
    ("sk-a", {"messages": BODY["messages"]}, None, 400, "invalid_request"),
    ("sk-a", None, b"{", 400, "invalid_json"),
    ("sk-a", None, b"\xff\xfe", 400, "invalid_json"),
    ("sk-a", None, b"[1]", 400, "invalid_request"),
])
def test_refusals_are_typed(stack, key, body, raw, status, kind):
    base, gw = stack[0], stack[1]
    balance = gw.keys["sk-a"].balance_msat
    code, out, _ = _call(base + "/v1/chat/completions", body, key=key, raw=raw)
    assert code == status and json.loads(out)["error"]["code"] == kind, out
    assert gw.keys["sk-a"].balance_msat == balance and gw.keys["sk-a"].inflight == 0      # a refusal costs nothing and holds no slot


def test_quote_models_health_and_unknown_routes(stack):
    base = stack[0]
    code, raw, _ = _call(base + "/v1/quote?model=tiny&prompt_tokens=10&max_tokens=20")
    assert code == 200 and json.loads(raw) == {"model": "tiny", "maxPriceMsat": 10 * 1 + 20 * 4}
    assert _call(base + "/v1/quote?model=tiny&prompt_tokens=ten")[0] == 400 and _call(base + "/v1/quote")[0] == 400
    assert _call(base + "/v1/quote?model=tiny&prompt_tokens=-1&max_tokens=1")[0] == 400
    code, raw, _ = _call(base + "/v1/models")
    assert [m["id"] for m in json.loads(raw)["data"]] == ["hydralisk", "openagents-network"]
    assert json.loads(_call(base + "/health")[1])["status"] == "ok"
    assert _call(base + "/nope")[0] == 404 and _call(base + "/v1/embeddings", BODY, key="sk-a")[0] == 404


def test_configuration_errors_name_the_entry(stack, tmp_path):
    good = stack[4]
    for patch, needle in (({"keys": [{"key": "k"}]}, "keys[0]: account"), ({"nodes": []}, "at least one node"),
                          ({"nodes": [{"id": "n", "kind": "carrier-pigeon", "endpoint": "x"}]}, "kind must be"),
                          ({"nodes": [{"id": "n", "kind": "serve", "endpoint": "http://h"}]}, "registered as 'openagents-network'"),
                          ({"nodes": [{"id": "p", "kind": "pool", "replicas": []}]}, "at least one replica"),
                          ({"plans": {"*": ["nobody"]}}, "plans:"), ({"pricing": [{"model": "m"}]}, "pricing:"),
                          ({"keys": good["keys"][:1] * 2}, "twice")):
        with pytest.raises(gs.ConfigError, match=needle.replace("[", r"\[").replace("]", r"\]").replace("*", r"\*")):
            gs.build_gateway({**good, **patch})
    path = tmp_path / "gw.json"
    path.write_text(json.dumps(good))
    out = subprocess.run([sys.executable, "-m", "openagents_b200.gateway.server", "--config", str(path), "--check"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0 and json.loads(out.stdout) == {"ok": True, "adapters": ["hydralisk", "openagents-network"], "keys": 3}
    path.write_text(json.dumps({**good, "nodes": []}))
    out = subprocess.run([sys.executable, "-m", "openagents_b200.gateway.server", "--config", str(path), "--check"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 2 and "at least one node" in out.stderr


def test_pool_of_openai_speaking_replicas(stack):
    """A pool node: two replicas of the same model server behind one adapter id; the session header pins a conversation to the
    replica that served it."""
    node_url, good = stack[3], stack[4]
    cfg = {**good, "nodes": [{"id": "hydralisk-pool", "kind": "pool", "replicas": [
        {"replicaId": "r0", "endpoint": node_url + "/v1", "bearer": "node-secret", "maxInflight": 2},
        {"replicaId": "r1", "endpoint": node_url + "/v1", "bearer": "node-secret", "maxInflight": 2}]}], "plans": {"*": ["hydralisk-pool"]}}
    gw = gs.build_gateway(cfg)
    httpd = gs.serve(gw, "127.0.0.1", 0)
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    try:
        base = f"http://127.0.0.1:{httpd.server_address[1]}"
        routes = []
        for _ in range(3):
            code, raw, _h = _call(base + "/v1/chat/completions", BODY, key="sk-a", headers={"x-openagents-session": "conv-1"})
            assert code == 200, raw
            routes.append(gw.registry.get("hydralisk-pool").last_route["replicaId"])
        assert len(set(routes)) == 1 and json.loads(raw)["openagents"]["route"] == "hydralisk-pool"
    finally:
        httpd.shutdown()
