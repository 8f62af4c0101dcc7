"""The OpenAI-compatible host adapter and the replica pool, against this package's own HTTP server and against fakes."""
import io
import json
import threading
import urllib.error

import pytest

from openagents_b200.gateway import fabric as fb
from openagents_b200.gateway import hydralisk as hy
from openagents_b200.gateway import prompt_cache as pc
from openagents_b200.models.config import TINY_LLAMA
from openagents_b200.models.weights import PLAN_Q8_0, random_weights, save_gguf
from openagents_b200.receipts import manifests as mf
from openagents_b200.serve.backend import CpuBackend
from openagents_b200.serve.server import ServedModel, ServerState, serve


@pytest.fixture(scope="module")
def base_url(tmp_path_factory):
    cfg = TINY_LLAMA.with_(vocab=512, d_model=64, n_heads=2, n_kv_heads=1, head_dim=32, ffn=128)
    p = str(tmp_path_factory.mktemp("m") / "tiny.gguf")
    save_gguf(p, cfg, random_weights(cfg, 0), PLAN_Q8_0)
    state = ServerState([ServedModel("tiny", CpuBackend.from_gguf(p), mf.artifact_digest(p), max_num_seqs=4)])
    httpd = serve(state, "127.0.0.1", 0)
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    yield f"http://127.0.0.1:{httpd.server_address[1]}/v1"
    httpd.shutdown()


def _req(stream=False, **pp):
    return fb.InferenceRequest("tiny", ({"role": "user", "content": "hello there"},), stream, {"max_tokens": 6, "temperature": 0, **pp})


def test_complete_and_stream_against_the_real_server(base_url):
    a = hy.HydraliskAdapter("hydralisk-vllm", "secret", base_url)
    r = a.complete(_req())
    assert r.usage.completion_tokens == 6 and r.usage.total_tokens == r.usage.prompt_tokens + 6 and r.served_model == "tiny"
    items = list(a.stream(_req(True)))
    assert items[-1][0] == "done" and all(k == "delta" for k, _ in items[:-1]) and len(items) > 1
    done = items[-1][1]
    assert done.content == "".join(t for k, t in items[:-1]) == r.content           # greedy: the stream is the same answer
    assert done.usage == r.usage
    with pytest.raises(fb.InferenceAdapterError) as e:
        a.complete(fb.InferenceRequest("nope", ({"role": "user", "content": "x"},), False, {}))
    assert e.value.http_status == 404 and not e.value.retryable


class _Resp(io.BytesIO):
    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


def _fake(answer=None, status=None, exc=None, calls=None):
    def opener(req, timeout=None):
        if calls is not None:
            calls.append(json.loads(req.data))
        if exc:
            raise exc
        if status:
            raise urllib.error.HTTPError(req.full_url, status, "x", {}, None)
        return _Resp(json.dumps(answer).encode())
    return opener


OK = {"model": "up", "choices": [{"message": {"role": "assistant", "content": "hi"}, "finish_reason": "stop"}],
      "usage": {"prompt_tokens": 3, "completion_tokens": 1, "total_tokens": 4, "prompt_tokens_details": {"cached_tokens": 2}}}


def test_receipt_first_rules_and_error_classes():
    calls = []
    a = hy.HydraliskAdapter("h", "k", "http://x/v1/", _fake(OK, calls=calls), upstream_model="openai/gpt-oss-20b")
    r = a.complete(_req(user="u1", not_forwarded=1))
    assert r.usage.cached_prompt_tokens == 2 and calls[0]["model"] == "openai/gpt-oss-20b" and "not_forwarded" not in calls[0] and calls[0]["user"] == "u1"
    no_usage = {k: v for k, v in OK.items() if k != "usage"}
    with pytest.raises(fb.InferenceAdapterError) as e:
        hy.HydraliskAdapter("h", "k", "http://x/v1", _fake(no_usage)).complete(_req())
    assert e.value.kind == "usage_missing" and not e.value.retryable
    for status, kind, retry in ((429, "rate_limited", True), (503, "service_overloaded", True), (500, "upstream_error", True), (400, "request_rejected", False)):
        with pytest.raises(fb.InferenceAdapterError) as e:
            hy.HydraliskAdapter("h", "k", "http://x/v1", _fake(status=status)).complete(_req())
        assert (e.value.kind, e.value.retryable) == (kind, retry)
    with pytest.raises(fb.InferenceAdapterError) as e:
        hy.HydraliskAdapter("h", "k", "http://x/v1", _fake(exc=OSError("refused"))).complete(_req())
    assert e.value.kind == "transport_error" and e.value.retryable
    with pytest.raises(fb.InferenceAdapterError) as e:
        hy.HydraliskAdapter("h", "k", "http://x/v1", _fake({"choices": []})).complete(_req())
    assert e.value.kind == "malformed_response"


def _pool(openers, **kw):
    reps = [{"replicaId": f"r{i}", "adapter": hy.HydraliskAdapter(f"r{i}", "k", "http://x/v1", op), "maxInflight": 1} for i, op in enumerate(openers)]
    t = [1000]

    def now():
        t[0] += 10
        return t[0]
    return hy.HydraliskPoolAdapter("hydralisk-vllm", reps, now_ms=now, **kw)


def test_pool_affinity_health_and_saturation():
    c0, c1 = [], []
    pool = _pool([_fake(OK, calls=c0), _fake(OK, calls=c1)])
    aff = pc.session_affinity_params("cacheaff:abc")
    pool.complete(_req(**aff))
    first = pool.last_route["replicaId"]
    assert first == "r0" and pool.live["r0"]["warm"] == "warm" and pool.live["r0"]["ttft"] is not None
    pool.complete(_req(**aff))
    assert pool.last_route["replicaId"] == "r0" and pool.last_route["affinityHit"] is True       # the session sticks to its replica
    pool.complete(_req())                                                                           # no hint: the warm replica ranks first
    assert pool.last_route["replicaId"] == "r0" and len(c0) == 3 and len(c1) == 0
    # a failing replica degrades, then leaves rotation; the error names the replica but carries the pool's adapter id
    bad = _pool([_fake(status=500), _fake(OK)])
    with pytest.raises(fb.InferenceAdapterError) as e:
        bad.complete(_req())
    assert e.value.adapter_id == "hydralisk-vllm" and "r0" in e.value.reason and bad.live["r0"]["health"] == "degraded"
    bad.complete(_req())
    assert bad.last_route["replicaId"] == "r1"                                   # the healthy replica now ranks first
    alone = _pool([_fake(status=500)], sleep=lambda ms: None)
    for want in ("degraded", "unhealthy"):
        with pytest.raises(fb.InferenceAdapterError):
            alone.complete(_req())
        assert alone.live["r0"]["health"] == want
    with pytest.raises(fb.InferenceAdapterError) as e:
        alone.complete(_req())
    assert e.value.kind == "glm_pool_saturated"                                  # out of rotation: nothing is sent any more
    # outside telemetry can take a replica out (oracle), and the admission snapshot follows
    ext = _pool([_fake(OK), _fake(OK)], routing_state_oracle=lambda rid: {"health": "unhealthy"} if rid == "r0" else None)
    ext.complete(_req())
    assert ext.last_route["replicaId"] == "r1"
    assert ext.route_admission() == {"reservedExternalHeadroomAvailable": True, "internalStressHeadroomAvailable": False, "reason": "external_reserve_only"}
    # saturation: everything unhealthy -> non-stream waits once then fails retryably (503); queue_then_429 ends with a 429
    slept = []
    sat = _pool([_fake(OK)], routing_state_oracle=lambda rid: {"health": "unhealthy"}, sleep=slept.append)
    with pytest.raises(fb.InferenceAdapterError) as e:
        sat.complete(_req())
    assert e.value.kind == "glm_pool_saturated" and e.value.retryable and slept == [250]
    sat.saturation_policy = "queue_then_429"
    with pytest.raises(fb.InferenceAdapterError) as e:
        sat.complete(_req())
    assert e.value.http_status == 429 and not e.value.retryable
    with pytest.raises(fb.InferenceAdapterError):
        sat.complete(_req(stream=True))                    # streams overflow at once by default


def test_pool_plugs_into_the_registry_and_router(base_url):
    from openagents_b200.gateway import router as rt
    pool = hy.HydraliskPoolAdapter(rt.HYDRALISK if hasattr(rt, "HYDRALISK") else "hydralisk-vllm",
                                   [{"replicaId": "a", "adapter": hy.HydraliskAdapter("a", "k", base_url), "maxInflight": 2}])
    reg = fb.ProviderRegistry()
    reg.register(pool)
    d = rt.dispatch_with_overflow(_req(), lambda a, r: a.complete(r), reg, plan=[pool.id])
    assert d.adapter_id == pool.id and d.value.usage.completion_tokens == 6
