"""Serve benchmark client and preflight against the in-tree server with a scripted backend (CPU)."""
import json
import os
import threading

import pytest

from openagents_b200.serve import bench_client as bc
from openagents_b200.serve.generation import ByteTokenizer
from openagents_b200.serve.server import ServedModel, ServerState, serve
from tests.test_tools import _Scripted


@pytest.fixture()
def endpoint():
    state = ServerState([ServedModel("scripted", _Scripted("muse-ready OK"), None, tokenizer=ByteTokenizer(512), max_num_seqs=2)])
    httpd = serve(state, "127.0.0.1", 0)
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    yield f"http://127.0.0.1:{httpd.server_address[1]}/v1"
    httpd.shutdown()


def test_stream_fold_times_first_token_and_content():
    ticks = iter([1.0, 2.0, 3.0])            # first reasoning token, first content token, end
    lines = ['data: {"choices":[{"delta":{"role":"assistant"}}]}', 'data: {"choices":[{"delta":{"reasoning_content":"hm"}}]}',
             b'data: {"choices":[{"delta":{"content":"muse"}}]}', 'data: {"choices":[{"delta":{"content":"-ready"},"finish_reason":"stop"}]}',
             'data: {"choices":[],"usage":{"completion_tokens":4},"timings":{"predicted_per_second":99.0}}', "data: [DONE]", "data: ignored"]
    r = bc.consume_stream(lines, started=0.5, clock=lambda: next(ticks))
    assert r["ttft_seconds"] == 0.5 and r["first_content_seconds"] == 1.5 and r["total_seconds"] == 2.5
    assert r["visible_output"] == "muse-ready" and r["reasoning_output"] == "hm" and r["finish_reason"] == "stop" and r["event_count"] == 5
    assert r["observed_completion_per_second"] == 2.0 and r["timings"]["predicted_per_second"] == 99.0


def test_benchmark_document_against_live_server(endpoint):
    doc = bc.run_benchmark(endpoint, "local", "scripted", "test", repetitions=2, only=["exact_instruction", "multi_turn_memory"], max_tokens=10,
                           server_pid=os.getpid())
    assert doc["schema"] == bc.BENCH_SCHEMA and len(doc["results"]) == 4
    r = doc["results"][0]
    assert r["http_status"] == 200 and r["ttft_seconds"] is not None and r["expected_observed"] and r["request"]["temperature"] == 0
    assert doc["summary"]["exact_instruction"] == {"ok": 2, "ttft_seconds_median": pytest.approx(doc["summary"]["exact_instruction"]["ttft_seconds_median"]),
                                                    "decode_tok_s_median": doc["summary"]["exact_instruction"]["decode_tok_s_median"], "expected_observed": 2}
    assert doc["summary"]["multi_turn_memory"]["expected_observed"] == 0        # the scripted answer lacks the codename
    assert doc["memory"]["samples"] >= 0
    assert [s["name"] for s in bc.scenarios()] == ["exact_instruction", "code_generation", "reasoning", "long_context_retrieval", "multi_turn_memory", "structured_json"]
    assert "Entry 0731: " in bc.long_context() and bc.long_context().count("LANTERN-4821") == 1
    assert bc.process_tree_rss_kib(os.getpid()) > 1000


def test_benchmark_records_connection_failure():
    r = bc.streamed_chat("http://127.0.0.1:9/v1", "k", "m", bc.scenarios()[0], 1)
    assert r["http_status"] is None and r["error"] and r["ttft_seconds"] is None and not r["expected_observed"]


def test_preflight_is_owner_gated_and_redacts(endpoint):
    with pytest.raises(PermissionError):
        bc.run_preflight(env={})
    with pytest.raises(PermissionError):
        bc.run_preflight(env={"B200_SERVING_BENCH": "1", "B200_SERVING_ENDPOINT": endpoint + "/chat/completions"})
    env = {"B200_SERVING_BENCH": "1", "B200_SERVING_ENDPOINT": endpoint + "/chat/completions", "B200_SERVING_OWNER_APPROVAL_REF": "approval.owner.1",
           "B200_SERVING_MODEL_REF": "scripted", "B200_SERVING_MAX_NEW_TOKENS": "13", "B200_SERVING_EXPECTED_OUTPUT": "muse-ready OK",
           "B200_SERVING_API_KEY": "secret-key-123"}
    ev = bc.run_preflight(env=env)
    assert ev["ready"] and ev["blockerRefs"] == [] and ev["servingReceipt"]["verification"] == {
        "parityPassed": True, "canaryRef": "canary.pylon.serving.known_answer.ok.v1", "canaryPassed": True, "replayMatched": True}
    text = json.dumps(ev)
    assert "127.0.0.1" not in text and "secret-key-123" not in text and "muse-ready" not in text and "Respond with" not in text
    ev = bc.run_preflight(env=dict(env, B200_SERVING_EXPECTED_OUTPUT="something else"))
    assert not ev["ready"] and "blocker.serving.canary_failed" in ev["blockerRefs"] and ev["servingReceipt"]["verification"]["replayMatched"]
