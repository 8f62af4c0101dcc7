"""Tool calling: choice normalisation, parsing, stream splitting, delta assembly, the tool loop, and the server route
with a backend whose "model" emits a scripted answer."""
import json
import threading
import urllib.request

import pytest
import torch

from openagents_b200.serve import tools as tl
from openagents_b200.serve.backend import Backend
from openagents_b200.serve.server import ServedModel, ServerState, serve

TOOLS = [{"type": "function", "function": {"name": "add", "parameters": {"type": "object", "properties": {"a": {"type": "number"}, "b": {"type": "number"}}}}},
         {"type": "function", "function": {"name": "now", "parameters": {"type": "object", "properties": {}}}}]


def test_choice_and_prompt():
    assert tl.normalize_tool_choice(None, TOOLS) == ("auto", None) and tl.normalize_tool_choice(None, []) == ("none", None)
    assert tl.normalize_tool_choice("required", TOOLS) == ("required", None)
    assert tl.normalize_tool_choice({"type": "function", "function": {"name": "add"}}, TOOLS) == ("named", "add")
    for bad in ("sometimes", {"type": "function", "function": {"name": "nope"}}):
        with pytest.raises(tl.ToolCallError):
            tl.normalize_tool_choice(bad, TOOLS)
    with pytest.raises(tl.ToolCallError):
        tl.normalize_tool_choice("required", [])
    m = tl.render_tools_system_message(TOOLS, "auto", None)
    assert m["content"] == tl.render_tools_system_message(list(reversed(TOOLS)), "auto", None)["content"]      # order-independent bytes
    assert tl.render_tools_system_message(TOOLS, "none", None) is None and "must call the tool add" in tl.render_tools_system_message(TOOLS, "named", "add")["content"]


def test_parse_and_finish():
    text = 'Let me compute. <tool_call>{"name": "add", "arguments": {"a": 1, "b": 2}}</tool_call> and <tool_call>{"name":"now","arguments":{}}</tool_call> <tool_call>{"name": "rm", "arguments": {}}</tool_call> <tool_call>{broken</tool_call>'
    content, calls = tl.parse_tool_calls(text, TOOLS)
    assert [c["function"]["name"] for c in calls] == ["add", "now"] and json.loads(calls[0]["function"]["arguments"]) == {"a": 1, "b": 2}
    assert "rm" in content and "broken" in content and calls[0]["id"] != calls[1]["id"]
    msg, fin = tl.finish_with_tools(text, TOOLS, "auto", None)
    assert fin == "tool_calls" and len(msg["tool_calls"]) == 2
    msg, fin = tl.finish_with_tools(text, TOOLS, "named", "now")
    assert [c["function"]["name"] for c in msg["tool_calls"]] == ["now"]
    assert tl.finish_with_tools("plain", TOOLS, "auto", None) == ({"role": "assistant", "content": "plain"}, "stop")
    assert tl.finish_with_tools(text, TOOLS, "none", None)[0]["content"] == text
    with pytest.raises(tl.ToolCallError) as e:
        tl.finish_with_tools("plain", TOOLS, "required", None)
    assert e.value.kind == "tool_call_required"


def test_stream_splitter_and_assembler():
    text = 'ok <tool_call>{"name": "add", "arguments": {"a": 1, "b": 2}}</tool_call> then <tool_call>{"name":"now","arguments":{}}</tool_call> done <to'
    sp, asm, deltas = tl.ToolCallStreamSplitter(TOOLS), tl.ToolCallDeltaAssembler(), []
    for i in range(0, len(text), 3):
        deltas += sp.feed(text[i:i + 3])
    deltas += sp.flush()
    for d in deltas:
        asm.feed(d)
        assert "<tool_call>" not in d.get("content", "")
    calls = asm.result()
    assert [c["function"]["name"] for c in calls] == ["add", "now"] and json.loads(calls[0]["function"]["arguments"]) == {"a": 1, "b": 2}
    assert asm.content == "ok  then  done <to" and sp.n_calls == 2 and all(c["id"] for c in calls)
    chunks = tl.parse_sse([b'data: {"choices": [{"delta": {"content": "a"}}]}\n', b": ping\n", "data: [DONE]\n", 'data: {"x": 1}\n'])
    assert chunks == [{"choices": [{"delta": {"content": "a"}}]}]


def test_request_lowering_and_tool_loop():
    req = tl.LlmRequest("m", [{"role": "user", "content": "1+2?"}], system="be exact", tools=[TOOLS[0]["function"]], tool_choice={"name": "add"},
                        options=tl.GenerationOptions(max_tokens=32, temperature=0.0, stop=("\n\n",)))
    body = req.to_openai()
    assert body["messages"][0] == {"role": "system", "content": "be exact"} and body["tool_choice"] == {"type": "function", "function": {"name": "add"}}
    assert body["tools"][0]["type"] == "function" and body["max_tokens"] == 32 and body["stop"] == ["\n\n"] and "top_p" not in body
    script = iter([
        {"choices": [{"message": {"role": "assistant", "content": None, "tool_calls": [
            {"id": "c1", "type": "function", "function": {"name": "add", "arguments": '{"a": 1, "b": 2}'}},
            {"id": "c2", "type": "function", "function": {"name": "boom", "arguments": "{}"}}]}}]},
        {"choices": [{"message": {"role": "assistant", "content": "3"}}]}])
    seen = []

    def complete(b):
        seen.append(b)
        return next(script)

    out = tl.run_tool_loop(complete, req, {"add": lambda a, b: {"sum": a + b}})
    assert out["message"]["content"] == "3" and out["steps"] == 2
    tool_msgs = [m for m in out["transcript"] if m.get("role") == "tool"]
    assert json.loads(tool_msgs[0]["content"]) == {"sum": 3} and "unknown tool" in tool_msgs[1]["content"]
    assert seen[1]["tool_choice"] == "auto"                     # a forced call is not forced again
    with pytest.raises(tl.ToolCallError):
        tl.run_tool_loop(lambda b: {"choices": [{"message": {"role": "assistant", "tool_calls": [{"id": "x", "type": "function", "function": {"name": "add", "arguments": "{}"}}]}}]},
                         req, {"add": lambda **k: 1}, max_steps=2)


class _Scripted(Backend):
    """A backend whose next-token logits spell out a fixed answer (byte tokenizer)."""
    vocab = 512

    def __init__(self, answer: str):
        self.ids = list(answer.encode()) + [0]
        self.pos = {}

    def begin(self, seq_id, prompt):
        self.pos[seq_id] = 0
        return 0

    def forward(self, seq_ids, new_tokens):
        out = torch.full((len(seq_ids), self.vocab), -10.0)
        for r, s in enumerate(seq_ids):
            if self.pos[s] > 0 or True:
                out[r, self.ids[min(self.pos[s], len(self.ids) - 1)]] = 10.0
            self.pos[s] += 1
        return out

    def end(self, seq_id):
        self.pos.pop(seq_id, None)

    def kv_stats(self):
        return {"pages_total": 0, "pages_free": 0, "prefix_hits": 0, "prefix_lookups": 0}

    def topology(self):
        return {"kind": "replicated", "stages": [{"nodeRef": "n", "layerStart": 0, "layerEnd": 1, "role": "stage"}]}


def _post(url, body):
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    try:
        with urllib.request.urlopen(req, timeout=60) as r:
            return r.status, r.read().decode()
    except urllib.error.HTTPError as e:
        return e.code, e.read().decode()


def test_server_tool_calls_non_stream_and_stream():
    answer = 'Sure. <tool_call>{"name": "add", "arguments": {"a": 2, "b": 5}}</tool_call>'
    from openagents_b200.serve.generation import ByteTokenizer
    state = ServerState([ServedModel("scripted", _Scripted(answer), None, tokenizer=ByteTokenizer(512), max_num_seqs=2)])
    httpd = serve(state, "127.0.0.1", 0)
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    url = f"http://127.0.0.1:{httpd.server_address[1]}/v1/chat/completions"
    try:
        body = {"model": "scripted", "messages": [{"role": "user", "content": "2+5"}], "tools": TOOLS, "max_tokens": len(answer.encode())}
        status, text = _post(url, body)
        out = json.loads(text)
        assert status == 200 and out["choices"][0]["finish_reason"] == "tool_calls"
        call = out["choices"][0]["message"]["tool_calls"][0]
        assert call["function"]["name"] == "add" and json.loads(call["function"]["arguments"]) == {"a": 2, "b": 5} and out["choices"][0]["message"]["content"] == "Sure."
        status, text = _post(url, dict(body, stream=True))
        chunks = tl.parse_sse(text.splitlines())
        asm = tl.ToolCallDeltaAssembler()
        for c in chunks:
            asm.feed(c["choices"][0]["delta"])
        assert asm.result()[0]["function"]["name"] == "add" and chunks[-1]["choices"][0]["finish_reason"] == "tool_calls" and "<tool_call>" not in asm.content
        assert _post(url, dict(body, tool_choice={"type": "function", "function": {"name": "now"}}))[0] == 422     # named call not produced
        assert _post(url, dict(body, tool_choice="sometimes"))[0] == 400
        status, text = _post(url, dict(body, tool_choice="none"))
        assert json.loads(text)["choices"][0]["message"]["content"] == answer
    finally:
        httpd.shutdown()


def test_attach_client_doctor_smoke_and_tool_loop_against_a_live_server(tmp_path, capsys):
    """The local attach path: base-URL resolution, the health and model-row contract, a smoke completion, and a completion with a
    tool loop whose records carry digests and lengths only."""
    import threading
    from openagents_b200.models.config import TINY_LLAMA
    from openagents_b200.models.weights import PLAN_Q8_0, random_weights, save_gguf
    from openagents_b200.receipts import manifests as mf
    from openagents_b200.serve import attach_client as ac
    from openagents_b200.serve.backend import CpuBackend
    from openagents_b200.serve.server import ServedModel, ServerState, serve
    assert ac.resolve_base_url("http://a/v1/", {}) == "http://a/v1"
    assert ac.resolve_base_url(None, {"PROBE_PSIONIC_BASE_URL": "http://c/v1", "PYLON_PSIONIC_BASE_URL": "http://b/v1"}) == "http://b/v1"
    assert ac.resolve_base_url(None, {"PROBE_PSIONIC_BASE_URL": "http://c/v1"}) == "http://c/v1" and ac.resolve_base_url(None, {}) == ac.DEFAULT_BASE_URL
    assert ac.admit_model_row({"id": "m", "artifact_digest": "sha256:" + "a" * 64})["admitted"]
    assert ac.admit_model_row({"id": "m", "manifest_ref": "manifest.models.m.v1"})["admitted"]
    assert not ac.admit_model_row({"id": "m", "artifact_digest": "md5:abc", "manifest_ref": "/home/me/m.json"})["admitted"]
    cfg = TINY_LLAMA.with_(vocab=512, d_model=64, n_heads=2, n_kv_heads=1, head_dim=32, ffn=128)
    p = str(tmp_path / "tiny.gguf")
    save_gguf(p, cfg, random_weights(cfg, 0), PLAN_Q8_0)
    httpd = serve(ServerState([ServedModel("tiny", CpuBackend.from_gguf(p), mf.artifact_digest(p), max_num_seqs=4)]), "127.0.0.1", 0)
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    try:
        base = f"http://127.0.0.1:{httpd.server_address[1]}/v1"
        c = ac.AttachClient(base)
        d = c.doctor()
        assert d["ok"] and d["executionEngine"] == "b200" and d["models"][0]["admitted"] and d["models"][0]["artifactDigest"].startswith("sha256:")
        s = c.smoke()
        assert s["ok"] and s["model"] == "tiny" and 1 <= s["usage"]["completion_tokens"] <= 4
        assert ac.main(["doctor", "--base-url", base]) == 0 and json.loads(capsys.readouterr().out)["ok"]
        LlmRequest, GenerationOptions = tl.LlmRequest, tl.GenerationOptions
        req = LlmRequest("tiny", [{"role": "user", "content": "secret question 12345"}], options=GenerationOptions(max_tokens=6, temperature=0))
        out = c.complete(req)
        assert out["steps"] == 1 and out["usage"]["completion_tokens"] >= 1
        text = json.dumps({k: out[k] for k in ("redactedTranscript", "toolCallReceipts")})
        assert "secret question" not in text and out["redactedTranscript"][0] == {"role": "user", "contentChars": 21, "contentDigest": out["redactedTranscript"][0]["contentDigest"], "toolCalls": 0}
        streamed = c.complete(req, stream=True)
        assert streamed["message"]["content"] == out["message"]["content"]          # greedy: the streamed answer is the same
    finally:
        httpd.shutdown()
    down = ac.AttachClient("http://127.0.0.1:1/v1", timeout_s=2).doctor()
    assert not down["ok"] and down["blockerRefs"] == ["blocker.attach.server_unreachable"]
    # a tool loop against a scripted server: receipts carry digests, a failing tool is marked
    script = [{"choices": [{"message": {"role": "assistant", "content": None, "tool_calls": [
                  {"id": "c1", "type": "function", "function": {"name": "add", "arguments": '{"a": 2, "b": 3}'}},
                  {"id": "c2", "type": "function", "function": {"name": "boom", "arguments": "{}"}}]}}], "usage": {"prompt_tokens": 5, "completion_tokens": 7}},
              {"choices": [{"message": {"role": "assistant", "content": "five"}}], "usage": {"prompt_tokens": 9, "completion_tokens": 1}}]
    fake = ac.AttachClient("http://unused/v1")
    fake._complete_once = lambda body, stream: script.pop(0)
    r = fake.complete(LlmRequest("m", [{"role": "user", "content": "2+3?"}], tools=[{"name": "add", "parameters": {}}]), {"add": lambda a, b: a + b, "boom": lambda: 1 / 0})
    assert r["message"]["content"] == "five" and r["steps"] == 2 and r["usage"] == {"prompt_tokens": 14, "completion_tokens": 8, "total_tokens": 22}
    rec = {x["tool"]: x for x in r["toolCallReceipts"]}
    assert rec["add"]["resultDigest"].startswith("sha256:") and rec["add"]["failed"] is False and rec["boom"]["failed"] is True
    assert '"b": 3' not in json.dumps(r["toolCallReceipts"]).replace("\\", "")


def test_command_line_input_errors_are_one_line_and_status_2(tmp_path):
    """A missing or malformed input ends a command with ``<prog>: error: ...`` on stderr and status 2, not a traceback."""
    import subprocess
    import sys
    bad = tmp_path / "bad.gguf"
    bad.write_bytes(b"GGUF\x03\x00\x00\x00")
    cases = [(["openagents_b200.gguf", "inspect", str(bad)], "b200-gguf: error:", "too small"),
             (["openagents_b200.gguf", "digest", str(tmp_path / "none.gguf")], "b200-gguf: error:", "No such file"),
             (["openagents_b200.data", "prepare", "--text", str(tmp_path / "none.txt"), "--out", str(tmp_path / "o")], "b200-data: error:", "No such file"),
             (["openagents_b200.serve.server", "-m", str(bad), "--backend", "cpu"], "b200-serve: error:", "too small")]
    for argv, head, needle in cases:
        out = subprocess.run([sys.executable, "-m", *argv], capture_output=True, text=True, timeout=300)
        assert out.returncode == 2 and out.stderr.strip().startswith(head) and needle in out.stderr and "Traceback" not in out.stderr, (argv, out.stderr)
    out = subprocess.run([sys.executable, "-m", "openagents_b200.gguf", "inspect", str(bad)], capture_output=True, text=True, timeout=300,
                         env={**__import__("os").environ, "B200_TRACEBACK": "1"})
    assert out.returncode == 1 and "Traceback" in out.stderr
