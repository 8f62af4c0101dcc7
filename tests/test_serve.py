"""Model server on the CPU backend: real HTTP round trips against a tiny GGUF model, the serve wire
contract with its parity gate, sessions and ``previous_response_id``, the scheduler, the node CLI
and the receipts (CPU)."""
import json
import subprocess
import threading
import urllib.error
import urllib.request

import pytest
import torch

from openagents_b200.models.config import TINY_LLAMA
from openagents_b200.models.weights import PLAN_Q8_0, random_weights, save_gguf
from openagents_b200.receipts import manifests as mf
from openagents_b200.serve.backend import CpuBackend
from openagents_b200.serve.generation import ByteTokenizer, SamplingParams, Scheduler
from openagents_b200.serve.server import ServedModel, ServerState, serve


@pytest.fixture(scope="module")
def gguf_path(tmp_path_factory):
    cfg = TINY_LLAMA.with_(vocab=512, d_model=64, n_heads=2, n_kv_heads=1, head_dim=32, ffn=128)
    p = str(tmp_path_factory.mktemp("m") / "tiny.gguf")
    save_gguf(p, cfg, random_weights(cfg, 0), PLAN_Q8_0)
    return p


@pytest.fixture(scope="module")
def server(gguf_path):
    model = ServedModel("tiny", CpuBackend.from_gguf(gguf_path), mf.artifact_digest(gguf_path), max_num_seqs=4)
    state = ServerState([model])
    httpd = serve(state, "127.0.0.1", 0)
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    yield f"http://127.0.0.1:{httpd.server_address[1]}", state
    httpd.shutdown()


def _get(url):
    with urllib.request.urlopen(url, timeout=60) as r:
        return r.status, r.read()


def _post(url, obj):
    req = urllib.request.Request(url, data=json.dumps(obj).encode(), headers={"Content-Type": "application/json"})
    try:
        with urllib.request.urlopen(req, timeout=120) as r:
            return r.status, r.read()
    except urllib.error.HTTPError as e:
        return e.code, e.read()


def test_health_models_status_metrics(server):
    base, _ = server
    code, body = _get(base + "/health")
    h = json.loads(body)
    assert code == 200 and h["execution_engine"] == "b200" and "/v1/chat/completions" in h["endpoints"]
    m = json.loads(_get(base + "/v1/models")[1])["data"][0]
    assert m["id"] == "tiny" and m["artifact_digest"].startswith("sha256:") and m["chat_template_digest"].startswith("sha256:")
    st = json.loads(_get(base + "/psionic/management/status")[1])
    assert st["models"][0]["backend"] == "cpu" and st["models"][0]["topology"]["stages"][0]["layerEnd"] == 2
    assert b"b200_requests_total" in _get(base + "/metrics")[1]


def test_chat_completion_and_stream_agree(server):
    base, _ = server
    body = {"model": "tiny", "messages": [{"role": "user", "content": "hello"}], "max_tokens": 12, "temperature": 0}
    code, raw = _post(base + "/v1/chat/completions", body)
    r = json.loads(raw)
    assert code == 200 and r["choices"][0]["finish_reason"] in ("length", "stop")
    assert r["usage"]["completion_tokens"] <= 12 and r["usage"]["total_tokens"] == r["usage"]["prompt_tokens"] + r["usage"]["completion_tokens"]
    code, raw = _post(base + "/v1/chat/completions", {**body, "stream": True})
    events = [l[6:] for l in raw.decode().split("\n") if l.startswith("data: ")]
    assert events[-1] == "[DONE]"
    text = "".join(json.loads(e)["choices"][0]["delta"].get("content", "") for e in events[:-1])
    assert text == r["choices"][0]["message"]["content"]
    assert _post(base + "/v1/chat/completions", {"model": "nope", "messages": [{"role": "user", "content": "x"}]})[0] == 404
    assert _post(base + "/v1/chat/completions", {"messages": []})[0] == 400


def test_serve_contract_parity_and_receipt(server):
    base, _ = server
    code, raw = _post(base + "/v1/serve", {"model": "tiny", "messages": [{"role": "user", "content": "abc"}],
                                           "passthroughParams": {"max_tokens": 8}, "requireExactGreedyParity": True})
    s = json.loads(raw)
    assert code == 200 and s["parityMode"] == "exact_greedy_parity" and s["parityVerified"] is True
    assert len(s["stages"]) == 1 and s["usage"]["totalTokens"] == s["usage"]["promptTokens"] + s["usage"]["completionTokens"]
    rec = mf.serving_receipt(s)
    assert rec["sharded"] is False and not mf.clears_paid_traffic(rec)        # no paid-traffic bundle: not cleared
    rec["paidTrafficVerification"] = {"parityPassed": True, "canaryPassed": True, "replayPassed": True, "payoutEligible": True, "blockerRefs": []}
    assert mf.clears_paid_traffic(rec)


def test_responses_with_previous_response_id_reuses_the_sequence(server):
    base, state = server
    code, raw = _post(base + "/v1/responses", {"model": "tiny", "input": "first turn", "max_output_tokens": 6})
    r1 = json.loads(raw)
    assert code == 200 and r1["status"] == "completed"
    code, raw = _post(base + "/v1/responses", {"model": "tiny", "input": "second", "previous_response_id": r1["id"], "max_output_tokens": 6})
    r2 = json.loads(raw)
    assert code == 200 and r2["previous_response_id"] == r1["id"]
    sess = state.sessions[state.responses[r2["id"]][0]]
    assert len(sess.responses) == 2
    # the second turn ran only its own tokens: the cache already held the first turn
    kv_tokens = state.default.backend.caches[sess.seq_id].length
    assert kv_tokens == len(sess.tokens)
    assert _post(base + "/v1/responses", {"input": "x", "previous_response_id": "resp-missing"})[0] == 404


def test_continuous_batching_matches_sequential(gguf_path):
    be = CpuBackend.from_gguf(gguf_path)
    tok = ByteTokenizer(be.cfg.vocab)
    prompts = [tok.encode(t) for t in ("alpha", "a much longer prompt than the others", "b")]
    solo = []
    for p in prompts:
        s = Scheduler(be, tok, max_num_seqs=1)
        r = s.submit(p, SamplingParams(max_tokens=6))
        s.run_until_done([r])
        solo.append(r.output)
    s = Scheduler(be, tok, max_num_seqs=3, prefill_chunk=8)          # chunked prefill + batched decode
    reqs = [s.submit(p, SamplingParams(max_tokens=6)) for p in prompts]
    s.run_until_done(reqs)
    assert [r.output for r in reqs] == solo
    assert s.stats["steps"] > 0 and s.stats["batch_size_sum"] / s.stats["steps"] > 1.0
    assert not be.caches                                              # finished sequences released their KV


def test_node_cli_against_reference_fixture(tmp_path):
    from openagents_b200 import _build
    _build.build_node()
    cli = str(_build.node_cli_path())
    import os
    # the reference's own fixture when its tree is at hand (OPENAGENTS_REFERENCE_DIR), else the same shape written here
    fx = os.path.join(os.environ.get("OPENAGENTS_REFERENCE_DIR", "/nonexistent"), "fixtures/cloud/psionic_worker_attachment_v1/mixed-readiness.json")
    if not os.path.exists(fx):
        fx = str(tmp_path / "fx.json")
        json.dump({"schema_version": "openagents.psionic_worker_attachment.v1", "updated_at_ms": 1, "workers": [
            {"product_id": "psionic.managed.inference", "worker_id": "w.i", "worker_kind": "inference", "ready": True, "crashed": False,
             "evidence_digest": "sha256:a", "detail": None},
            {"product_id": "psionic.managed.training", "worker_id": "w.t", "worker_kind": "training", "ready": False, "crashed": True,
             "evidence_digest": "sha256:b", "detail": None},
            {"product_id": "psionic.managed.sandbox", "worker_id": "w.s", "worker_kind": "sandbox", "ready": False, "crashed": False,
             "evidence_digest": "sha256:c", "detail": None}]}, open(fx, "w"))
    d = str(tmp_path)
    assert subprocess.run([cli, "psionic", "attach", "--file", fx, "--state-dir", d], capture_output=True).returncode == 0
    st = json.loads(subprocess.run([cli, "status", "--json", "--state-dir", d], capture_output=True, text=True).stdout)
    assert st["capabilities"]["inference_products"] == ["psionic.managed.inference"]
    assert st["capabilities"]["training_products"] == [] and st["capabilities"]["sandbox_profiles"] == []   # crashed / not ready
    r = subprocess.run([cli, "psionic", "receipt", "append", "--state-dir", d, "--assignment-id", "asg.1", "--product-id",
                        "psionic.managed.inference", "--worker-id", "w.i", "--status", "succeeded", "--evidence-digest", "sha256:ev"],
                       capture_output=True, text=True)
    rec = json.loads(r.stdout)
    assert r.returncode == 0 and rec["schema_version"] == "openagents.psionic_execution_receipt.v1" and rec["receipt_digest"].startswith("sha256:")
    st = json.loads(subprocess.run([cli, "status", "--json", "--state-dir", d], capture_output=True, text=True).stdout)
    assert st["psionic_execution_receipt_digests"] == [rec["receipt_digest"]]
    # rejections: ready and crashed at once; sandbox receipt without a profile digest; bad digest
    bad = json.load(open(fx))
    bad["workers"][0]["crashed"] = True
    json.dump(bad, open(tmp_path / "bad.json", "w"))
    assert subprocess.run([cli, "psionic", "attach", "--file", str(tmp_path / "bad.json"), "--state-dir", d], capture_output=True).returncode == 3
    assert subprocess.run([cli, "psionic", "receipt", "append", "--state-dir", d, "--assignment-id", "a", "--product-id", "sandbox.x",
                           "--worker-id", "w", "--status", "succeeded", "--evidence-digest", "sha256:e"], capture_output=True).returncode == 3
    assert subprocess.run([cli, "psionic", "receipt", "append", "--state-dir", d, "--assignment-id", "a", "--product-id", "p",
                           "--worker-id", "w", "--status", "succeeded", "--evidence-digest", "md5:e"], capture_output=True).returncode == 3


def test_manifests_and_payout_split(gguf_path):
    mm = mf.model_artifact_manifest(gguf_path, "llama", "Q8_0", "sha256:" + "0" * 64)
    assert mf.verify_manifest(mm) and mm["artifactDigest"] == mf.artifact_digest(gguf_path)
    rm = mf.release_manifest("0.1.0", {"model": gguf_path}, [mm])
    assert mf.verify_manifest(rm)
    rm["version"] = "0.1.1"
    assert not mf.verify_manifest(rm)
    stages = [{"stageIndex": 0, "layerStart": 0, "layerEnd": 11, "gpuResident": True},
              {"stageIndex": 1, "layerStart": 11, "layerEnd": 32, "gpuResident": True}]
    rec = mf.sharded_run_receipt("sha256:m", 32, stages)
    assert mf.structural_errors(rec) == []
    split = mf.payout_split(rec, 1001)
    assert sum(s["payoutSats"] for s in split) == 1001 and split[0]["payoutSats"] == 344 and split[1]["payoutSats"] == 657
    gap = mf.sharded_run_receipt("sha256:m", 32, [stages[0], {**stages[1], "layerStart": 12}])
    assert any("gap" in e for e in mf.structural_errors(gap))
    whole = mf.sharded_run_receipt("sha256:m", 32, [{"stageIndex": 0, "layerStart": 0, "layerEnd": 32, "gpuResident": True}])
    assert len(mf.structural_errors(whole)) >= 2
    with pytest.raises(ValueError):
        mf.payout_split(mf.sharded_run_receipt("sha256:m", 32, stages, "mismatch"), 10)


# ---------------------------------------------------------------- scheduler: failures stay with their request

class _FakeBackend:
    """Scripted backend: counts calls, serves arg-max ``(last token + 1) % 50``, fails where told to."""
    name = "fake"

    def __init__(self, max_context=64, fail_seq=None):
        from openagents_b200.models.config import TINY_LLAMA
        self.cfg = TINY_LLAMA.with_(vocab=512)
        self._max, self.fail_seq = max_context, fail_seq
        self.open, self.ended, self.batches, self.published = {}, [], [], {}
        self.last_d2h_bytes = 0

    @property
    def max_context(self):
        return self._max

    def begin(self, seq_id, prompt):
        self.open[seq_id] = 0
        return 0

    def step(self, seq_ids, new_tokens, params, uniforms):
        if self.fail_seq is not None and self.fail_seq in seq_ids:
            raise MemoryError("KV cache is out of pages")
        self.batches.append(list(seq_ids))
        for s, t in zip(seq_ids, new_tokens):
            self.open[s] += len(t)
        self.last_d2h_bytes = 4 * len(seq_ids)
        return [(t[-1] + 1) % 50 for t in new_tokens]

    def publish(self, seq_id, tokens):
        self.published[seq_id] = list(tokens)

    def end(self, seq_id):
        self.ended.append(seq_id)
        self.open.pop(seq_id, None)


def test_failed_request_does_not_block_the_queue():
    from openagents_b200.serve.generation import RequestRejected
    be = _FakeBackend(max_context=32)
    sch = Scheduler(be, ByteTokenizer(512), max_num_seqs=4, prefill_chunk=64)
    with pytest.raises(RequestRejected):            # longer than the context window: refused at the door
        sch.submit(list(range(1, 30)), SamplingParams(max_tokens=8))
    assert not sch.waiting and sch.stats["rejected"] == 1
    bad = sch.submit([1, 2, 3], SamplingParams(max_tokens=4))
    good = sch.submit([4, 5, 6], SamplingParams(max_tokens=4))
    be.fail_seq = 1                                  # the first sequence the scheduler opens
    sch.run_until_done([bad, good], max_steps=50)
    assert bad.finish_reason == "error" and isinstance(bad.error, MemoryError)
    assert good.finish_reason == "length" and good.output == [7, 8, 9, 10]
    assert 1 in be.ended and not sch.waiting and not sch.running and sch.stats["errors"] == 1
    later = sch.submit([9], SamplingParams(max_tokens=2))     # and the scheduler keeps serving
    sch.run_until_done([later], max_steps=10)
    assert later.output == [10, 11]


def test_prefill_is_batched_and_sessions_publish_their_whole_history():
    be = _FakeBackend()
    sch = Scheduler(be, ByteTokenizer(512), max_num_seqs=8, prefill_chunk=64)
    reqs = [sch.submit([10 + i, 11 + i, 12 + i], SamplingParams(max_tokens=3)) for i in range(4)]
    sch.step()
    assert be.batches[0] == [1, 2, 3, 4]             # four prompts shared one forward call
    assert sch.stats["prefill_seqs_sum"] / sch.stats["prefill_calls"] == 4
    sch.run_until_done(reqs, max_steps=20)
    assert sch.stats["batch_size_sum"] / sch.stats["steps"] == 4 and sch.stats["d2h_bytes"] > 0
    first = sch.submit([1, 2], SamplingParams(max_tokens=2), keep_sequence=True)
    sch.run_until_done([first])
    turn2 = sch.submit([30, 31], SamplingParams(max_tokens=2), seq_id=first.seq_id, keep_sequence=True, history=[1, 2, 3])
    sch.run_until_done([turn2])
    assert be.published[first.seq_id] == [1, 2, 3, 30, 31]      # earlier turns + the new one, never the new turn alone


def test_concurrent_http_requests_share_decode_batches(gguf_path):
    model = ServedModel("tiny", CpuBackend.from_gguf(gguf_path), None, max_num_seqs=8)
    state = ServerState([model])
    httpd = serve(state, "127.0.0.1", 0)
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    base = f"http://127.0.0.1:{httpd.server_address[1]}"
    out = [None] * 8

    def one(i):
        body = {"messages": [{"role": "user", "content": f"question number {i}"}], "max_tokens": 64, "temperature": 0, "stream": True}
        out[i] = _post(base + "/v1/chat/completions", body)

    import time
    ts = [threading.Thread(target=one, args=(i,)) for i in range(8)]
    with model.lock:                 # hold the scheduler until every connection has reached its submit
        for t in ts:
            t.start()
        time.sleep(1.0)
    for t in ts:
        t.join(timeout=300)
    httpd.shutdown()
    assert all(o is not None and o[0] == 200 and b"[DONE]" in o[1] for o in out)
    s = model.sched.stats
    assert s["batch_size_sum"] / s["steps"] > 4, s      # the eight streams decoded together, not one after another
    assert state.ledger.total() > 0 and len(state.ledger.rows) == 8
    model.close()


def test_over_long_prompt_is_rejected_and_server_keeps_working(server):
    base, state = server
    long_text = "x" * (state.default.backend.cfg.context + 10)
    code, raw = _post(base + "/v1/chat/completions", {"messages": [{"role": "user", "content": long_text}], "max_tokens": 4})
    assert code == 400 and json.loads(raw)["error"]["type"] == "context_length_exceeded"
    code, raw = _post(base + "/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 3, "temperature": 0})
    assert code == 200 and json.loads(raw)["usage"]["completion_tokens"] <= 3


def test_sampling_on_host_matches_its_definition():
    from openagents_b200.serve.backend import sample_row
    logits = torch.tensor([0.1, 3.0, 2.5, -1.0, 2.9])
    assert sample_row(logits, SamplingParams(temperature=0.0), 0.7) == 1
    p = SamplingParams(temperature=1.0, top_k=3, top_p=1.0)
    probs = torch.softmax(torch.tensor([3.0, 2.9, 2.5]), 0)          # candidates 1, 4, 2 in that order
    assert sample_row(logits, p, 0.0) == 1
    assert sample_row(logits, p, float(probs[0]) + 1e-3) == 4
    assert sample_row(logits, p, 0.999) == 2
    assert sample_row(logits, SamplingParams(temperature=1.0, top_k=3, top_p=0.2), 0.999) == 1    # top-p keeps only the best


def test_shutdown_route_is_off_unless_allowed(gguf_path):
    model = ServedModel("tiny", CpuBackend.from_gguf(gguf_path), mf.artifact_digest(gguf_path), max_num_seqs=2)
    state = ServerState([model])
    httpd = serve(state, "127.0.0.1", 0)
    t = threading.Thread(target=httpd.serve_forever, daemon=True)
    t.start()
    url = f"http://127.0.0.1:{httpd.server_address[1]}"
    status, _ = _post(url + "/admin/shutdown", {})
    assert status == 404 and t.is_alive()
    state.allow_shutdown = True
    status, body = _post(url + "/admin/shutdown", {})
    assert status == 200 and json.loads(body)["stopping"] is True
    t.join(10)
    assert not t.is_alive()
    model.close()


def test_admitted_chat_template_is_rendered_in_a_sandbox(gguf_path, monkeypatch):
    from openagents_b200.control.node_bridge import template_admitted, template_digest
    from openagents_b200.serve.generation import render_chat
    tpl = ("{{ bos_token }}{% for m in messages %}<|start|>{{ m['role'] }}\\n{{ m['content'] }}<|end|>\\n{% endfor %}"
           "{% if add_generation_prompt %}<|start|>assistant\\n{% endif %}{% if reasoning_effort is defined %}[{{ reasoning_effort }}]{% endif %}")
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hi"}]
    out = render_chat(msgs, tpl, bos_token="<s>", reasoning_effort="low")
    assert out == "<s><|start|>system\\nbe brief<|end|>\\n<|start|>user\\nhi<|end|>\\n<|start|>assistant\\n[low]"
    builtin = render_chat(msgs)
    assert builtin.endswith("<|assistant|>\n") and render_chat(msgs, None) == builtin
    # the sandbox: no reaching into Python internals, no mutation of the request; a failing template falls back
    assert render_chat(msgs, "{{ messages.__class__.__mro__ }}") == builtin
    assert render_chat(msgs, "{% set _ = messages.append({'role': 'x'}) %}{{ messages | length }}") == builtin and len(msgs) == 2
    assert render_chat(msgs, "{{ raise_exception('only user/assistant roles') }}") == builtin
    # the server renders a template only when its digest is admitted
    assert not template_admitted(tpl)
    monkeypatch.setenv("B200_CHAT_TEMPLATE_ALLOW", template_digest(tpl))
    assert template_admitted(tpl)
    model = ServedModel("tiny", CpuBackend.from_gguf(gguf_path), mf.artifact_digest(gguf_path), max_num_seqs=2, chat_template=tpl)
    state = ServerState([model])
    r1, u1 = state.complete(model, msgs, {"max_tokens": 2})
    model.chat_template = None
    r2, u2 = state.complete(model, msgs, {"max_tokens": 2})
    assert u1["prompt_tokens"] != u2["prompt_tokens"]            # different prompt text reached the tokenizer
    model.close()


def test_stream_flushes_bytes_held_back_as_incomplete_utf8(gguf_path):
    """A model that ends on a byte which starts a multi-byte character: the streamed text equals the plain answer."""
    class _Tail(CpuBackend):
        def step(self, seq_ids, new_tokens, params, uniforms):
            out = super().step(seq_ids, new_tokens, params, uniforms)
            return [0xE2 for _ in out]                    # first byte of a three-byte sequence, never completed
    be = _Tail.from_gguf(gguf_path)
    model = ServedModel("tiny", be, None, max_num_seqs=2)
    state = ServerState([model])
    httpd = serve(state, "127.0.0.1", 0)
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    base = f"http://127.0.0.1:{httpd.server_address[1]}"
    body = {"messages": [{"role": "user", "content": "x"}], "max_tokens": 3, "temperature": 0}
    _, plain = _post(base + "/v1/chat/completions", body)
    _, raw = _post(base + "/v1/chat/completions", {**body, "stream": True})
    text = "".join((json.loads(ln[5:])["choices"][0]["delta"].get("content") or "") for ln in raw.decode().splitlines()
                   if ln.startswith("data:") and "[DONE]" not in ln)
    want = json.loads(plain)["choices"][0]["message"]["content"]
    assert want and text == want
    httpd.shutdown()
    model.close()


def test_ngram_speculation_gives_exactly_the_greedy_output(gguf_path):
    """Prompt-lookup drafts verified in one forward: same tokens as plain greedy decoding, fewer steps, KV rolled back
    after rejected tails (a second turn on the same session still matches), stop conditions honoured mid-draft."""
    from openagents_b200.serve.generation import SpeculationConfig, ngram_draft
    assert ngram_draft([1, 2, 3, 4, 5, 1, 2, 3], 3, 4) == [4, 5, 1, 2] and ngram_draft([1, 2, 3], 3, 4) == []
    prompt = list(b"abcabcabcabc the cat sat on the mat the cat sat on")
    outs, steps = {}, {}
    for name, spec in (("plain", None), ("spec", SpeculationConfig(max_batch=4, ngram=3, draft=4))):
        be = CpuBackend.from_gguf(gguf_path)
        sch = Scheduler(be, ByteTokenizer(be.cfg.vocab), max_num_seqs=4, speculation=spec)
        r = sch.submit(prompt, SamplingParams(max_tokens=40), keep_sequence=True)
        sch.run_until_done([r])
        # a second turn on the same sequence: only correct if the KV cache holds exactly the accepted tokens
        feed = [r.output[-1]] + list(b" again")
        r2 = sch.submit(feed, SamplingParams(max_tokens=12), seq_id=r.seq_id, keep_sequence=True, history=prompt + r.output[:-1])
        sch.run_until_done([r2])
        outs[name], steps[name] = (r.output, r2.output, r.finish_reason), sch.stats["steps"]
        if spec:
            st = sch.stats
            assert st["spec_steps"] > 0 and st["spec_drafted"] >= st["spec_accepted"] >= 0
            held = lambda q: len(q.output) - (1 if q.finish_reason == "length" else 0)      # an end-of-sequence token was sampled from the last output's forward
            assert be.seq_len(r.seq_id) == len(prompt) + held(r) + len(feed) + held(r2)
            rate = sch.speculation_acceptance_rate
            assert rate is not None and 0.0 <= rate <= 1.0
    assert outs["spec"] == outs["plain"]
    assert steps["spec"] <= steps["plain"]
    # sampling requests and large batches never speculate
    be = CpuBackend.from_gguf(gguf_path)
    sch = Scheduler(be, ByteTokenizer(be.cfg.vocab), max_num_seqs=8, speculation=SpeculationConfig(max_batch=1))
    rs = [sch.submit(prompt, SamplingParams(max_tokens=6)) for _ in range(2)] + [sch.submit(prompt, SamplingParams(max_tokens=6, temperature=0.8, seed=1))]
    sch.run_until_done(rs)
    assert sch.stats["spec_steps"] == 0


def test_speculation_is_disclosed_per_request(gguf_path):
    from openagents_b200.serve.generation import SpeculationConfig
    model = ServedModel("tiny", CpuBackend.from_gguf(gguf_path), None, max_num_seqs=2, speculation=SpeculationConfig())
    state = ServerState([model])
    msgs = [{"role": "user", "content": "abcabcabcabc the cat sat on the mat the cat sat on"}]
    r, usage = state.complete(model, msgs, {"max_tokens": 24})
    sp = usage["speculation"]
    assert sp["mode"] == "n_gram" and sp["draftTokensProposed"] == r.spec_proposed and sp["draftTokensAccepted"] == r.spec_accepted
    assert state.status()["models"][0]["levers"]["speculation"] == "n_gram"
    plain = ServedModel("tiny2", CpuBackend.from_gguf(gguf_path), None, max_num_seqs=2)
    assert "speculation" not in ServerState([plain]).complete(plain, msgs, {"max_tokens": 4})[1]
    model.close()
    plain.close()


def test_logprobs_of_the_chosen_tokens(server, gguf_path):
    """``logprobs: true`` on a non-streamed completion: one extra forward scores the generated tokens; a greedy token's
    log-probability is the maximum of its distribution, and the values equal a direct computation on the oracle."""
    import math
    import torch
    from openagents_b200.oracle.models import llama_forward
    base, state = server
    m0 = state.models["tiny"] if isinstance(state.models, dict) else state.models[0]
    open_before = m0.backend.kv_stats()["sequences"]          # sessions of earlier tests may still hold theirs
    body = {"model": "tiny", "messages": [{"role": "user", "content": "hello"}], "max_tokens": 5, "logprobs": True}
    code, raw = _post(base + "/v1/chat/completions", body)
    assert code == 200, raw
    c = json.loads(raw)["choices"][0]
    rows = c["logprobs"]["content"]
    assert 1 <= len(rows) <= 5 and all(r["logprob"] <= 0.0 and r["top_logprobs"] == [] and isinstance(r["bytes"], list) for r in rows)
    m = state.models["tiny"] if isinstance(state.models, dict) else state.models[0]
    from openagents_b200.serve.generation import render_chat
    prompt = m.tok.encode(render_chat(body["messages"], m.chat_template))
    be = m.backend
    out_ids, feed = [], list(prompt)
    logits = llama_forward(be.cfg, be.W, torch.tensor(feed), None).double()
    for r in rows:
        lp = torch.log_softmax(logits[-1], -1)
        nxt = int(lp.argmax())
        assert r["logprob"] == pytest.approx(float(lp[nxt]), abs=1e-4) and math.isfinite(r["logprob"])
        out_ids.append(nxt)
        feed.append(nxt)
        logits = llama_forward(be.cfg, be.W, torch.tensor(feed), None).double()
    assert be.kv_stats()["sequences"] == open_before        # the scoring sequence was closed
    assert _post(base + "/v1/chat/completions", {**body, "stream": True})[0] == 400
    assert _post(base + "/v1/chat/completions", {**body, "top_logprobs": 3})[0] == 400
    assert "logprobs" not in json.loads(_post(base + "/v1/chat/completions", {**body, "logprobs": False})[1])["choices"][0]


def test_text_completions_with_echo_and_logprobs(server):
    """``/v1/completions``: generation on a raw prompt, and ``max_tokens: 0`` + ``echo`` + ``logprobs`` as a scoring call (the
    log-likelihood request of evaluation harnesses), checked against the oracle."""
    import torch
    from openagents_b200.oracle.models import llama_forward
    base, state = server
    m = state.models["tiny"] if isinstance(state.models, dict) else state.models[0]
    code, raw = _post(base + "/v1/completions", {"model": "tiny", "prompt": "abc", "max_tokens": 4})
    c = json.loads(raw)
    assert code == 200 and c["object"] == "text_completion" and c["usage"] == {"prompt_tokens": 3, "completion_tokens": c["usage"]["completion_tokens"], "total_tokens": 3 + c["usage"]["completion_tokens"]}
    assert c["choices"][0]["logprobs"] is None and 1 <= c["usage"]["completion_tokens"] <= 4
    code, raw = _post(base + "/v1/completions", {"model": "tiny", "prompt": "hello world", "max_tokens": 0, "echo": True, "logprobs": 1})
    s = json.loads(raw)["choices"][0]
    ids = m.tok.encode("hello world")
    want = torch.log_softmax(llama_forward(m.backend.cfg, m.backend.W, torch.tensor(ids), None).double(), -1)
    assert code == 200 and s["text"] == "hello world" and s["logprobs"]["token_ids"] == ids and s["logprobs"]["token_logprobs"][0] is None
    for i in range(1, len(ids)):
        assert s["logprobs"]["token_logprobs"][i] == pytest.approx(float(want[i - 1, ids[i]]), abs=1e-4)
    assert s["logprobs"]["text_offset"] == list(range(len(ids))) and s["logprobs"]["tokens"][:2] == ["h", "e"]
    # generation + logprobs without echo: only the new tokens are listed; token ids as the prompt
    code, raw = _post(base + "/v1/completions", {"model": "tiny", "prompt": ids, "max_tokens": 3, "logprobs": True})
    g = json.loads(raw)["choices"][0]
    assert code == 200 and len(g["logprobs"]["token_logprobs"]) == len(g["logprobs"]["token_ids"]) <= 3 and all(x <= 0 for x in g["logprobs"]["token_logprobs"])
    for bad in ({"prompt": ""}, {"prompt": [["a"], ["b"]]}, {"prompt": "x", "max_tokens": 0}, {"prompt": "x", "stream": True}, {"prompt": [10 ** 9]}):
        assert _post(base + "/v1/completions", {"model": "tiny", **bad})[0] == 400
    assert "/v1/completions" in json.loads(_get(base + "/health")[1])["endpoints"]


def test_remote_scorers_agree_with_the_in_process_ones(server, tmp_path):
    import numpy as np
    from openagents_b200.data import TokenDataset, write_token_shard
    from openagents_b200.eval import multiple_choice, perplexity
    from openagents_b200.eval.remote import loglikelihood, multiple_choice_http, perplexity_http
    base, state = server
    m = state.models["tiny"] if isinstance(state.models, dict) else state.models[0]
    items = [{"context": "the cat", "choices": [" sat", " flew away"], "answer": 0}]
    with m.lock:
        local = multiple_choice(m.backend, items, m.tok)
    remote = multiple_choice_http(base, "tiny", items, m.tok)
    assert remote["picks"][0]["scores"] == pytest.approx(local["picks"][0]["scores"], abs=1e-4) and remote["accuracy"] == local["accuracy"]
    assert loglikelihood(base, "tiny", [1, 2, 3], [4, 5]) < 0
    write_token_shard(tmp_path / "v.b2tk", np.random.default_rng(3).integers(0, 500, 80))
    ds = TokenDataset(tmp_path / "v.b2tk", seq_len=16)
    r = perplexity_http(base, "tiny", ds, max_windows=2)
    with m.lock:
        l = perplexity(m.backend, ds, max_windows=2)
    # a window of 16 inputs and its final target is 17 ids on the wire: the same 16 predictions the in-process scorer makes
    assert r["targets"] == l["targets"] == 2 * 16 and r["loss"] == pytest.approx(l["loss"], abs=1e-4)


# ---- mistyped requests: a typed 400 that names the field, never an engine error, a dropped connection or a stuck scheduler
_M = [{"role": "user", "content": "hi"}]
_BAD_BODIES = [
    ("/v1/chat/completions", {"model": ["tiny"]}, "model"),
    ("/v1/chat/completions", {"model": {"a": 1}}, "model"),
    ("/v1/chat/completions", {"messages": [[]]}, "messages[0]"),
    ("/v1/chat/completions", {"messages": [{"role": 5, "content": "x"}]}, "role"),
    ("/v1/chat/completions", {"messages": [{"role": "user", "content": 3.5}]}, "content"),
    ("/v1/chat/completions", {"messages": 1e9}, "messages"),
    ("/v1/chat/completions", {"max_tokens": [1]}, "max_tokens"),
    ("/v1/chat/completions", {"max_tokens": 3.5}, "max_tokens"),
    ("/v1/chat/completions", {"max_tokens": "many"}, "max_tokens"),
    ("/v1/chat/completions", {"max_tokens": -1}, "max_tokens"),
    ("/v1/chat/completions", {"max_tokens": True}, "max_tokens"),
    ("/v1/chat/completions", {"temperature": "hot"}, "temperature"),
    ("/v1/chat/completions", {"temperature": -0.5}, "temperature"),
    ("/v1/chat/completions", {"top_p": [1, 2]}, "top_p"),
    ("/v1/chat/completions", {"top_p": 1.5}, "top_p"),
    ("/v1/chat/completions", {"top_k": {}}, "top_k"),
    ("/v1/chat/completions", {"seed": ""}, "seed"),
    ("/v1/chat/completions", {"seed": -1}, "seed"),
    ("/v1/chat/completions", {"stop": 3.5}, "stop"),
    ("/v1/chat/completions", {"stop": True}, "stop"),
    ("/v1/chat/completions", {"stop": [[]]}, "stop"),
    ("/v1/chat/completions", {"stream": 1e9}, "stream"),
    ("/v1/chat/completions", {"stream": [1]}, "stream"),
    ("/v1/chat/completions", {"tools": "hammer"}, "tools"),
    ("/v1/chat/completions", {"tools": [1]}, "tools"),
    ("/v1/chat/completions", {"chat_template_kwargs": [1, 2]}, "chat_template_kwargs"),
    ("/v1/chat/completions", {"chat_template_kwargs": {"messages": []}}, "chat_template_kwargs"),
    ("/v1/chat/completions", {"top_logprobs": "x"}, "top_logprobs"),
    ("/v1/chat/completions", {"user": [[]]}, "user"),
    ("/v1/responses", {"previous_response_id": {}}, "previous_response_id"),
    ("/v1/responses", {"input": True}, "input"),
    ("/v1/responses", {"input": [1, 2]}, "input[0]"),
    ("/v1/completions", {"prompt": 3.5}, "prompt"),
    ("/v1/completions", {"prompt": "abc", "echo": "yes"}, "echo"),
    ("/v1/completions", {"prompt": "abc", "max_tokens": [2]}, "max_tokens"),
    ("/v1/serve", {"messages": True}, "messages"),
    ("/v1/serve", {"passthroughParams": 7}, "passthroughParams"),
    ("/v1/serve", {"passthroughParams": {"top_k": []}}, "top_k"),
]


@pytest.mark.parametrize("path,patch,field", _BAD_BODIES, ids=[f"{p.rsplit('/', 1)[-1]}-{json.dumps(b)[:40]}" for p, b, _ in _BAD_BODIES])
def test_mistyped_request_fields_get_a_typed_400(server, path, patch, field):
    base, _ = server
    body = {"model": "tiny", "messages": _M, "max_tokens": 2, **patch}
    code, raw = _post(base + path, body)
    err = json.loads(raw)["error"]
    assert code == 400 and err["type"] == "invalid_request_error" and field in err["message"], (code, raw)
    code, raw = _post(base + "/v1/chat/completions", {"model": "tiny", "messages": _M, "max_tokens": 2})     # and the server still serves
    assert code == 200 and json.loads(raw)["usage"]["completion_tokens"] >= 1


def test_bodies_that_are_not_json_objects_get_a_400(server):
    base, _ = server
    for raw in (b"{", b"[]", b"null", b"\xff\xfe{}", b"12"):
        req = urllib.request.Request(base + "/v1/chat/completions", data=raw, headers={"Content-Type": "application/json"})
        with pytest.raises(urllib.error.HTTPError) as e:
            urllib.request.urlopen(req, timeout=60)
        assert e.value.code == 400 and json.loads(e.value.read())["error"]["type"] == "invalid_request_error"


def test_lenient_spellings_of_valid_requests_are_accepted(server):
    base, _ = server
    for patch in ({"max_tokens": 2.0}, {"stop": None}, {"stop": []}, {"stop": ""}, {"top_p": 0}, {"top_k": 0}, {"seed": 7, "temperature": 0.7},
                  {"stream": None}, {"tools": None}, {"chat_template_kwargs": {"reasoning_effort": "low"}}, {"model": ""}, {"user": "u-1"}):
        code, raw = _post(base + "/v1/chat/completions", {"model": "tiny", "messages": _M, "max_tokens": 2, **patch})
        assert code == 200, (patch, raw)


def test_scheduling_thread_survives_a_request_it_cannot_process(gguf_path):
    """Whatever a request does to the scheduler's own bookkeeping (here: a stop entry that is not a string, put past the HTTP
    checks), that request ends with an error and the next one is served; nothing waits on a dead thread."""
    model = ServedModel("tiny", CpuBackend.from_gguf(gguf_path), None, max_num_seqs=4)
    try:
        with pytest.raises(TypeError):
            model.generate([1, 2, 3], SamplingParams(max_tokens=3, stop=(3.5,)))
        assert model.thread.is_alive()
        ok = model.generate([1, 2, 3], SamplingParams(max_tokens=3))
        assert len(ok.output) >= 1 and ok.finish_reason in ("length", "stop")

        def boom():
            raise RuntimeError("step failed")
        step, model.sched.step = model.sched.step, boom            # a step that raises outright: every waiter is released
        with pytest.raises(RuntimeError, match="step failed"):
            model.generate([1, 2, 3], SamplingParams(max_tokens=3))
        model.sched.step = step
        assert model.thread.is_alive() and len(model.generate([4, 5], SamplingParams(max_tokens=2)).output) >= 1
    finally:
        model.close()


def test_session_turns_streamed_as_growing_snapshots(server):
    """``POST /v1/sessions/{id}/responses/stream``: one ``snapshot`` event per step whose content grows toward the answer, then
    ``completed``; the turn lands in the session exactly like a non-streamed one (same tokens, KV kept for the next turn)."""
    base, state = server

    def events(raw):
        out = []
        for block in raw.decode().split("\n\n"):
            lines = dict(l.split(": ", 1) for l in block.split("\n") if ": " in l)
            if "event" in lines:
                out.append((lines["event"], json.loads(lines["data"])))
        return out

    sid = json.loads(_post(base + "/v1/sessions", {"model": "tiny", "instructions": "Be brief."})[1])["id"]
    ref = json.loads(_post(base + "/v1/sessions", {"model": "tiny", "instructions": "Be brief."})[1])["id"]
    code, raw = _post(base + f"/v1/sessions/{sid}/responses/stream", {"prompt": "hello there", "max_tokens": 6})
    assert code == 200
    ev = events(raw)
    snaps = [d for e, d in ev if e == "snapshot"]
    assert [e for e, _ in ev][-1] == "completed" and len(snaps) >= 1
    assert [d["sequence"] for d in snaps] == list(range(len(snaps)))
    assert all(b["content"].startswith(a["content"]) for a, b in zip(snaps, snaps[1:]))            # each snapshot extends the last
    assert all(d["finish_reason"] is None for d in snaps[:-1]) and snaps[-1]["finish_reason"] in ("length", "stop")
    done = ev[-1][1]
    assert done["output"] == snaps[-1]["content"] == done["content"] and done["model"] == "tiny" and done["usage"]["completion_tokens"] == 6
    plain = json.loads(_post(base + f"/v1/sessions/{ref}/responses", {"prompt": "hello there", "max_tokens": 6})[1])
    assert plain["output_text"] == done["output"] and plain["usage"]["prompt_tokens"] == done["usage"]["prompt_tokens"]
    # the second turn continues the kept sequence on both; the instructions were part of the first turn only
    code, raw = _post(base + f"/v1/sessions/{sid}/responses/stream", {"prompt": "and then?", "max_tokens": 4})
    second = events(raw)[-1][1]
    plain2 = json.loads(_post(base + f"/v1/sessions/{ref}/responses", {"prompt": "and then?", "max_tokens": 4})[1])
    assert second["output"] == plain2["output_text"] and second["usage"]["prompt_tokens"] == plain2["usage"]["prompt_tokens"] < done["usage"]["prompt_tokens"]
    assert state.sessions[sid].tokens == state.sessions[ref].tokens
    assert _post(base + "/v1/sessions/sess-nope/responses/stream", {"prompt": "x"})[0] == 404
    code, raw = _post(base + f"/v1/sessions/{sid}/responses/stream", {"prompt": 5})
    assert code == 400 and "prompt" in json.loads(raw)["error"]["message"]


def test_attach_client_streams_a_session_turn(server):
    from openagents_b200.serve.attach_client import AttachClient
    base, _ = server
    c = AttachClient(base + "/v1")
    sid = c.create_session("tiny", instructions="Be brief.")
    got = list(c.stream_turn(sid, "hello there", max_tokens=5))
    assert [k for k, _ in got][-1] == "completed" and all(k == "snapshot" for k, _ in got[:-1])
    assert got[-1][1]["output"] == got[-2][1] and got[-1][1]["usage"]["completion_tokens"] == 5


def test_mixed_concurrent_traffic_with_abandoned_streams_leaves_nothing_behind(gguf_path):
    """Eight clients at once over every generating route, some hanging up in the middle of a stream: every request is answered,
    no handler or scheduler state is left over (sequences, KV tokens, sessions), and the server still answers afterwards."""
    import random
    import socket
    model = ServedModel("tiny", CpuBackend.from_gguf(gguf_path), None, max_num_seqs=4)
    state = ServerState([model])
    httpd = serve(state, "127.0.0.1", 0)
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    port = httpd.server_address[1]
    base = f"http://127.0.0.1:{port}"

    def abandon(path, body):
        s = socket.create_connection(("127.0.0.1", port))
        data = json.dumps(body).encode()
        s.sendall(f"POST {path} HTTP/1.1\r\nHost: x\r\nContent-Type: application/json\r\nContent-Length: {len(data)}\r\n\r\n".encode() + data)
        s.recv(200)
        s.close()

    problems = []

    def client(i):
        rnd = random.Random(i)
        for j in range(8):
            msgs = [{"role": "user", "content": f"hello {i} {j} " + "x" * rnd.randrange(40)}]
            try:
                k = (i + j) % 5
                if k == 0:
                    code = _post(base + "/v1/chat/completions", {"messages": msgs, "max_tokens": rnd.randrange(1, 10)})[0]
                elif k == 1:
                    code = _post(base + "/v1/chat/completions", {"messages": msgs, "max_tokens": 6, "stream": True})[0]
                elif k == 2:
                    abandon("/v1/chat/completions", {"messages": msgs, "max_tokens": 48, "stream": True})
                    code = 200
                elif k == 3:
                    code = _post(base + "/v1/completions", {"prompt": "abc " * 5, "max_tokens": 3, "echo": True, "logprobs": 1})[0]
                else:
                    sid = json.loads(_post(base + "/v1/sessions", {})[1])["id"]
                    _post(base + f"/v1/sessions/{sid}/responses/stream", {"prompt": "hi", "max_tokens": 4})
                    code = _post(base + f"/v1/sessions/{sid}/responses", {"prompt": "more", "max_tokens": 4})[0]
                    urllib.request.urlopen(urllib.request.Request(base + f"/v1/sessions/{sid}", method="DELETE"), timeout=60).read()
                if code != 200:
                    problems.append((k, code))
            except Exception as e:      # noqa: BLE001
                problems.append((i, j, repr(e)))

    try:
        threads = [threading.Thread(target=client, args=(i,)) for i in range(8)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout=240)
        assert not any(t.is_alive() for t in threads) and problems == []
        import time
        deadline = time.time() + 10               # an abandoned stream is cancelled when its next token cannot be written
        while time.time() < deadline and (model.sched.running or model.sched.waiting):
            time.sleep(0.05)
        assert not model.sched.running and not model.sched.waiting and state.sessions == {}
        assert model.backend.kv_stats()["sequences"] == 0 and model.backend.kv_stats()["tokens"] == 0
        assert model.sched.stats["errors"] == 0 and model.thread.is_alive()
        assert _post(base + "/v1/chat/completions", {"messages": [{"role": "user", "content": "still there?"}], "max_tokens": 2})[0] == 200
    finally:
        httpd.shutdown()
        model.close()


class _LimitedPool:
    """A CPU backend whose KV pool holds at most ``limit`` sequences (``begin`` beyond that raises ``MemoryError``, as the paged
    pool does when it is out of pages) and whose ``step`` can be made to fail once."""

    def __init__(self, inner, limit):
        self.inner, self.limit, self.open, self.fail_next_step = inner, limit, set(), None

    def __getattr__(self, name):
        return getattr(self.inner, name)

    def begin(self, seq_id, prompt):
        if len(self.open) >= self.limit:
            raise MemoryError("KV cache is out of pages")
        r = self.inner.begin(seq_id, prompt)
        self.open.add(seq_id)
        return r

    def end(self, seq_id):
        self.open.discard(seq_id)
        return self.inner.end(seq_id)

    def step(self, *a, **kw):
        if self.fail_next_step is not None:
            e, self.fail_next_step = self.fail_next_step, None
            raise e
        return self.inner.step(*a, **kw)


def test_idle_sessions_are_evicted_by_cap_by_age_and_when_the_kv_pool_runs_out(gguf_path):
    be = _LimitedPool(CpuBackend.from_gguf(gguf_path), limit=3)
    model = ServedModel("tiny", be, None, max_num_seqs=4)
    state = ServerState([model])
    state.max_sessions = 3
    httpd = serve(state, "127.0.0.1", 0)
    threading.Thread(target=httpd.serve_forever, daemon=True).start()
    base = f"http://127.0.0.1:{httpd.server_address[1]}"
    try:
        turn = lambda **kw: _post(base + "/v1/responses", {"input": "hello", "max_tokens": 3, **kw})
        first = json.loads(turn()[1])["id"]
        ids = [json.loads(turn()[1])["id"] for _ in range(2)]
        assert len(state.sessions) == 3 and len(be.open) == 3                       # each conversation keeps its sequence
        # the cap: a fourth conversation pushes the least recently used one out, and its response id stops resolving
        fourth = json.loads(turn()[1])["id"]
        assert len(state.sessions) == 3 and len(be.open) == 3 and state.sessions_evicted == 1
        code, raw = turn(previous_response_id=first)
        assert code == 404 and "expired" in json.loads(raw)["error"]["message"]
        assert turn(previous_response_id=ids[1])[0] == 200                           # the others continue
        # the pool is full of idle conversations: a plain request evicts some of them and is then served
        state.max_sessions = 100
        code, raw = _post(base + "/v1/chat/completions", {"messages": [{"role": "user", "content": "room?"}], "max_tokens": 2})
        assert code == 200 and state.sessions_evicted >= 2 and len(be.open) < 3, raw
        # age: a conversation idle for longer than the time-to-live goes at the next sweep
        keep = json.loads(turn()[1])["id"]
        for s in state.sessions.values():
            s.last_used -= state.session_ttl_s + 1
        assert state.reap_sessions() >= 1
        assert state.sessions == {} and be.open == set() and turn(previous_response_id=keep)[0] == 404
        assert "b200_sessions_evicted_total" in _get(base + "/metrics")[1].decode()
        assert json.loads(_get(base + "/psionic/management/status")[1])["sessions_evicted"] == state.sessions_evicted
        # a later turn that fails closes the sequence it continued (nothing keeps the forgotten conversation's pages)
        sid = json.loads(_post(base + "/v1/sessions", {})[1])["id"]
        assert _post(base + f"/v1/sessions/{sid}/responses", {"prompt": "one", "max_tokens": 2})[0] == 200 and len(be.open) == 1
        be.fail_next_step = RuntimeError("injected engine failure")
        code, raw = _post(base + f"/v1/sessions/{sid}/responses", {"prompt": "two", "max_tokens": 2})
        assert code == 500 and "injected" in raw.decode() and be.open == set() and state.sessions[sid].seq_id is None
        assert _post(base + f"/v1/sessions/{sid}/responses", {"prompt": "three", "max_tokens": 2})[0] == 200      # the session starts over
        # with nothing left to evict, exhaustion is the typed 503
        be.limit = 0
        state.drop_session(sid)
        code, raw = _post(base + "/v1/chat/completions", {"messages": [{"role": "user", "content": "x"}], "max_tokens": 2})
        assert code == 503 and json.loads(raw)["error"]["type"] == "kv_cache_exhausted"
    finally:
        httpd.shutdown()
        model.close()
