"""Evaluation scorers on the fp32 CPU backend, metric gates and the decision."""
import math

import numpy as np
import pytest
import torch

from openagents_b200.data import TokenDataset, write_token_shard
from openagents_b200.eval import EvalPack, MetricGate, decide, eval_run_evidence, exact_match, multiple_choice, perplexity, run_pack
from openagents_b200.models.config import ModelConfig
from openagents_b200.models.weights import random_weights
from openagents_b200.oracle.models import llama_forward
from openagents_b200.serve.backend import CpuBackend
from openagents_b200.serve.generation import ByteTokenizer

CFG = ModelConfig(name="tiny", arch="llama", vocab=300, d_model=32, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=8, ffn=64, context=128)


@pytest.fixture(scope="module")
def backend():
    return CpuBackend(CFG, {k: v.float() for k, v in random_weights(CFG, 0).items()})


def test_score_matches_full_forward_and_survives_truncate(backend):
    toks = [5, 17, 200, 3, 42, 42, 9]
    logits = llama_forward(CFG, backend.W, torch.tensor(toks), None).double()
    want = torch.log_softmax(logits, -1)
    backend.begin(1, toks)
    got = backend.score(1, toks[:4], [toks[1], toks[2], -1, toks[4]])
    assert got[2] == 0.0
    assert got[0] == pytest.approx(float(want[0, toks[1]]), abs=1e-5) and got[3] == pytest.approx(float(want[3, toks[4]]), abs=1e-5)
    again = backend.score(1, toks[4:6], [toks[5], toks[6]])
    assert again[1] == pytest.approx(float(want[5, toks[6]]), abs=1e-5)
    backend.truncate(1, 4)
    assert backend.score(1, toks[4:6], [toks[5], toks[6]]) == pytest.approx(again, abs=1e-9)
    backend.end(1)


def test_perplexity_matches_cross_entropy(backend, tmp_path):
    rng = np.random.default_rng(0)
    t = rng.integers(0, CFG.vocab, 200)
    mask = np.ones(200, dtype=np.uint8)
    mask[:40] = 0
    write_token_shard(tmp_path / "held.b2tk", t, mask)
    ds = TokenDataset(tmp_path / "held.b2tk", seq_len=32)
    r = perplexity(backend, ds, bytes_per_token=1.0)
    nll, n = 0.0, 0
    for w in range(len(ds)):
        tok, tgt, _ = ds.window(w)
        lp = torch.log_softmax(llama_forward(CFG, backend.W, tok, None).double(), -1)
        keep = tgt >= 0
        nll -= float(lp[torch.arange(32)[keep], tgt[keep]].sum())
        n += int(keep.sum())
    assert r["targets"] == n == 6 * 32 - 39 and r["loss"] == pytest.approx(nll / n, rel=1e-6)
    assert r["perplexity"] == pytest.approx(math.exp(nll / n), rel=1e-6) and r["bitsPerByte"] == pytest.approx(nll / n / math.log(2), rel=1e-6)
    assert abs(r["loss"] - math.log(CFG.vocab)) < 1.0                 # a random model is near uniform
    assert backend.kv_stats()["sequences"] == 0                      # every sequence was closed


def test_multiple_choice_ranks_by_likelihood(backend):
    tok = ByteTokenizer(CFG.vocab)
    items = [{"context": "abc", "choices": ["de", "xyz", "q"], "answer": 0}, {"context": "k", "choices": ["mm", "n"], "answer": 1}]
    r = multiple_choice(backend, items, tok, length_normalised=False)
    for it, p in zip(items, r["picks"]):
        ctx = tok.encode(it["context"])
        for ch, s in zip(it["choices"], p["scores"]):
            c = tok.encode(ch)
            lp = torch.log_softmax(llama_forward(CFG, backend.W, torch.tensor(ctx + c), None).double(), -1)
            want = sum(float(lp[len(ctx) - 1 + i, c[i]]) for i in range(len(c)))
            assert s == pytest.approx(want, abs=1e-5)
        assert p["pick"] == max(range(len(p["scores"])), key=lambda i: p["scores"][i])
    assert r["accuracy"] in (0.0, 0.5, 1.0) and backend.kv_stats()["sequences"] == 0


def test_exact_match_generates_greedily(backend):
    tok = ByteTokenizer(CFG.vocab)
    prompt = tok.encode("hi")
    backend.begin(7, prompt)
    out, feed = [], prompt
    for _ in range(4):
        nxt = int(backend.forward([7], [feed])[0].argmax())
        out.append(nxt)
        feed = [nxt]
    backend.end(7)
    r = exact_match(backend, [{"prompt": "hi", "answer": tok.decode(out)}, {"prompt": "hi", "answer": "certainly not this"}], tok, max_new_tokens=4)
    assert [row["match"] for row in r["rows"]] == [True, False] and r["exactMatch"] == 0.5


def test_gates_decide_continue_hold_rollback():
    gates = [MetricGate("heldout.loss", "<=", 6.0), MetricGate("mc.accuracy", ">=", 0.25), MetricGate("heldout.loss", "<=", 9.0, rollback_on_fail=True),
             MetricGate("em.exactMatch", ">=", 0.9, required=False)]
    ok = decide({"heldout.loss": 5.7, "mc.accuracy": 0.5, "em.exactMatch": 0.1}, gates)
    assert ok["decisionState"] == "continue" and ok["metricGateCount"] == 4 and ok["passedMetricGateCount"] == 3
    assert decide({"heldout.loss": 6.5, "mc.accuracy": 0.5}, gates)["decisionState"] == "hold"
    assert decide({"heldout.loss": 11.0, "mc.accuracy": 0.5}, gates)["decisionState"] == "rollback"
    assert decide({"heldout.loss": float("nan"), "mc.accuracy": 0.5}, gates)["decisionState"] == "rollback"
    assert decide({"mc.accuracy": 0.5}, gates[:2])["decisionState"] == "hold"           # a missing metric fails its gate
    with pytest.raises(ValueError):
        MetricGate("x", "==", 1.0)


def test_pack_runs_and_becomes_evidence(backend, tmp_path):
    write_token_shard(tmp_path / "h.b2tk", np.random.default_rng(1).integers(0, CFG.vocab, 100))
    ds = TokenDataset(tmp_path / "h.b2tk", seq_len=16)
    pack = EvalPack("benchmark://b200/tiny/checkpoint_eval@1",
                    tasks=[{"name": "heldout", "kind": "perplexity", "dataset": ds, "max_windows": 3},
                           {"name": "mc", "kind": "multiple_choice", "items": [{"context": "ab", "choices": ["c", "d"], "answer": 0}]}],
                    gates=[MetricGate("heldout.loss", "<=", 7.0), MetricGate("heldout.perplexity", "<=", 1000.0), MetricGate("mc.accuracy", ">=", 0.0),
                           MetricGate("heldout.windows", ">=", 3)])
    d = run_pack(pack, backend, ByteTokenizer(CFG.vocab), "checkpoint://b200/tiny/step8")
    assert d["decisionState"] == "continue" and d["metricGateCount"] == d["passedMetricGateCount"] == 4
    assert d["packDigest"] == pack.digest() and d["metrics"]["heldout.windows"] == 3.0
    ev = eval_run_evidence(d, "2026-01-01T00:00:00Z")
    assert ev["evidenceKind"] == "eval_run" and ev["status"] == "completed" and ev["authority"]["noDirectModulePromotion"]
    worse = EvalPack(pack.package_ref, pack.tasks, [MetricGate("heldout.loss", "<=", 1.0)])
    assert worse.digest() != pack.digest()
    d2 = run_pack(worse, backend, ByteTokenizer(CFG.vocab), "checkpoint://b200/tiny/step8")
    assert d2["decisionState"] == "hold" and eval_run_evidence(d2, "2026-01-01T00:00:00Z")["status"] == "needs_review"


def test_command_line_runs_a_pack_on_a_gguf_file(tmp_path, capsys):
    import json
    from openagents_b200.eval.__main__ import main, parse_gate
    from openagents_b200.models.weights import PLAN_Q8_0, save_gguf
    cfg = CFG.with_(d_model=64, n_heads=2, n_kv_heads=1, head_dim=32, ffn=128, vocab=512)
    path = str(tmp_path / "m.gguf")
    save_gguf(path, cfg, random_weights(cfg, 0), PLAN_Q8_0)
    write_token_shard(tmp_path / "v.b2tk", np.random.default_rng(2).integers(0, 512, 200))
    (tmp_path / "mc.jsonl").write_text('{"context": "ab", "choices": ["c", "dd"], "answer": 1}\n')
    rc = main(["--model", path, "--backend", "cpu", "--heldout", str(tmp_path / "v.b2tk"), "--seq-len", "32", "--max-windows", "2",
               "--choices", str(tmp_path / "mc.jsonl"), "--gate", "heldout.loss:<=:8", "--gate", "mc.accuracy:>=:2:optional", "--out", str(tmp_path / "d.json")])
    d = json.loads(capsys.readouterr().out)
    assert rc == 0 and d["decisionState"] == "continue" and d["metricGateCount"] == 2 and d["passedMetricGateCount"] == 1
    assert d["evidence"]["evidenceKind"] == "eval_run" and json.loads((tmp_path / "d.json").read_text())["packDigest"] == d["packDigest"]
    rc = main(["--model", path, "--backend", "cpu", "--heldout", str(tmp_path / "v.b2tk"), "--seq-len", "32", "--max-windows", "1", "--gate", "heldout.loss:<=:1:rollback"])
    assert rc == 4 and json.loads(capsys.readouterr().out)["decisionState"] == "rollback"
    g = parse_gate("a.b:>=:0.5:rollback")
    assert g.rollback_on_fail and g.required and g.threshold == 0.5


def test_task_files_are_checked_line_by_line(tmp_path):
    import json
    from openagents_b200.eval.scorers import load_items
    p = tmp_path / "mc.jsonl"
    good = {"context": "2 + 2 =", "choices": [" 4", " 5"], "answer": 0}
    p.write_text(json.dumps(good) + "\n\n" + json.dumps(good) + "\n")
    assert load_items(str(p), "multiple_choice") == [good, good]
    for line, needle in (("{oops", "not JSON"), ("7", "JSON object"), (json.dumps({**good, "choices": [" 4"]}), "two or more"), (json.dumps({**good, "answer": 2}), "index of one of the 2"),
                         (json.dumps({**good, "answer": True}), "index"), (json.dumps({**good, "context": ""}), "context"), (json.dumps({**good, "choices": [" 4", 5]}), "choices")):
        p.write_text(json.dumps(good) + "\n" + line + "\n")
        with pytest.raises(ValueError, match=rf"mc\.jsonl:2: .*{needle}"):
            load_items(str(p), "multiple_choice")
    p.write_text(json.dumps({"prompt": "Say hi", "answer": "hi"}) + "\n")
    assert len(load_items(str(p), "exact_match")) == 1
    p.write_text(json.dumps({"prompt": "Say hi"}) + "\n")
    with pytest.raises(ValueError, match=r"mc\.jsonl:1: .*prompt"):
        load_items(str(p), "exact_match")
    p.write_text("\n")
    with pytest.raises(ValueError, match="no items"):
        load_items(str(p), "exact_match")
    with pytest.raises(ValueError, match="unknown task kind"):
        load_items(str(p), "essay")
