"""Instruction-tuning lane: template, loss mask, corpus manifest, masked shard, and the lane report with its resume drill
(on a small CPU trainer that has the same interface as the GPU one)."""
import os

import pytest
import torch
import torch.nn.functional as F

from openagents_b200.data import BatchLoader, ByteBpe, TokenDataset
from openagents_b200.train import sft

RECORDS = [
    {"messages": [{"role": "system", "content": "You answer briefly."}, {"role": "user", "content": "What is two plus two?"},
                  {"role": "assistant", "content": "Four."}]},
    {"messages": [{"role": "user", "content": "Name a colour."}, {"role": "assistant", "content": "Blue."},
                  {"role": "user", "content": "Another one."}, {"role": "assistant", "content": "Green."}]},
    {"messages": [{"role": "user", "content": "Say hello."}, {"role": "assistant", "content": "Hello there."}]},
]


def _tok():
    text = " ".join(m["content"] for r in RECORDS for m in r["messages"]).encode()
    return ByteBpe.train(text * 3, 30, special=sft.SPECIAL_TOKENS)


def test_mask_covers_exactly_the_assistant_turns():
    tok = _tok()
    rows = sft.generation_mask_fixture(RECORDS[1]["messages"], tok)
    trained = "".join(r["text"] for r in rows if r["trainable"])
    assert trained == "Blue.<|end|>Green.<|end|>"
    assert "".join(r["text"] for r in rows) == sft.render_text(RECORDS[1]["messages"])
    assert sft.generation_prompt(RECORDS[2]["messages"][:1]).endswith("<|assistant|>\n")
    with pytest.raises(ValueError):
        sft.render_example([{"role": "user", "content": "no answer"}], tok)
    with pytest.raises(ValueError):
        sft.render_example([{"role": "tool", "content": "x"}, {"role": "assistant", "content": "y"}], tok)


def test_corpus_manifest_commits_to_records_and_template(tmp_path):
    tok = _tok()
    c = sft.build_corpus(RECORDS, tok, "example_corpus@v1")
    m = c.manifest
    assert m["recordCount"] == 3 and m["totalTrainableTokens"] + m["totalMaskedTokens"] == len(c.ids)
    assert m["totalTrainableTokens"] == int(c.mask.sum()) > 0
    assert m["template"]["templateDigest"] == sft.template_digest() and m["manifestDigest"].startswith("sha256:")
    changed = [dict(RECORDS[0]), *RECORDS[1:]]
    changed[0] = {"messages": RECORDS[0]["messages"][:-1] + [{"role": "assistant", "content": "Five."}]}
    assert sft.build_corpus(changed, tok, "example_corpus@v1").manifest["manifestDigest"] != m["manifestDigest"]
    info = sft.pack(c, tmp_path / "sft.b2tk", repeat=4)
    assert info["masked"] and info["tokens"] == 4 * len(c.ids)
    ds = TokenDataset(tmp_path / "sft.b2tk", seq_len=16)
    _, tgt, n = ds.window(0)
    assert n == int(c.mask[1:17].sum()) and [t for t in tgt.tolist() if t >= 0] == [int(i) for i, k in zip(c.ids[1:17], c.mask[1:17]) if k]


def test_cosine_schedule_has_the_stated_floor():
    assert sft.cosine_lr(0, 8, 1.0) == pytest.approx(1.0)
    assert sft.cosine_lr(8, 8, 1.0) == pytest.approx(0.1)
    assert sft.cosine_lr(4, 8, 1.0, ratio_bps=0) == pytest.approx(0.5)
    assert sft.cosine_lr(0, 8, 1.0, warmup_steps=4) == pytest.approx(0.25)


class TinyTrainer:
    """Embedding -> linear LM with AdamW on the CPU; the lane only needs the interface."""

    def __init__(self, vocab, total_steps):
        g = torch.Generator().manual_seed(0)
        self.emb = (torch.randn(vocab, 16, generator=g) * 0.1).requires_grad_(True)
        self.out = (torch.randn(16, vocab, generator=g) * 0.1).requires_grad_(True)
        self.opt = torch.optim.AdamW([self.emb, self.out], lr=0.05)
        self.step_count, self.total = 0, total_steps

    @property
    def master(self):
        return torch.cat([self.emb.detach().reshape(-1), self.out.detach().reshape(-1)])

    @property
    def m(self):
        st = self.opt.state
        return torch.cat([st[p]["exp_avg"].reshape(-1) for p in (self.emb, self.out)]) if st else None

    v = None

    def train_step(self, tok, tgt, n_valid=None):
        for g in self.opt.param_groups:
            g["lr"] = sft.cosine_lr(self.step_count, self.total, 0.05)
        logits = self.emb[tok.reshape(-1)] @ self.out
        loss = F.cross_entropy(logits, tgt.reshape(-1), ignore_index=-1)
        self.opt.zero_grad()
        loss.backward()
        self.opt.step()
        self.step_count += 1
        return loss.detach()

    def save_checkpoint(self, d):
        os.makedirs(d, exist_ok=True)
        torch.save({"emb": self.emb.detach(), "out": self.out.detach(), "opt": self.opt.state_dict(), "step": self.step_count}, os.path.join(d, "s.pt"))

    def load_checkpoint(self, d):
        s = torch.load(os.path.join(d, "s.pt"))
        with torch.no_grad():
            self.emb.copy_(s["emb"])
            self.out.copy_(s["out"])
        self.opt.load_state_dict(s["opt"])
        self.step_count = s["step"]


def test_lane_report_and_resume_drill(tmp_path):
    tok = _tok()
    c = sft.build_corpus(RECORDS, tok, "example_corpus@v1")
    sft.pack(c, tmp_path / "sft.b2tk", repeat=8)
    ds = TokenDataset(tmp_path / "sft.b2tk", seq_len=16)
    rep = sft.run_lane(lambda: TinyTrainer(tok.vocab_size, 8), lambda start: BatchLoader(ds, 1, 4, seed=1, start_batch=start, pin=False),
                       steps=8, checkpoint_at=3, ckpt_dir=str(tmp_path / "ck"), corpus_manifest=c.manifest)
    assert rep["completedSteps"] == 8 and rep["lossImproved"] and rep["lastLoss"] < rep["firstLoss"]
    d = rep["resumeDrill"]
    assert d == {**d, "checkpointAtStep": 3, "resumedSteps": 5, "restoredStateBitExact": True, "sameBatchesAfterResume": True,
                 "postResumeLossesAgree": True}
    assert d["postResumeLossesBitExact"]                     # the CPU stand-in is deterministic
    assert all(0 < r["trainableTokens"] < 64 for r in rep["stepReceipts"])
    assert rep["corpus"]["manifestDigest"] == c.manifest["manifestDigest"] and rep["reportDigest"].startswith("sha256:")
    with pytest.raises(ValueError):
        sft.run_lane(lambda: None, lambda s: None, steps=4, checkpoint_at=4, ckpt_dir="x", corpus_manifest=c.manifest)


def test_trainer_schedules_cosine_wsd_constant():
    from openagents_b200.train.trainer import TrainConfig, lr_schedule
    cos = TrainConfig(lr=1.0, warmup_steps=2, total_steps=10)
    assert [round(lr_schedule(cos, s), 4) for s in (0, 1, 2, 6, 10, 50)] == [0.5, 1.0, 1.0, 0.55, 0.1, 0.1]
    assert lr_schedule(cos, 6) == pytest.approx(sft.cosine_lr(6, 10, 1.0, 1000, warmup_steps=2))
    wsd = TrainConfig(lr=1.0, warmup_steps=2, total_steps=20, schedule="wsd", decay_fraction=0.25)
    lrs = [lr_schedule(wsd, s) for s in range(22)]
    assert lrs[0] == 0.5 and all(x == 1.0 for x in lrs[1:15]) and lrs[15] < 1.0 and lrs[19] == pytest.approx(0.1) and lrs[21] == pytest.approx(0.1)
    assert all(a > b for a, b in zip(lrs[14:19], lrs[15:20]))                      # strictly decreasing through the decay phase
    assert lr_schedule(TrainConfig(lr=2.0, total_steps=10, schedule="constant"), 7) == 2.0 and lr_schedule(TrainConfig(lr=2.0), 99) == 2.0
    with pytest.raises(ValueError):
        lr_schedule(TrainConfig(schedule="step"), 0)


def test_distillation_records_from_a_teacher_backend_feed_the_lane(tmp_path):
    """Sequence-level distillation: the teacher (the fp32 CPU backend here) answers captured prompts through the scheduler, the
    answers become chat records, the student's lane trains on them; both are then scored on the same items."""
    from openagents_b200.models.config import ModelConfig
    from openagents_b200.models.weights import random_weights
    from openagents_b200.serve.backend import CpuBackend
    from openagents_b200.train import distill
    text = " ".join(m["content"] for r in RECORDS for m in r["messages"]).encode()
    tok = ByteBpe.train(text * 3, 30, special=sft.SPECIAL_TOKENS)

    class Tok:                                   # the serving tokenizer interface over the same BPE
        eos_id = tok.special_ids["<|end|>"]
        vocab_size = 400
        encode, decode = staticmethod(tok.encode), staticmethod(lambda ids: tok.decode([i for i in ids if i < tok.vocab_size]))
    cfg = ModelConfig(name="teacher", arch="llama", vocab=400, d_model=32, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=8, ffn=64, context=256)
    teacher = CpuBackend(cfg, {k: v.float() for k, v in random_weights(cfg, 3).items()})
    prompts = ["What is two plus two?", "Name a colour.", "Say hello."]
    recs, man = distill.teacher_records(teacher, Tok, prompts, max_new_tokens=6)
    assert man["prompts"] == 3 and man["records"] + man["dropped"] == 3 and man["records"] >= 1 and man["inputDistributionDigest"].startswith("sha256:")
    assert all(r["messages"][-1]["role"] == "assistant" and r["messages"][-1]["content"] and "<|end|>" not in r["messages"][-1]["content"] for r in recs)
    again, man2 = distill.teacher_records(teacher, Tok, prompts, max_new_tokens=6)
    assert man2["recordsDigest"] == man["recordsDigest"]                      # greedy teacher: the capture is reproducible
    many, man3 = distill.teacher_records(teacher, Tok, prompts[:1], max_new_tokens=6, answers_per_prompt=4, temperature=1.0, seed=5)
    assert man3["answersPerPrompt"] == 4 and 1 <= man3["records"] <= 4
    # the student lane consumes the records unchanged
    c = sft.build_corpus(recs, tok, "distilled@v1")
    sft.pack(c, tmp_path / "d.b2tk", repeat=40)
    ds = TokenDataset(tmp_path / "d.b2tk", seq_len=16)
    rep = sft.run_lane(lambda: TinyTrainer(tok.vocab_size, 6), lambda start: BatchLoader(ds, 1, 4, seed=1, start_batch=start, pin=False),
                       steps=6, checkpoint_at=2, ckpt_dir=str(tmp_path / "ck"), corpus_manifest=c.manifest)
    assert rep["lossImproved"] and rep["corpus"]["datasetIdentity"] == "distilled@v1"
    q = distill.quality_delta(teacher, teacher, Tok, Tok, [{"prompt": sft.generation_prompt([{"role": "user", "content": prompts[0]}]),
                                                            "answer": recs[0]["messages"][-1]["content"]}], max_new_tokens=6)
    assert q["qualityDeltaBps"] == 0 and q["baselineQualityScoreBps"] == q["candidateQualityScoreBps"] and q["items"] == 1


def test_record_files_are_checked_line_by_line(tmp_path):
    """A tuning file is user data: a bad line is reported with the file and the line number, before any training starts."""
    import json
    good = {"messages": [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "hello"}]}
    p = tmp_path / "records.jsonl"
    p.write_text(json.dumps(good) + "\n\n" + json.dumps(good) + "\n")
    assert len(sft.load_records(str(p))) == 2
    cases = [("{not json", "not JSON"), ("[1, 2]", "a record is a JSON object"), ('{"messages": "hi"}', "non-empty list of messages"),
             ('{"messages": [{"role": "wizard", "content": "x"}]}', r"messages\[0\]"), ('{"messages": [{"role": "user", "content": 5}]}', r"messages\[0\]"),
             ('{"messages": [5]}', r"messages\[0\]"), ('{"messages": [{"role": "user", "content": "only a question"}]}', "assistant")]
    for line, needle in cases:
        p.write_text(json.dumps(good) + "\n" + line + "\n")
        with pytest.raises(ValueError, match=rf"records\.jsonl:2: .*{needle}"):
            sft.load_records(str(p))
    p.write_text("\n\n")
    with pytest.raises(ValueError, match="no records"):
        sft.load_records(str(p))
    pair = {"messages": [{"role": "user", "content": "red or blue?"}], "chosen": "red", "rejected": "blue"}
    p.write_text(json.dumps(pair) + "\n")
    assert sft.load_records(str(p), preference=True) == [pair]
    for patch, needle in (({"chosen": ""}, "chosen"), ({"rejected": 5}, "rejected"), ({"messages": []}, "messages")):
        p.write_text(json.dumps({**pair, **patch}) + "\n")
        with pytest.raises(ValueError, match=rf"records\.jsonl:1: .*{needle}"):
            sft.load_records(str(p), preference=True)
    with pytest.raises(ValueError, match="record 0"):
        sft.build_corpus([7], None, "x")
