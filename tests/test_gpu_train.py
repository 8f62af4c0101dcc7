"""Trainer checks on one GPU: gradients against autograd on the fp32 oracle, loss goes down, and
the fused optimizer step against torch.optim.AdamW."""
import math

import pytest
import torch

from openagents_b200.models.config import GPT2_SMALL

pytestmark = pytest.mark.gpu


def _small_cfg():
    from openagents_b200.train.trainer import TrainConfig
    m = GPT2_SMALL.with_(n_layers=2, d_model=128, n_heads=2, n_kv_heads=2, head_dim=64, ffn=512, vocab=1000, context=64)
    return TrainConfig(model=m, global_batch=4, micro_batch=4, seq_len=64, lr=1e-3, weight_decay=0.1, grad_clip=1.0)


def test_gradients_match_oracle_autograd():
    from openagents_b200.oracle.models import gpt2_forward
    from openagents_b200.train.trainer import Trainer, synthetic_batch
    cfg = _small_cfg()
    tr = Trainer(cfg, "cuda:0")
    tok, tgt = synthetic_batch(cfg, 1, 0, 0, "cuda:0")
    tok, tgt = tok.cuda(), tgt.cuda()
    loss = tr.model.forward_backward(tok[0], tgt[0])
    tr.check_status()
    # oracle on the bf16-rounded working parameters
    W = {}
    for sl in tr.slots:
        x = tr.params[sl.offset: sl.offset + sl.numel].view(*sl.shape).float()
        if sl.name == "token_embd.weight":
            x = x[: cfg.model.vocab]
        W[sl.name] = x.clone().requires_grad_(True)
    logits = gpt2_forward(cfg.model, W, tok[0].long())
    ref = torch.nn.functional.cross_entropy(logits.view(-1, cfg.model.vocab), tgt[0].reshape(-1).long())
    ref.backward()
    assert abs(loss.item() - ref.item()) < 2e-2
    worst = 0.0
    for sl in tr.slots:
        g = tr.grads[sl.offset: sl.offset + sl.numel].view(*sl.shape)
        if sl.name == "token_embd.weight":
            assert float(g[cfg.model.vocab:].abs().max()) == 0.0       # padded vocabulary rows get no gradient
            g = g[: cfg.model.vocab]
        r = W[sl.name].grad
        rel = (g - r).norm().item() / (r.norm().item() + 1e-12)
        worst = max(worst, rel)
        assert rel < 0.08, (sl.name, rel)
    assert worst > 0.0


def test_loss_decreases_and_optimizer_matches_adamw():
    from openagents_b200.train.trainer import Trainer, synthetic_batch
    cfg = _small_cfg()
    tr = Trainer(cfg, "cuda:0")
    tok, tgt = synthetic_batch(cfg, tr.accum, 0, 0, "cuda:0")
    tok, tgt = tok.cuda(), tgt.cuda()
    # reference AdamW on the same gradients for the first step
    tr.model.forward_backward(tok[0], tgt[0])
    g0 = tr.grads.clone()
    w0 = tr.master.clone()
    gn = g0.norm().item()
    tr.optimizer_step()
    tr.check_status()
    assert abs(tr.grad_norm() - gn) < 1e-3 * gn
    clip = min(1.0, cfg.grad_clip / (gn + 1e-6))
    p = w0.clone().requires_grad_(True)
    dec, nod = p[: tr.decay_end], p[tr.decay_end:]
    opt = torch.optim.AdamW([{"params": [p], "weight_decay": 0.0}], lr=cfg.lr, betas=cfg.betas, eps=cfg.eps)
    p.grad = g0 * clip
    opt.step()
    with torch.no_grad():
        p[: tr.decay_end] -= cfg.lr * cfg.weight_decay * w0[: tr.decay_end]
    assert torch.allclose(tr.master, p.detach(), atol=1e-6, rtol=1e-5)
    assert torch.equal(tr.params, tr.master.bfloat16())
    assert float(tr.grads.abs().max()) == 0.0
    # a few steps on one fixed batch: the loss must fall well below ln(V)
    losses = []
    for _ in range(12):
        losses.append(tr.train_step(tok, tgt).item())
    assert losses[-1] < losses[0] - 0.5 and losses[0] < math.log(cfg.model.vocab) + 0.5
    tr.check_status()


def test_masked_targets_match_oracle_and_loader_feeds_the_trainer(tmp_path):
    """Instruction-tuning shape: half of the targets masked (-1), loss and gradients averaged over the rest; then batches
    from token shards through the prefetching loader."""
    import numpy as np
    from openagents_b200.data import BatchLoader, TokenDataset, write_token_shard
    from openagents_b200.oracle.models import gpt2_forward
    from openagents_b200.train.trainer import Trainer, synthetic_batch
    cfg = _small_cfg()
    tr = Trainer(cfg, "cuda:0")
    tok, tgt = synthetic_batch(cfg, 1, 0, 0, "cuda:0")
    tok, tgt = tok.cuda(), tgt.cuda()
    keep = torch.rand(tgt.shape, device="cuda", generator=torch.Generator("cuda").manual_seed(1)) < 0.5
    tgt = torch.where(keep, tgt, torch.full_like(tgt, -1))
    n_valid = int(keep.sum())
    loss = tr.model.forward_backward(tok[0], tgt[0], denom=float(n_valid))
    tr.check_status()
    W = {}
    for sl in tr.slots:
        x = tr.params[sl.offset: sl.offset + sl.numel].view(*sl.shape).float()
        if sl.name == "token_embd.weight":
            x = x[: cfg.model.vocab]
        W[sl.name] = x.clone().requires_grad_(True)
    logits = gpt2_forward(cfg.model, W, tok[0].long())
    ref = torch.nn.functional.cross_entropy(logits.view(-1, cfg.model.vocab), tgt[0].reshape(-1).long(), ignore_index=-1)
    ref.backward()
    assert abs(loss.item() - ref.item()) < 2e-2
    for sl in tr.slots:
        g = tr.grads[sl.offset: sl.offset + sl.numel].view(*sl.shape)
        if sl.name == "token_embd.weight":
            g = g[: cfg.model.vocab]
        r = W[sl.name].grad
        assert (g - r).norm().item() / (r.norm().item() + 1e-12) < 0.08, sl.name
    tr.grads.zero_()

    # a periodic token stream with the odd positions masked: learnable, and n_valid is half of every batch
    period = np.arange(37) * 13 % 1000
    stream = np.tile(period, 400)
    mask = (np.arange(stream.size) % 2).astype(np.uint8)
    write_token_shard(tmp_path / "a.b2tk", stream[:9000], mask[:9000])
    write_token_shard(tmp_path / "b.b2tk", stream[9000:], mask[9000:])
    ds = TokenDataset([tmp_path / "a.b2tk", tmp_path / "b.b2tk"], cfg.seq_len)
    ld = BatchLoader(ds, tr.accum, cfg.micro_batch, seed=3)
    losses = []
    for _ in range(30):
        t, g, nv, _ = ld.next()
        assert t.is_pinned() and nv == t.numel() // 2
        losses.append(tr.train_step(t.cuda(non_blocking=True), g.cuda(non_blocking=True), nv).item())
    tr.check_status()
    assert losses[0] > 5.0 and losses[-1] < losses[0] - 2.0, losses


def test_sft_lane_on_the_trainer_with_resume_drill(tmp_path):
    """The instruction-tuning lane end to end on the GPU trainer: masked shard, cosine schedule, checkpoint at step 3, a fresh
    trainer resumed from it; the restored state is bit-identical and the resumed losses agree with the uninterrupted run."""
    import dataclasses
    from openagents_b200.data import BatchLoader, ByteBpe, TokenDataset
    from openagents_b200.train import sft
    from openagents_b200.train.trainer import Trainer
    records = [{"messages": [{"role": "user", "content": f"What is {a} plus {b}?"}, {"role": "assistant", "content": f"It is {a + b}."}]}
               for a in range(6) for b in range(6)]
    text = "\n".join(m["content"] for r in records for m in r["messages"]).encode()
    tok = ByteBpe.train(text, 64, special=sft.SPECIAL_TOKENS)
    corpus = sft.build_corpus(records, tok, "sums@v1")
    sft.pack(corpus, tmp_path / "sft.b2tk", repeat=3)
    cfg = dataclasses.replace(_small_cfg(), total_steps=9, lr=3e-3)
    assert tok.vocab_size <= cfg.model.vocab
    ds = TokenDataset(tmp_path / "sft.b2tk", cfg.seq_len)
    rep = sft.run_lane(lambda: Trainer(cfg, "cuda:0"), lambda start: BatchLoader(ds, 1, cfg.micro_batch, seed=2, start_batch=start),
                       steps=9, checkpoint_at=3, ckpt_dir=str(tmp_path / "drill"), corpus_manifest=corpus.manifest, device="cuda:0",
                       loss_tolerance=2e-2)
    d = rep["resumeDrill"]
    assert rep["lossImproved"] and rep["lastLoss"] < rep["firstLoss"] - 0.5, rep["stepReceipts"]
    assert d["restoredStateBitExact"] and d["sameBatchesAfterResume"] and d["postResumeLossesAgree"], d
    assert all(0 < r["trainableTokens"] < 4 * 64 for r in rep["stepReceipts"])


def test_dpo_gradients_match_autograd_and_preferences_are_learned():
    """Preference optimisation through the fused cross-entropy's per-row factors: gradients against autograd of the pair loss on
    the fp32 oracle, then a few steps on fixed pairs (the loss falls below ln 2, every pair ends up ranked correctly)."""
    import dataclasses
    import math
    from openagents_b200.data import ByteBpe
    from openagents_b200.oracle.models import gpt2_forward
    from openagents_b200.train import dpo, sft
    from openagents_b200.train.trainer import Trainer
    cfg = dataclasses.replace(_small_cfg(), lr=2e-3, weight_decay=0.0)
    tok = ByteBpe.train(b"What is the capital? Paris. London. red green blue yes no maybe", 10, special=sft.SPECIAL_TOKENS)
    pairs = [{"messages": [{"role": "user", "content": f"Question {i}: red or blue?"}], "chosen": "red " * (1 + i % 2), "rejected": "blue"} for i in range(2)]
    tokens, targets, _ = dpo.build_preference_batch(pairs, tok, cfg.seq_len)
    assert tokens.shape[0] == cfg.micro_batch
    tokens, targets = tokens[None].cuda(), targets[None].cuda()
    tr = Trainer(cfg, "cuda:0")
    d = dpo.DpoTrainer(tr, beta=0.5)
    ref = d.reference_logps(tokens, targets)
    tr.check_status()
    assert ref.shape == (1, 4) and bool((ref < 0).all())
    shifted = ref + torch.tensor([[0.3, -0.2, 0.1, 0.4]], device="cuda")          # margins away from zero, so both signs of factor matter
    stats = {}
    loss = tr.model.forward_backward(tokens[0], targets[0], row_scale_fn=lambda rows: dpo.dpo_row_scales(rows, shifted[0], 0.5, 2, stats))
    tr.check_status()
    W = {}
    for sl in tr.slots:
        x = tr.params[sl.offset: sl.offset + sl.numel].view(*sl.shape).float()
        if sl.name == "token_embd.weight":
            x = x[: cfg.model.vocab]
        W[sl.name] = x.clone().requires_grad_(True)
    logits = gpt2_forward(cfg.model, W, tokens[0].long())
    nll = torch.nn.functional.cross_entropy(logits.view(-1, cfg.model.vocab), targets[0].reshape(-1).long(), ignore_index=-1, reduction="none")
    pol = -nll.view(4, -1).sum(1)
    m = 0.5 * ((pol[:2] - shifted[0, :2]) - (pol[2:] - shifted[0, 2:]))
    want = torch.nn.functional.softplus(-m).mean()
    want.backward()
    assert abs(loss.item() - want.item()) < 2e-2
    for sl in tr.slots:
        g = tr.grads[sl.offset: sl.offset + sl.numel].view(*sl.shape)
        if sl.name == "token_embd.weight":
            g = g[: cfg.model.vocab]
        r = W[sl.name].grad
        assert (g - r).norm().item() / (r.norm().item() + 1e-12) < 0.08, sl.name
    tr.grads.zero_()
    losses = [d.train_step(tokens, targets, ref).item() for _ in range(25)]
    tr.check_status()
    assert abs(losses[0] - math.log(2.0)) < 0.05                                  # policy == reference: every margin is zero
    assert losses[-1] < 0.35 and d.reward_accuracy() == 1.0, losses


def test_launcher_lanes_from_files(tmp_path, capsys):
    """``b200-train`` end to end on files: pre-training from prepared shards (and a resumed run continuing the data stream), the
    instruction-tuning lane and the preference lane."""
    import json
    from openagents_b200.data.__main__ import main as data_main
    from openagents_b200.train.launcher import main as train_main
    (tmp_path / "c.txt").write_text("\n\n".join(f"Document {i} tells of river {i % 7}, its boats, mills and the grain market of town {i}." for i in range(400)))
    assert data_main(["prepare", "--text", str(tmp_path / "c.txt"), "--out", str(tmp_path / "d"), "--merges", "64", "--no-refine"]) == 0
    capsys.readouterr()
    common = ["--layers", "2", "--global-batch", "8", "--micro-batch", "4", "--seq-len", "64", "--lr", "1e-3"]
    shards = [str(p) for p in sorted((tmp_path / "d").glob("train-*.b2tk"))]
    train_main(common + ["--steps", "4", "--data", *shards, "--ckpt-dir", str(tmp_path / "ck")])
    recs = [json.loads(x) for x in capsys.readouterr().out.splitlines() if x.startswith("{")]
    steps = [r for r in recs if r.get("event") == "step"]
    assert recs[0]["event"] == "data" and len(steps) == 4 and steps[-1]["loss"] < steps[0]["loss"]
    train_main(common + ["--steps", "1", "--data", *shards, "--resume", str(tmp_path / "ck" / "step00000004")])
    recs = [json.loads(x) for x in capsys.readouterr().out.splitlines() if x.startswith("{")]
    assert [r["step"] for r in recs if r.get("event") == "step"] == [5]
    with open(tmp_path / "chat.jsonl", "w") as f:
        for a in range(5):
            for b in range(5):
                f.write(json.dumps({"messages": [{"role": "user", "content": f"What is {a} plus {b}?"}, {"role": "assistant", "content": f"It is {a + b}."}]}) + "\n")
    train_main(common + ["--lane", "sft", "--steps", "6", "--sft-records", str(tmp_path / "chat.jsonl"), "--sft-merges", "32", "--ckpt-dir", str(tmp_path / "sft"),
                         "--report", str(tmp_path / "sft.json"), "--export-gguf", str(tmp_path / "tuned.gguf")])
    capsys.readouterr()
    rep = json.loads((tmp_path / "sft.json").read_text())
    assert rep["completedSteps"] == 6 and rep["lossImproved"] and rep["resumeDrill"]["restoredStateBitExact"] and rep["resumeDrill"]["checkpointAtStep"] == 2
    # the tuned checkpoint carries its tokenizer and goes straight into the evaluator on the GPU backend
    from openagents_b200.eval.__main__ import main as eval_main
    (tmp_path / "em.jsonl").write_text(json.dumps({"prompt": "<|user|>\nWhat is 1 plus 1?<|end|>\n<|assistant|>\n", "answer": "It is 2."}) + "\n")
    rc = eval_main(["--model", str(tmp_path / "tuned.gguf"), "--backend", "cuda", "--exact", str(tmp_path / "em.jsonl"), "--max-new-tokens", "8",
                    "--gate", "em.exactMatch:>=:0:optional"])
    d = json.loads(capsys.readouterr().out.splitlines()[-1])
    assert rc == 0 and d["backend"] == "cuda" and d["tasks"]["em"]["items"] == 1
    with open(tmp_path / "pairs.jsonl", "w") as f:
        for i in range(6):
            f.write(json.dumps({"messages": [{"role": "user", "content": f"Pick a colour, number {i}."}], "chosen": "red", "rejected": "blue"}) + "\n")
    train_main(common + ["--lane", "dpo", "--steps", "6", "--dpo-pairs", str(tmp_path / "pairs.jsonl"), "--sft-merges", "16", "--beta", "0.5"])
    steps = [json.loads(x) for x in capsys.readouterr().out.splitlines() if x.startswith("{")]
    assert len(steps) == 6 and abs(steps[0]["pair_loss"] - 0.693) < 0.05 and steps[-1]["pair_loss"] < steps[0]["pair_loss"]


def test_gpt2_checkpoint_is_served_on_the_training_kernels(tmp_path):
    """A trained GPT-2-shape checkpoint through the serving interface on the GPU (recompute on the trainer's forward kernels)
    against the fp32 oracle backend; then the same backend over a live trainer's buffers (on-policy sampling)."""
    from openagents_b200.data import ByteBpe
    from openagents_b200.serve.backend import open_backend
    from openagents_b200.serve.generation import SamplingParams, Scheduler
    from openagents_b200.serve.gpt2_backend import Gpt2CudaBackend
    from openagents_b200.serve.server import load_tokenizer
    from openagents_b200.train.trainer import Trainer, synthetic_batch
    cfg = _small_cfg()
    tr = Trainer(cfg, "cuda:0")
    tok, tgt = synthetic_batch(cfg, tr.accum, 0, 0, "cuda:0")
    tok, tgt = tok.cuda(), tgt.cuda()
    for _ in range(3):
        tr.train_step(tok, tgt)
    bpe = ByteBpe.train(b"the cat sat on the mat " * 8, 20, special=["<|end|>"])
    path = str(tmp_path / "tuned.gguf")
    tr.export_gguf(path, tokenizer=bpe)
    gpu, cpu = open_backend(path, "cuda", max_num_seqs=4), open_backend(path, "cpu")
    assert type(gpu).__name__ == "Gpt2CudaBackend" and gpu.max_context == 64
    seqs = {1: [5, 17, 200, 3, 42, 42, 9], 2: [7] * 30, 3: [999, 0, 1], 4: [11, 12], 5: [400, 500, 600, 700]}       # five sequences: two groups of rows
    for b in (gpu, cpu):
        for s, t in seqs.items():
            b.begin(s, t)
    a = gpu.forward(list(seqs), list(seqs.values()))
    b = cpu.forward(list(seqs), list(seqs.values()))
    assert a.shape == b.shape == (5, cfg.model.vocab)
    assert (a - b).abs().max().item() < 0.08 * b.abs().max().item() + 0.05
    la, lb = gpu.score(1, [8, 9, 10], [9, 10, -1]), cpu.score(1, [8, 9, 10], [9, 10, -1])
    assert la[2] == 0.0 and max(abs(x - y) for x, y in zip(la, lb)) < 0.1
    gpu.truncate(1, 7)
    assert gpu.seq_len(1) == 7 and len(gpu.verify(1, [8, 9])) == 2
    loaded, _ = load_tokenizer(path, cfg.model.vocab)
    sch = Scheduler(open_backend(path, "cuda", max_num_seqs=4), loaded, max_num_seqs=4)
    reqs = [sch.submit(loaded.encode("the cat"), SamplingParams(max_tokens=6)) for _ in range(3)]
    sch.run_until_done(reqs)
    assert all(1 <= len(r.output) <= 6 for r in reqs) and reqs[0].output == reqs[1].output        # greedy: same prompt, same answer
    # on-policy: the backend reads the trainer's own buffers, so an optimizer step changes what it samples from
    live = Gpt2CudaBackend.over_trainer(tr)
    live.begin(1, [1, 2, 3])
    before = live.forward([1], [[1, 2, 3]])
    ref = open_backend(path, "cpu")
    ref.begin(1, [1, 2, 3])
    assert (before - ref.forward([1], [[1, 2, 3]])).abs().max().item() < 0.1
    for _ in range(3):
        tr.train_step(tok, tgt)
    live.truncate(1, 0)
    after = live.forward([1], [[1, 2, 3]])
    assert (after - before).abs().max().item() > 1e-3
    tr.check_status()


def test_rollout_policy_gradient_raises_the_reward():
    """On-policy roll-outs from the trainer's own weights through the scheduler, graded, group-relative advantages, one
    optimizer step per round through the per-row factors: the mean reward of a dense toy reward goes up."""
    import dataclasses
    from openagents_b200.serve.generation import ByteTokenizer
    from openagents_b200.train.rollout import RolloutTrainer
    from openagents_b200.train.trainer import Trainer
    cfg = dataclasses.replace(_small_cfg(), lr=3e-3, weight_decay=0.0, global_batch=8, micro_batch=4)
    tr = Trainer(cfg, "cuda:0")
    assert tr.accum == 2

    def reward(task, text, ids):                      # the share of sampled ids below 128: dense, and about 1/8 at the start
        return sum(i < 128 for i in ids) / max(1, len(ids))

    rt = RolloutTrainer(tr, ByteTokenizer(cfg.model.vocab), reward_fn=reward, group_size=4, max_new_tokens=8, temperature=1.0, top_k=64, seed=1)
    tasks = [{"prompt": "ab"}, {"prompt": "cd"}]
    recs = [rt.step(tasks) for _ in range(30)]
    tr.check_status()
    first = sum(r["meanReward"] for r in recs[:5]) / 5
    last = sum(r["meanReward"] for r in recs[-5:]) / 5
    assert all(r["rollouts"] == 8 for r in recs) and any(r["trainedRows"] > 0 for r in recs)
    assert last > first + 0.2, (first, last, [round(r["meanReward"], 2) for r in recs])
    assert rt.backend.kv_stats()["sequences"] == 0
