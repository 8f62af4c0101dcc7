"""Local-update rounds: admission rules, aggregation, the outer optimizer, and two gloo replicas that end every round on
identical parameters while exchanging one vector per round."""
import os

import pytest
import torch

from openagents_b200.train import diloco as dl


class _Quad:
    """A trainer stand-in: minimises 0.5 |theta - target|^2 on noisy gradients with plain SGD."""

    def __init__(self, dim, target, seed, lr=0.2):
        self.master = torch.zeros(dim)
        self.target, self.lr, self.g = target, lr, torch.Generator().manual_seed(seed)

    def train_step(self, tok, tgt):
        grad = self.master - self.target + 0.05 * torch.randn(self.master.shape, generator=self.g)
        self.master = self.master - self.lr * grad
        return 0.5 * float(((self.master - self.target) ** 2).sum())

    def set_master(self, t):
        self.master = t.clone()


def _batches(n, width=8):
    return [(torch.zeros(2, width, dtype=torch.long), torch.zeros(2, width, dtype=torch.long)) for _ in range(n)]


def test_admission_aggregation_and_outer_step():
    cfg = dl.DilocoConfig(inner_steps=4, min_participants=2, min_weight_fraction=0.6, max_staleness_windows=1)
    tags = dict((t[0], t[1]) for t in cfg.window_tags(3, "ckpt.3"))
    assert tags["sync_profile"] == "diloco" and tags["planned_local_steps"] == "4" and tags["base_checkpoint"] == "ckpt.3" and tags["round"] == "3"
    mk = lambda who, rnd, base, delta, tokens, steps=4: dl.LocalUpdate(who, rnd, base, torch.tensor(delta), steps, tokens)
    ups = [mk("a", 3, "ckpt.3", [1.0, 0.0], 300), mk("b", 3, "ckpt.3", [0.0, 2.0], 100), mk("c", 2, "ckpt.2", [9.0, 9.0], 100),
           mk("d", 1, "ckpt.1", [9.0, 9.0], 100), mk("e", 3, "ckpt.3", [float("nan"), 0.0], 100), mk("f", 3, "ckpt.WRONG", [1.0, 1.0], 100),
           mk("g", 3, "ckpt.3", [1.0, 1.0], 100, steps=0)]
    adm = dl.admit_updates(ups, cfg, 3, "ckpt.3", planned_participants=4)
    st = {d["participant"]: d["status"] for d in adm["decisions"]}
    assert st == {"a": "accepted", "b": "accepted", "c": "replay_required", "d": "sync_reentry", "e": "rejected", "f": "replay_required", "g": "rejected"}
    assert [u.participant for u in adm["admitted"]] == ["a", "b"] and adm["sealable"]
    g = dl.aggregate(adm["admitted"], cfg)                                 # token-weighted: 0.75 a + 0.25 b
    assert torch.allclose(g, torch.tensor([0.75, 0.5]))
    assert torch.allclose(dl.aggregate(adm["admitted"], dl.DilocoConfig(aggregation_rule="uniform_avg")), torch.tensor([0.5, 1.0]))
    strict = dl.admit_updates(ups[:1], dl.DilocoConfig(min_participants=2), 3, "ckpt.3", planned_participants=4)
    assert not strict["sealable"] and strict["blockers"] == ["min_participants_not_met", "min_weight_fraction_not_met"]
    # Nesterov: v1 = g, step = lr (mu v1 + g); v2 = mu v1 + g2
    opt = dl.OuterOptimizer(dl.DilocoConfig(outer_lr=0.5, outer_momentum=0.9))
    th = opt.step(torch.zeros(2), torch.tensor([1.0, 0.0]))
    assert torch.allclose(th, torch.tensor([-0.5 * 1.9, 0.0]))
    th2 = opt.step(th, torch.tensor([1.0, 0.0]))
    assert torch.allclose(th2, th - 0.5 * (0.9 * 1.9 + 1.0) * torch.tensor([1.0, 0.0]))
    saved = opt.state_dict()
    again = dl.OuterOptimizer(opt.cfg)
    again.load_state_dict(saved)
    assert torch.equal(again.step(th2, torch.ones(2)), opt.step(th2, torch.ones(2)))
    with pytest.raises(ValueError):
        dl.aggregate([], cfg)


def _replica(rank, world, port, out):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    target = torch.tensor([1.0, -2.0, 3.0, 0.5])
    tr = _Quad(4, target, seed=10 + rank)
    rep = dl.DilocoReplica(tr, dl.DilocoConfig(inner_steps=5, outer_lr=0.7, outer_momentum=0.5, min_participants=2), f"replica.{rank}")
    errs = []
    for rnd in range(6):
        rec = rep.run_round(_batches(5))
        errs.append(float((tr.master - target).norm()))
        assert rec["sealed"] and rec["participants"] == 2 and rec["localSteps"] == 5 and rec["tokensAllReplicas"] == 2 * 5 * 16
    # a round in which rank 1's local training diverges (not finite): one valid participant of the two required
    if rank == 1:
        tr.lr = float("nan")
    rec = rep.run_round(_batches(5))
    torch.save({"master": tr.master, "errs": errs, "last": rec, "rounds": rep.round_index, "base": rep.base_checkpoint}, f"{out}/r{rank}.pt")
    dist.destroy_process_group()


def test_two_replicas_stay_identical_and_converge(tmp_path):
    import socket
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_replica, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    a, b = torch.load(tmp_path / "r0.pt"), torch.load(tmp_path / "r1.pt")
    assert a["errs"][-1] < 0.2 * a["errs"][0] and a["errs"][-1] < 0.3                 # converged towards the target
    # the poisoned round had one valid participant of two required: not sealed, both replicas back on the same base
    assert a["last"]["sealed"] is False and b["last"]["sealed"] is False and a["last"]["participants"] == 1
    assert torch.equal(a["master"], b["master"]) and bool(torch.isfinite(a["master"]).all())
    assert a["rounds"] == 7 and a["base"] == "checkpoint.round.6"                     # the base did not advance in the unsealed round


def test_launcher_flags_travel_in_the_environment(monkeypatch):
    """``--nproc N`` re-executes under torch.distributed.run, whose parser would read ``--nproc`` as an abbreviation of its
    own option if the worker's flags followed the module name; they go through the environment instead."""
    import json
    from openagents_b200.train import launcher as L
    seen = {}
    monkeypatch.setattr(L.subprocess, "call", lambda cmd, env=None: seen.update(cmd=cmd, env=env) or 0)
    monkeypatch.delenv("RANK", raising=False)
    with pytest.raises(SystemExit) as e:
        L.main(["--nproc", "2", "--sync-profile", "diloco", "--inner-steps", "4", "--steps", "8"])
    assert e.value.code == 0
    assert seen["cmd"][-2:] == ["-m", "openagents_b200.train.launcher"] and "--nproc-per-node=2" in seen["cmd"]
    assert "127.0.0.1" in seen["cmd"] and "--nproc" not in seen["cmd"]
    argv = json.loads(seen["env"]["B200_TRAIN_ARGV"])
    assert argv == ["--nproc", "2", "--sync-profile", "diloco", "--inner-steps", "4", "--steps", "8"]
    got = {}
    monkeypatch.setattr(L, "worker", lambda args: got.update(profile=args.sync_profile, inner=args.inner_steps, steps=args.steps))
    monkeypatch.setenv("RANK", "1")
    monkeypatch.setenv("B200_TRAIN_ARGV", seen["env"]["B200_TRAIN_ARGV"])
    L.main([])
    assert got == {"profile": "diloco", "inner": 4, "steps": 8}
