"""The plain-PyTorch training arm (baseline/gpt2_torch.py): it learns, and its DDP path keeps two ranks in step."""
import os
import socket
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from baseline.gpt2_torch import run_train_baseline  # noqa: E402
from openagents_b200.models.config import ModelConfig  # noqa: E402

CFG = ModelConfig(name="tiny-gpt2", arch="gpt2", vocab=97, d_model=32, n_layers=2, n_heads=4, n_kv_heads=4, ffn=64, context=16)


def _batches(rank):
    g = torch.Generator().manual_seed(rank)
    tok = torch.randint(0, CFG.vocab, (2, 4, 9), generator=g)       # accum 2, micro-batch 4, 8 positions
    return [(tok[..., :-1].contiguous(), tok[..., 1:].contiguous())]


def test_baseline_arm_learns_on_one_rank():
    r = run_train_baseline(CFG, torch.device("cpu"), 0, 1, _batches(0), accum=2, steps=12, warmup=1, lr=3e-3)
    assert r["ms_per_step"] > 0
    assert abs(r["losses"][0] - r["first_loss_expected"]) < 0.5        # random init: about ln(vocab)
    assert r["losses"][-1] < r["losses"][0] - 0.3                      # the same batch repeated: the loss falls


def _rank(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    r = run_train_baseline(CFG, torch.device("cpu"), rank, world, _batches(rank), accum=2, steps=3, warmup=1, lr=3e-3, barrier=dist.barrier)
    q.put((rank, r["losses"]))
    dist.destroy_process_group()


def test_baseline_arm_ddp_two_ranks():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    got = dict(q.get(timeout=60) for _ in ps)
    for p in ps:
        p.join(60)
        assert p.exitcode == 0
    assert len(got[0]) == len(got[1]) == 4
    assert got[0][0] != got[1][0]                     # different data per rank
    assert all(l == l and l < 10 for l in got[0] + got[1])
