"""Mixture-of-experts engine: routing + dispatch + grouped GEMMs + combine against the CPU oracle, on one
GPU and expert-parallel on two."""
import pytest
import torch

from openagents_b200.models.config import GPT_OSS_20B
from openagents_b200.models.weights import PLAN_MOE, load_gguf_float, random_weights, save_gguf
from openagents_b200.oracle.models import KVCacheRef, llama_forward

pytestmark = pytest.mark.gpu

TINY_MOE = GPT_OSS_20B.with_(n_layers=3, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=256, vocab=512,
                             n_experts=8, top_k=2, sliding_window=16, context=512, name="tiny-moe")


def _make(tmp_path, seed=5):
    p = str(tmp_path / "moe.gguf")
    W = random_weights(TINY_MOE, seed)
    for k in W:                       # a wider router spread than N(0, 0.02) so that top-k margins are not ties
        if k.endswith("ffn_gate_inp.weight"):
            W[k] = W[k] * 20
    save_gguf(p, TINY_MOE, W, PLAN_MOE)
    return p


def _prompts(n, seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, TINY_MOE.vocab, (int(torch.randint(5, 40, (1,), generator=g)),), generator=g) for _ in range(n)]


def _check_against_oracle(eng, cfg2, W, prompts, seq0=0):
    B = len(prompts)
    ids = list(range(seq0, seq0 + B))
    for s in ids:
        eng.begin(s)
    logits, nxt = eng.forward_tokens(ids, [x.tolist() for x in prompts])
    caches = [KVCacheRef(cfg2.n_layers) for _ in range(B)]
    ref = torch.stack([llama_forward(cfg2, W, prompts[b], caches[b])[-1] for b in range(B)])
    scale = ref.std().item()
    assert (logits.cpu() - ref).abs().max().item() < 0.08 * scale
    toks = ref.argmax(-1).tolist()
    for step in range(4):
        logits, nxt = eng.decode(ids, toks, use_graph=(step > 1))
        ref = torch.stack([llama_forward(cfg2, W, torch.tensor([toks[b]]), caches[b])[-1] for b in range(B)])
        assert (logits.cpu() - ref).abs().max().item() < 0.08 * scale, step
        toks = ref.argmax(-1).tolist()
    eng.check_status()
    assert eng.ep.heap.status() == (0, 0)


def test_moe_ffn_block_matches_oracle(tmp_path):
    """Router + dispatch + grouped GEMMs + combine alone, against the oracle's moe_ffn on the same rows."""
    from openagents_b200.models.moe_engine import MoEEngine
    from openagents_b200.models.qweight import GGUFSource
    from openagents_b200.ops import cuda_ops as ops
    from openagents_b200.oracle.models import moe_ffn
    p = _make(tmp_path)
    cfg2, W = load_gguf_float(p)
    src = GGUFSource(p, "cuda")
    eng = MoEEngine(src.cfg, src, max_batch=8, max_ctx=128, max_tokens=256)
    for T in (50, 200, 3):
        hb = torch.randn(T, cfg2.d_model, generator=torch.Generator().manual_seed(T)).bfloat16().cuda()
        eng.hf32[:T].copy_(hb.float())
        x = eng.x[:T]
        x.zero_()
        for li in (0, 1):
            ops.moe_zero(eng.counts)
            x.zero_()
            eng._ffn_dense(li, eng.layers[li], T, x, hb, None, None)
            ref = moe_ffn(cfg2, W, f"blk.{li}.", hb.float().cpu())
            rp, ri = torch.topk(hb.float().cpu() @ W[f"blk.{li}.ffn_gate_inp.weight"].t(), cfg2.top_k)
            assert torch.equal(eng.topk_ids[:T].cpu().long(), ri), (T, li)
            assert torch.allclose(eng.topk_w[:T].cpu(), torch.softmax(rp, -1), atol=1e-5), (T, li)
            assert int(eng.counts[li & 1].sum()) == T * cfg2.top_k
            err = (x.cpu() - ref).abs().max().item()
            assert err < 0.03 * ref.abs().max().item() + 1e-4, (T, li, err, ref.abs().max().item())
    eng.check_status()


def test_moe_single_gpu_matches_oracle(tmp_path):
    from openagents_b200.models.moe_engine import MoEEngine
    from openagents_b200.models.qweight import GGUFSource
    p = _make(tmp_path)
    cfg2, W = load_gguf_float(p)
    src = GGUFSource(p, "cuda")
    eng = MoEEngine(src.cfg, src, max_batch=8, max_ctx=128, max_tokens=256)
    assert eng.placement_digest().startswith("sha256:")
    _check_against_oracle(eng, cfg2, W, _prompts(3, 1))
    # the routing the kernel reports is the oracle's: top-k ids of the last forward's tokens
    from openagents_b200.oracle import nn
    assert eng.topk_w[:3].sum(-1).sub(1).abs().max().item() < 1e-5


def _ep_worker(rank, world, path):
    from openagents_b200.models.moe_engine import MoEEngine
    from openagents_b200.models.qweight import GGUFSource
    cfg2, W = load_gguf_float(path)
    src = GGUFSource(path, f"cuda:{rank}")
    eng = MoEEngine(src.cfg, src, device=f"cuda:{rank}", max_batch=8, max_ctx=128, max_tokens=256, ep_rank=rank, ep_world=world)
    assert eng.E_local == TINY_MOE.n_experts // world
    # every rank serves its own sequences; the experts they hit live on both ranks
    _check_against_oracle(eng, cfg2, W, _prompts(3, 10 + rank))


def test_moe_expert_parallel_two_gpus(tmp_path):
    from test_gpu_multi import _need, _run
    _need(2)
    _run(_ep_worker, 2, _make(tmp_path))
