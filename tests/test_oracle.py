"""CPU reference math: gradient checks and model-level sanity (mirrors the reference's own tests:
cs336-a1-real-gradient-workload.test.ts:50-83 central finite differences, :85-118 loss decreases)."""
import math

import torch

from openagents_b200.models.config import GPT2_SMALL, TINY_LLAMA, ModelConfig
from openagents_b200.models.weights import load_gguf_float, random_weights, save_gguf
from openagents_b200.oracle import nn
from openagents_b200.oracle.models import KVCacheRef, gpt2_forward, greedy_generate, llama_forward


def test_rmsnorm_matches_reference_formula():
    x = torch.tensor([[1.0, -2.0, 3.0, 0.5]], dtype=torch.float64)
    g = torch.tensor([1.0, 0.5, 2.0, 1.0], dtype=torch.float64)
    inv = 1.0 / math.sqrt(float((x ** 2).mean()) + 1e-5)
    assert torch.allclose(nn.rmsnorm(x, g, 1e-5), x * inv * g)


def test_rope_styles_preserve_norm_and_relative_phase():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 2, 8, generator=g, dtype=torch.float64)
    for style in ("pairs", "half"):
        y = nn.rope(x, torch.arange(5), 10000.0, style)
        assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
        # dot products depend only on the position difference
        q = nn.rope(x[:1].expand(5, -1, -1), torch.arange(5), 10000.0, style)
        k = nn.rope(x[1:2].expand(5, -1, -1), torch.arange(5) + 3, 10000.0, style)
        d = (q * k).sum(-1)
        assert torch.allclose(d, d[:1].expand_as(d))


def test_attention_window_and_sinks():
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(6, 4, 8, generator=g, dtype=torch.float64) for _ in range(3))
    k, v = k[:, :2], v[:, :2]
    pos = torch.arange(6)
    full = nn.attention(q, k, v, pos, pos)
    win = nn.attention(q, k, v, pos, pos, window=6)
    assert torch.allclose(full, win)
    w2 = nn.attention(q, k, v, pos, pos, window=1)          # only the token itself
    assert torch.allclose(w2, v.repeat_interleave(2, 1))
    s = nn.attention(q, k, v, pos, pos, sinks=torch.full((4,), -1e9, dtype=torch.float64))
    assert torch.allclose(full, s)
    s2 = nn.attention(q, k, v, pos, pos, sinks=torch.zeros(4, dtype=torch.float64))
    assert (s2.norm(dim=-1) < full.norm(dim=-1) + 1e-9).all()


def test_finite_difference_gradients_tiny_llama():
    cfg = ModelConfig(n_layers=1, d_model=8, n_heads=2, n_kv_heads=1, head_dim=4, ffn=12, vocab=7, context=16)
    W = {k: v.double().requires_grad_(True) for k, v in random_weights(cfg, 0).items()}
    for k in W:
        if "norm" not in k:
            W[k].data.mul_(10.0)
    toks = torch.tensor([1, 3, 5, 2, 6])
    tgt = torch.tensor([3, 5, 2, 6, 0])

    def loss():
        return torch.nn.functional.cross_entropy(llama_forward(cfg, W, toks), tgt)

    l = loss()
    l.backward()
    worst = 0.0
    for name, p in W.items():
        flat, gflat = p.data.view(-1), p.grad.view(-1)
        for i in range(0, flat.numel(), max(1, flat.numel() // 7)):
            old = flat[i].item()
            flat[i] = old + 1e-5
            lp = loss().item()
            flat[i] = old - 1e-5
            lm = loss().item()
            flat[i] = old
            fd = (lp - lm) / 2e-5
            worst = max(worst, abs(fd - gflat[i].item()) / max(1e-8, abs(fd) + abs(gflat[i].item())))
    assert worst < 1e-5


def test_cache_matches_full_forward():
    cfg = TINY_LLAMA.with_(vocab=200)
    W = random_weights(cfg, 1)
    toks = torch.arange(10) % 200
    full = llama_forward(cfg, W, toks)
    cache = KVCacheRef(cfg.n_layers)
    a = llama_forward(cfg, W, toks[:6], cache)
    b = llama_forward(cfg, W, toks[6:], cache)
    assert torch.allclose(torch.cat((a, b)), full, atol=1e-5)


def test_tiny_llama_gguf_greedy(tmp_path):
    """Benchmark configuration 1: tiny llama, Q8_0 GGUF, 32-token prompt, 64 greedy tokens on CPU."""
    cfg = TINY_LLAMA
    W = random_weights(cfg, 0)
    p = str(tmp_path / "tiny.gguf")
    save_gguf(p, cfg, W)
    cfg2, W2 = load_gguf_float(p)
    assert cfg2.n_layers == 2 and cfg2.d_model == 256 and cfg2.ffn == 688 and cfg2.n_kv_heads == 2
    assert abs(cfg2.norm_eps - 1e-5) < 1e-9
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab, (32,), generator=g)
    ids, logits = greedy_generate(cfg2, W2, prompt, 64)
    assert ids.shape == (64,) and logits.shape == (64, cfg.vocab)
    ids2, _ = greedy_generate(cfg2, W2, prompt, 64)
    assert torch.equal(ids, ids2)


def test_gpt2_loss_near_uniform_at_init():
    cfg = GPT2_SMALL.with_(n_layers=2, d_model=64, n_heads=4, head_dim=16, ffn=128, vocab=97, context=32)
    W = random_weights(cfg, 0)
    toks = torch.randint(0, 97, (2, 16), generator=torch.Generator().manual_seed(0))
    logits = gpt2_forward(cfg, W, toks)
    tgt = torch.randint(0, 97, (2, 16), generator=torch.Generator().manual_seed(9))
    loss = torch.nn.functional.cross_entropy(logits.view(-1, 97), tgt.view(-1))
    assert abs(loss.item() - math.log(97)) < 0.2
