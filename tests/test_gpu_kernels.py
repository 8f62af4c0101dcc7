"""sm_100a kernels against plain PyTorch fp32 references of the same op."""
import math

import pytest
import torch

from openagents_b200.gguf import GgmlType
from openagents_b200.gguf import torch_codecs as tc

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _ops():
    from openagents_b200.ops import cuda_ops
    return cuda_ops


def _qweight(x, t):
    from openagents_b200.models.qweight import QWeight, RawTensor
    return QWeight.from_raw(RawTensor(t, tuple(x.shape), tc.quantize(x, t)))


def _randn(*shape, seed=0, scale=1.0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return torch.randn(*shape, generator=g, device=DEV) * scale


def _quant_x(x):
    """Reference of the activation quantizer: per-32 int8 with fp32 scale."""
    xb = x.reshape(x.shape[0], -1, 32)
    d = xb.abs().amax(-1, keepdim=True) / 127.0
    q = torch.where(d > 0, torch.round(xb / d), torch.zeros_like(xb))
    return (q * d).reshape(x.shape), q, d


def _alloc_q(nb, K):
    return (torch.empty((nb, K), dtype=torch.int8, device=DEV), torch.empty((nb, K // 32), device=DEV),
            torch.empty((nb, K // 16), device=DEV))


def test_rmsnorm_and_quant():
    ops = _ops()
    T, D = 5, 1024
    x, g = _randn(T, D, seed=1), _randn(D, seed=2) * 0.1 + 1.0
    xq, xd, xs = _alloc_q(T, D)
    hf = torch.empty((T, D), device=DEV)
    hb = torch.empty((T, D), dtype=torch.bfloat16, device=DEV)
    ops.rmsnorm(x, g, 1e-5, xq=xq, xd=xd, xs16=xs, hb=hb, hf=hf)
    ref = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * g
    assert torch.allclose(hf, ref, atol=1e-5, rtol=1e-5)
    assert torch.allclose(hb.float(), ref, atol=2e-2, rtol=1e-2)
    deq_ref, q_ref, d_ref = _quant_x(ref)
    # undo the byte order and compare the dequantized activations
    inv = torch.tensor(tc.X8_POS, device=DEV)
    q = xq.view(T, D // 8, 8)[:, :, inv].reshape(T, D // 32, 32).float()
    assert torch.allclose(q * xd[..., None], deq_ref.reshape(T, D // 32, 32), atol=float(d_ref.max()) * 1.01)
    s16 = (q.reshape(T, D // 16, 16).sum(-1) * xd.repeat_interleave(2, dim=1))
    assert torch.allclose(xs, s16, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("t", [GgmlType.Q4_K, GgmlType.Q6_K, GgmlType.Q8_0, GgmlType.MXFP4])
def test_dequant_matches_codec(t):
    ops = _ops()
    N, K = 96, 1024
    x = _randn(N, K, seed=3, scale=0.02)
    w = _qweight(x, t)
    out = torch.empty((N, K), dtype=torch.bfloat16, device=DEV)
    ops.dequant_bf16(w.wt, w.main, w.plane2, out, N, K)
    ref = tc.dequantize(tc.quantize(x, t), t, (N, K))
    assert torch.allclose(out.float(), ref, atol=1e-4, rtol=8e-3)


@pytest.mark.parametrize("t", [GgmlType.Q4_K, GgmlType.Q6_K, GgmlType.Q8_0, GgmlType.BF16])
@pytest.mark.parametrize("nb", [1, 3, 8])
def test_matvec_store_and_resid(t, nb):
    ops = _ops()
    N, K = 200, 1024   # N not a multiple of 32: exercises the row tail
    W = _randn(N, K, seed=4, scale=0.02)
    w = _qweight(W, t)
    Wd = tc.dequantize(tc.quantize(W, t), t, (N, K)) if t != GgmlType.BF16 else W.bfloat16().float()
    x = _randn(nb, K, seed=5)
    bias = _randn(N, seed=6)
    xq, xd, xs = _alloc_q(nb, K)
    ops.quantize_x(x, xq, xd, xs)
    y = torch.zeros((nb, N), device=DEV)
    ops.matvec(w.wt, w.main, w.plane2, N, K, nb, xq=xq, xd=xd, xs16=xs, xf=x, epi=ops.EPI_STORE, bias=bias, y=y, ldy=N)
    ref = x @ Wd.t() + bias
    tol = 0.02 * ref.std().item()
    assert (y - ref).abs().max().item() < 4 * tol, (y - ref).abs().max().item()
    # exact against the same quantized activations
    if t != GgmlType.BF16:
        xdq, _, _ = _quant_x(x)
        ref_q = xdq @ Wd.t() + bias
        assert torch.allclose(y, ref_q, atol=2e-3 * ref.std().item() + 1e-5, rtol=1e-4)
    r = _randn(nb, N, seed=7)
    y2 = r.clone()
    ops.matvec(w.wt, w.main, w.plane2, N, K, nb, xq=xq, xd=xd, xs16=xs, xf=x, epi=ops.EPI_RESID, resid=y2, y=y2, ldy=N)
    assert torch.allclose(y2, r + (y - bias), atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("t", [GgmlType.Q4_K, GgmlType.BF16])
@pytest.mark.parametrize("nb", [1, 4])
def test_matvec_swiglu(t, nb):
    ops = _ops()
    F, K = 256, 512
    W = _randn(2 * F, K, seed=8, scale=0.05)                  # gate rows, then up rows
    Wi = torch.stack((W[:F], W[F:]), dim=1).reshape(2 * F, K)  # the kernels read them interleaved (gate_0, up_0, ...)
    w = _qweight(Wi, t)
    Wd = tc.dequantize(tc.quantize(W, t), t, (2 * F, K)) if t != GgmlType.BF16 else W.bfloat16().float()
    x = _randn(nb, K, seed=9)
    xq, xd, xs = _alloc_q(nb, K)
    ops.quantize_x(x, xq, xd, xs)
    xin = _quant_x(x)[0] if t != GgmlType.BF16 else x
    gu = xin @ Wd.t()
    ref = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
    y = torch.zeros((nb, F), device=DEV)
    ops.matvec(w.wt, w.main, w.plane2, F, K, nb, xq=xq, xd=xd, xs16=xs, xf=x, epi=ops.EPI_SWIGLU_F32, y=y, ldy=F)
    assert torch.allclose(y, ref, atol=2e-3 * ref.std().item() + 1e-5, rtol=1e-3)
    oq, od, os16 = _alloc_q(nb, F)
    ops.matvec(w.wt, w.main, w.plane2, F, K, nb, xq=xq, xd=xd, xs16=xs, xf=x, epi=ops.EPI_SWIGLU_Q8, oq=oq, od=od, os16=os16)
    inv = torch.tensor(tc.X8_POS, device=DEV)
    q = oq.view(nb, F // 8, 8)[:, :, inv].reshape(nb, F // 32, 32).float()
    deq = (q * od[..., None]).reshape(nb, F)
    assert (deq - ref).abs().max().item() <= ref.abs().max().item() / 127.0 * 0.6 + 2e-3 * ref.std().item()


def test_embedding_types():
    ops = _ops()
    V, D = 300, 512
    E = _randn(V, D, seed=10, scale=0.02)
    ids = torch.tensor([0, 5, 299, 17], dtype=torch.int32, device=DEV)
    for t, et in ((GgmlType.Q6_K, ops.EMB_Q6KR), (GgmlType.Q8_0, ops.EMB_Q8R), (GgmlType.BF16, ops.EMB_BF16)):
        w = _qweight(E, t)
        ref = tc.dequantize(tc.quantize(E, t), t, (V, D))[ids.long()]
        out = torch.empty((4, D), device=DEV)
        ops.embedding(ids, out, et, w.main, w.plane2)
        assert torch.allclose(out, ref, atol=1e-6, rtol=1e-5)
    out = torch.ones((4, D), device=DEV)
    w = _qweight(E, GgmlType.BF16)
    ops.embedding(ids, out, ops.EMB_BF16, w.main, None, vocab_lo=100, vocab_n=100)
    assert out.abs().sum().item() == 0.0


@pytest.mark.parametrize("style", ["pairs", "half"])
def test_rope_kv_write(style):
    from openagents_b200.oracle import nn
    ops = _ops()
    T, Hq, Hkv, hd = 6, 4, 2, 64
    qkv = _randn(T, (Hq + 2 * Hkv) * hd, seed=11)
    pos = torch.tensor([0, 1, 2, 700, 3000, 8191], dtype=torch.int32, device=DEV)
    slot = torch.tensor([16, 17, 18, 3, 40, 5], dtype=torch.int32, device=DEV)
    kc = torch.zeros((4, Hkv, 16, hd), dtype=torch.float16, device=DEV)
    vc = torch.zeros_like(kc)
    q32 = torch.empty((T, Hq * hd), device=DEV)
    q16 = torch.empty((T, Hq * hd), dtype=torch.float16, device=DEV)
    ops.rope_kv(qkv, pos, slot, q32, q16, kc, vc, Hq, Hkv, hd, 16, 500000.0, 0 if style == "pairs" else 1, 0.125)
    q, k, v = qkv.cpu().split([Hq * hd, Hkv * hd, Hkv * hd], dim=-1)
    qr = nn.rope(q.view(T, Hq, hd), pos.cpu(), 500000.0, style) * 0.125
    kr = nn.rope(k.view(T, Hkv, hd), pos.cpu(), 500000.0, style)
    assert torch.allclose(q32.cpu().view(T, Hq, hd), qr, atol=2e-5)
    assert torch.allclose(q16.cpu().float().view(T, Hq, hd), qr, atol=2e-3)
    for i in range(T):
        s = int(slot[i])
        assert torch.allclose(kc[s // 16, :, s % 16].cpu().float(), kr[i], atol=4e-3)
        assert torch.allclose(vc[s // 16, :, s % 16].cpu().float(), v.view(T, Hkv, hd)[i], atol=4e-3)


def test_rope_table_matches_direct():
    ops = _ops()
    T, Hq, Hkv, hd = 5, 4, 2, 128
    qkv = _randn(T, (Hq + 2 * Hkv) * hd, seed=12)
    pos = torch.tensor([0, 5, 1023, 4000, 9000], dtype=torch.int32, device=DEV)   # last one is beyond the table
    slot = torch.tensor([0, 1, 2, 3, -1], dtype=torch.int32, device=DEV)            # last one writes no KV
    tab = ops.rope_table(8192, hd, 500000.0, DEV)
    outs = []
    for table in (None, tab):
        kc = torch.zeros((2, Hkv, 16, hd), dtype=torch.float16, device=DEV)
        vc = torch.zeros_like(kc)
        q32 = torch.empty((T, Hq * hd), device=DEV)
        ops.rope_kv(qkv, pos, slot, q32, None, kc, vc, Hq, Hkv, hd, 16, 500000.0, 0, 1.0, table=table)
        outs.append((q32, kc, vc))
    for a, b in zip(*outs):
        assert torch.equal(a, b)
    assert outs[1][1][0, :, 4:].abs().sum().item() == 0.0


@pytest.mark.parametrize("M,N,K", [(64, 4096, 14336), (8, 512, 4096), (64, 192, 1024)])
def test_gemm_split_k_inplace_residual(M, N, K):
    """Few output tiles: the in-place residual add runs split over K with vector reductions."""
    ops = _ops()
    A = _randn(M, K, seed=31).bfloat16()
    B = _randn(N, K, seed=32, scale=0.05).bfloat16()
    bias = _randn(N, seed=33)
    x0 = _randn(M, N, seed=34)
    ref = x0 + bias + A.float() @ B.float().t()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for split_k, tile_n in ((0, 0), (1, 0), (3, 0), (0, -1), (1, -1)):      # tile_n -1: weights as the 128-row operand
        x = x0.clone()
        ops.gemm_bf16(A, B, M, N, K, out_f32=x, resid_f32=x, bias=bias, status=status, split_k=split_k, tile_n=tile_n)
        assert (x - ref).abs().max().item() < 2e-3 * math.sqrt(K) * 0.05 + 1e-3, (split_k, tile_n)
    out = torch.zeros((M, N), device=DEV)
    outb = torch.zeros((M, N), dtype=torch.bfloat16, device=DEV)
    ops.gemm_bf16(A, B, M, N, K, out_f32=out, out_bf16=outb, bias=bias, act=ops.ACT_GELU, tile_n=-1, status=status)
    g = torch.nn.functional.gelu(ref - x0, approximate="tanh")
    assert torch.allclose(out, g, atol=2e-2, rtol=1e-3) and torch.allclose(outb.float(), g, atol=5e-2, rtol=2e-2)
    assert int(status.item()) == 0


def _paged_kv(B, Hkv, hd, lens, seed):
    """Random K/V for B sequences scattered over shuffled pages.  Returns caches, table, dense K/V."""
    max_pages = (max(lens) + 15) // 16
    n_pages = B * max_pages + 3
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(n_pages, generator=g)
    table = torch.zeros((B, max_pages), dtype=torch.int32)
    kc = torch.zeros((n_pages, Hkv, 16, hd), dtype=torch.float16)
    vc = torch.zeros_like(kc)
    Ks, Vs = [], []
    for b in range(B):
        K = torch.randn(lens[b], Hkv, hd, generator=g).half()
        V = torch.randn(lens[b], Hkv, hd, generator=g).half()
        Ks.append(K.float())
        Vs.append(V.float())
        for p in range((lens[b] + 15) // 16):
            pid = int(perm[b * max_pages + p])
            table[b, p] = pid
            n = min(16, lens[b] - p * 16)
            kc[pid, :, :n] = K[p * 16: p * 16 + n].transpose(0, 1)
            vc[pid, :, :n] = V[p * 16: p * 16 + n].transpose(0, 1)
    return kc.to(DEV), vc.to(DEV), table.to(DEV), Ks, Vs


@pytest.mark.parametrize("hd,Hq,Hkv", [(128, 8, 2), (64, 16, 2), (128, 4, 4)])
@pytest.mark.parametrize("S", [1, 5])
@pytest.mark.parametrize("window,use_sinks", [(0, False), (40, True)])
def test_attn_decode(hd, Hq, Hkv, S, window, use_sinks):
    from openagents_b200.oracle import nn
    ops = _ops()
    lens = [1, 17, 130, 333]
    B = len(lens)
    kc, vc, table, Ks, Vs = _paged_kv(B, Hkv, hd, lens, seed=12)
    q = _randn(B, Hq * hd, seed=13) * (1.0 / math.sqrt(hd))
    sinks = _randn(Hq, seed=14) if use_sinks else None
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=DEV)
    out = torch.empty((B, Hq * hd), device=DEV)
    oq, od, os16 = _alloc_q(B, Hq * hd)
    scratch = torch.empty(ops.attn_decode_scratch_floats(B, Hq, Hkv, hd, S), device=DEV)
    counters = torch.zeros(B * Hkv, dtype=torch.int32, device=DEV)
    for _ in range(2):   # second run checks the counters were left at zero
        ops.attn_decode(q, kc, vc, table, seq_lens, B, Hq, Hkv, hd, window=window, S=S, sinks=sinks, out_f32=out,
                        oq=oq, od=od, os16=os16, scratch=scratch, counters=counters)
        for b in range(B):
            L = lens[b]
            ref = nn.attention(q[b].cpu().view(1, Hq, hd), Ks[b], Vs[b], torch.tensor([L - 1]), torch.arange(L),
                               window=window, sinks=sinks.cpu() if use_sinks else None, scale=1.0).reshape(-1)
            assert torch.allclose(out[b].cpu(), ref, atol=2e-3, rtol=2e-3), (b, (out[b].cpu() - ref).abs().max())
    assert int(counters.abs().sum()) == 0
    inv = torch.tensor(tc.X8_POS, device=DEV)
    deq = (oq.view(B, -1, 8)[:, :, inv].reshape(B, -1, 32).float() * od[..., None]).reshape(B, -1)
    assert (deq - out).abs().max().item() <= out.abs().max().item() / 127 * 0.6


@pytest.mark.parametrize("hd,Hq,Hkv", [(128, 4, 2), (64, 4, 1)])
@pytest.mark.parametrize("window,use_sinks", [(0, False), (50, True)])
def test_attn_prefill(hd, Hq, Hkv, window, use_sinks):
    from openagents_b200.oracle import nn
    ops = _ops()
    ctx = [70, 200, 129]        # keys in cache after the chunk
    qlen = [70, 64, 1]          # new query tokens (second sequence has 136 cached tokens)
    B = len(ctx)
    kc, vc, table, Ks, Vs = _paged_kv(B, Hkv, hd, ctx, seed=15)
    T = sum(qlen)
    q = (_randn(T, Hq * hd, seed=16) * (1.0 / math.sqrt(hd))).half()
    sinks = _randn(Hq, seed=17) if use_sinks else None
    q_start = torch.tensor([0, 70, 134], dtype=torch.int32, device=DEV)
    out = torch.empty((T, Hq * hd), device=DEV)
    outb = torch.empty((T, Hq * hd), dtype=torch.bfloat16, device=DEV)
    lse = torch.empty((T, Hq), device=DEV)
    ops.attn_prefill(q, kc, vc, table, table.shape[1], q_start, torch.tensor(qlen, dtype=torch.int32, device=DEV),
                     torch.tensor(ctx, dtype=torch.int32, device=DEV), B, max(qlen), Hq, Hkv, hd, window=window,
                     sinks=sinks, out_bf16=outb, out_f32=out, lse=lse)
    for b in range(B):
        s, n = int(q_start[b]), qlen[b]
        qpos = torch.arange(ctx[b] - n, ctx[b])
        ref = nn.attention(q[s:s + n].float().cpu().view(n, Hq, hd), Ks[b], Vs[b], qpos, torch.arange(ctx[b]),
                           window=window, sinks=sinks.cpu() if use_sinks else None, scale=1.0).reshape(n, -1)
        assert torch.allclose(out[s:s + n].cpu(), ref, atol=3e-3, rtol=3e-3), (b, (out[s:s + n].cpu() - ref).abs().max())
        assert torch.allclose(outb[s:s + n].float().cpu(), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("Hq,Hkv,window,use_sinks,qk_gain", [(4, 2, 0, False, 1.0), (8, 2, 96, True, 1.0), (2, 2, 0, True, 1.0),
                                                             (4, 2, 0, True, 6.0), (4, 4, 160, False, 5.0)])
def test_attn_prefill_tc05(Hq, Hkv, window, use_sinks, qk_gain):
    """tcgen05 prefill attention (head dim 128) against the fp32 oracle: cold prefill longer than one query
    tile, a chunk on top of cached context, a one-token chunk, and a sequence that ends mid key block.
    ``qk_gain`` > 1 spreads the scores (standard deviation ~ gain), so that row maxima keep jumping by more
    than the kernel's rescale step and the in-tensor-memory rescale of the output rows runs many times."""
    from openagents_b200.oracle import nn
    ops = _ops()
    hd = 128
    ctx = [300, 200, 129, 513]
    qlen = [300, 64, 1, 257]
    B = len(ctx)
    kc, vc, table, Ks, Vs = _paged_kv(B, Hkv, hd, ctx, seed=35)
    T = sum(qlen)
    q = (_randn(T, Hq * hd, seed=36) * (qk_gain / math.sqrt(hd))).half()
    sinks = _randn(Hq, seed=37) if use_sinks else None
    starts = [sum(qlen[:b]) for b in range(B)]
    q_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
    outb = torch.zeros((T, Hq * hd), dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.attn_prefill_tc05(q, kc, vc, table, q_start, torch.tensor(qlen, dtype=torch.int32, device=DEV),
                          torch.tensor(ctx, dtype=torch.int32, device=DEV), B, max(qlen), Hq, Hkv, window=window, sinks=sinks,
                          out_bf16=outb, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for b in range(B):
        s, n = starts[b], qlen[b]
        qpos = torch.arange(ctx[b] - n, ctx[b])
        ref = nn.attention(q[s:s + n].float().cpu().view(n, Hq, hd), Ks[b], Vs[b], qpos, torch.arange(ctx[b]),
                           window=window, sinks=sinks.cpu() if use_sinks else None, scale=1.0).reshape(n, -1)
        err = (outb[s:s + n].float().cpu() - ref).abs().max().item()
        assert err < 2e-2, (b, err)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (300, 520, 200), (64, 768, 768), (1024, 2304, 768), (257, 64, 4096)])
@pytest.mark.parametrize("tile_n", [0, 64, 128, 256])
def test_gemm_bf16(M, N, K, tile_n):
    ops = _ops()
    A = _randn(M, K, seed=18).bfloat16()
    B = _randn(N, K, seed=19).bfloat16()
    bias = _randn(N, seed=20)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.zeros((M, N), device=DEV)
    outb = torch.zeros((M, N), dtype=torch.bfloat16, device=DEV)
    ops.gemm_bf16(A, B, M, N, K, out_f32=out, out_bf16=outb, bias=bias, tile_n=tile_n, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ref = A.float() @ B.float().t() + bias
    err = (out - ref).abs().max().item()
    assert err < 2e-3 * math.sqrt(K), err
    assert torch.allclose(outb.float(), ref, atol=0.05 * ref.abs().max().item() / 4, rtol=2e-2)


def test_gemm_epilogues():
    ops = _ops()
    M, N, K = 200, 384, 256
    A = _randn(M, K, seed=21).bfloat16()
    B = _randn(N, K, seed=22, scale=0.05).bfloat16()
    bias = _randn(N, seed=23)
    resid = _randn(M, N, seed=24)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    base = A.float() @ B.float().t()
    out = resid.clone()
    ops.gemm_bf16(A, B, M, N, K, out_f32=out, resid_f32=out, bias=bias, status=status)   # in-place residual
    assert torch.allclose(out, base + bias + resid, atol=2e-2, rtol=1e-3)
    out = torch.zeros((M, N), device=DEV)
    ops.gemm_bf16(A, B, M, N, K, out_f32=out, bias=bias, act=ops.ACT_GELU, status=status)
    assert torch.allclose(out, torch.nn.functional.gelu(base + bias, approximate="tanh"), atol=2e-2, rtol=1e-3)
    acc = resid.clone()
    ops.gemm_bf16(A, B, M, N, K, out_f32=acc, accumulate=True, status=status)
    assert torch.allclose(acc, resid + base, atol=2e-2, rtol=1e-3)
    rb = resid.bfloat16()
    outb = torch.zeros((M, N), dtype=torch.bfloat16, device=DEV)
    ops.gemm_bf16(A, B, M, N, K, out_bf16=outb, resid_bf16=rb, status=status)
    assert torch.allclose(outb.float(), base + rb.float(), atol=0.1, rtol=2e-2)
    assert int(status.item()) == 0


def test_argmax_and_sampling():
    ops = _ops()
    T, V = 5, 50257
    logits = _randn(T, V, seed=25)
    logits[1, 777] = 50.0
    logits[2, 3] = logits[2, 9] = 60.0     # tie: lowest index wins
    ids = torch.zeros(T, dtype=torch.int32, device=DEV)
    vals = torch.zeros(T, device=DEV)
    ops.argmax(logits, ids, vals)
    assert torch.equal(ids.long().cpu(), logits.argmax(-1).cpu())
    assert int(ids[2]) == 3 and float(vals[1]) == 50.0
    # rows split over many blocks: same answer, twice in a row (the scratch resets itself)
    sc = ops.argmax_scratch(T, DEV)
    for _ in range(2):
        ids2 = torch.zeros(T, dtype=torch.int32, device=DEV)
        vals2 = torch.zeros(T, device=DEV)
        ops.argmax(logits, ids2, vals2, vocab_offset=7, scratch=sc)
        assert torch.equal(ids2, ids + 7) and torch.equal(vals2, vals)
    assert int(sc.abs().sum()) == 0
    neg = -torch.rand(3, 40000, device=DEV) - 1.0
    ids3 = torch.zeros(3, dtype=torch.int32, device=DEV)
    ops.argmax(neg, ids3, None, scratch=sc)
    assert torch.equal(ids3.long().cpu(), neg.argmax(-1).cpu())
    # top-1 sampling is arg-max whatever the random number
    u = torch.rand(T, device=DEV)
    scratch = torch.empty((T, V), device=DEV)
    out = torch.zeros(T, dtype=torch.int32, device=DEV)
    ops.sample_topk(logits, 1.0, 1, 1.0, u, out, scratch)
    assert torch.equal(out, ids)
    # with k=8 every draw must come from the 8 largest logits, and a tiny top-p collapses to arg-max
    ops.sample_topk(logits, 0.8, 8, 1.0, u, out, scratch)
    top8 = logits.topk(8, dim=-1).indices
    assert all(int(out[t]) in top8[t].tolist() for t in range(T))
    ops.sample_topk(logits, 1.0, 8, 1e-6, u, out, scratch)
    assert torch.equal(out, ids)


def test_swiglu_add_cast_transpose():
    ops = _ops()
    T, F = 7, 300
    gu = _randn(T, 2 * F, seed=26)
    of = torch.empty((T, F), device=DEV)
    ob = torch.empty((T, F), dtype=torch.bfloat16, device=DEV)
    ref = torch.nn.functional.silu(gu[:, 0::2]) * gu[:, 1::2]           # (gate_i, up_i) sit in adjacent columns
    ops.swiglu(gu, F, ob=ob, of=of)
    assert torch.allclose(of, ref, atol=1e-5, rtol=1e-5) and torch.allclose(ob.float(), ref, atol=2e-2, rtol=1e-2)
    ops.swiglu(gu, F, ob=ob, zero_after=True)
    assert torch.allclose(ob.float(), ref, atol=2e-2, rtol=1e-2) and float(gu.abs().max()) == 0.0
    a, b = _randn(1001, seed=27), _randn(1001, seed=28)
    c = a.clone()
    ops.add_inplace(c, b)
    assert torch.equal(c, a + b)
    y = torch.empty(1001, dtype=torch.bfloat16, device=DEV)
    ops.f32_to_bf16(a, y)
    assert torch.equal(y, a.bfloat16())
    m = _randn(70, 45, seed=29).bfloat16()
    mt = torch.empty((45, 70), dtype=torch.bfloat16, device=DEV)
    ops.transpose_bf16(m, mt)
    assert torch.equal(mt, m.t().contiguous())


def test_train_ops_match_torch():
    from openagents_b200.ops import train_ops as tops
    M, D, F_, V = 96, 256, 512, 1000
    x = _randn(M, D, seed=30).bfloat16()
    g, b = (_randn(D, seed=31) * 0.1 + 1.0), _randn(D, seed=32) * 0.1
    y = torch.empty_like(x)
    mean, rstd = torch.empty(M, device=DEV), torch.empty(M, device=DEV)
    tops.layernorm_fwd(x, g, b, 1e-5, y, mean, rstd)
    xr = x.float().requires_grad_(True)
    gr, br = g.clone().requires_grad_(True), b.clone().requires_grad_(True)
    ref = torch.nn.functional.layer_norm(xr, (D,), gr, br, 1e-5)
    assert torch.allclose(y.float(), ref, atol=3e-2, rtol=2e-2)
    dy = _randn(M, D, seed=33).bfloat16()
    ref.backward(dy.float())
    dx = torch.full((M, D), 0.5, dtype=torch.bfloat16, device=DEV)
    dg, db = torch.zeros(D, device=DEV), torch.zeros(D, device=DEV)
    tops.layernorm_bwd(dy, x, g, mean, rstd, dx, True, dg, db)
    assert torch.allclose(dx.float(), xr.grad + 0.5, atol=6e-2, rtol=3e-2)
    assert torch.allclose(dg, gr.grad, atol=0.15, rtol=2e-2) and torch.allclose(db, br.grad, atol=0.15, rtol=2e-2)
    # rows wider than the register-resident limit (1024) and a row count that is not a multiple of the warps per CTA
    M2, D2 = 37, 1280
    x2, dy2 = _randn(M2, D2, seed=70).bfloat16(), _randn(M2, D2, seed=71).bfloat16()
    g2, b2 = (_randn(D2, seed=72) * 0.1 + 1.0), _randn(D2, seed=73) * 0.1
    y2, mean2, rstd2 = torch.empty_like(x2), torch.empty(M2, device=DEV), torch.empty(M2, device=DEV)
    tops.layernorm_fwd(x2, g2, b2, 1e-5, y2, mean2, rstd2)
    xr2, gr2, br2 = x2.float().requires_grad_(True), g2.clone().requires_grad_(True), b2.clone().requires_grad_(True)
    ref2 = torch.nn.functional.layer_norm(xr2, (D2,), gr2, br2, 1e-5)
    assert torch.allclose(y2.float(), ref2, atol=3e-2, rtol=2e-2)
    ref2.backward(dy2.float())
    dx2 = torch.zeros((M2, D2), dtype=torch.bfloat16, device=DEV)
    dg2, db2 = torch.zeros(D2, device=DEV), torch.zeros(D2, device=DEV)
    tops.layernorm_bwd(dy2, x2, g2, mean2, rstd2, dx2, False, dg2, db2)
    assert torch.allclose(dx2.float(), xr2.grad, atol=6e-2, rtol=3e-2)
    assert torch.allclose(dg2, gr2.grad, atol=0.15, rtol=2e-2) and torch.allclose(db2, br2.grad, atol=0.15, rtol=2e-2)
    # GELU
    h = _randn(M, F_, seed=34).bfloat16()
    a = torch.empty_like(h)
    tops.gelu_fwd(h, a)
    hr = h.float().requires_grad_(True)
    ar = torch.nn.functional.gelu(hr, approximate="tanh")
    assert torch.allclose(a.float(), ar, atol=2e-2, rtol=2e-2)
    da = _randn(M, F_, seed=35).bfloat16()
    ar.backward(da.float())
    dh = da.clone()
    tops.gelu_bwd(h, dh)
    assert torch.allclose(dh.float(), hr.grad, atol=3e-2, rtol=3e-2)
    # bias gradient
    gb = torch.zeros(F_, device=DEV)
    tops.bias_grad(da, gb)
    assert torch.allclose(gb, da.float().sum(0), atol=1e-2, rtol=1e-3)
    # fused cross-entropy (vocabulary padded to 1024 columns; one masked row)
    ldl = 1024
    logits = (_randn(M, ldl, seed=36) * 2).bfloat16()
    tgt = torch.randint(0, V, (M,), device=DEV, dtype=torch.int32)
    tgt[5] = -1
    lr_ = logits[:, :V].float().requires_grad_(True)
    keep = tgt >= 0
    lref = torch.nn.functional.cross_entropy(lr_[keep], tgt[keep].long(), reduction="none")
    (lref.sum() / M).backward()
    loss = torch.empty(M, device=DEV)
    work = logits.clone()
    tops.ce_fused(work, tgt, loss, 1.0 / M, V)
    assert torch.allclose(loss[keep], lref, atol=2e-2, rtol=1e-2) and float(loss[5]) == 0.0
    assert torch.allclose(work[:, :V].float(), lr_.grad, atol=2e-4 + 1e-2 * lr_.grad.abs().max().item(), rtol=2e-2)
    assert float(work[:, V:].abs().sum()) == 0.0
    # embedding forward / backward
    Vv, T = 50, 8
    wte, wpe = _randn(Vv, D, seed=37).bfloat16(), _randn(T, D, seed=38).bfloat16()
    ids = torch.randint(0, Vv, (3 * T,), device=DEV, dtype=torch.int32)
    e = torch.empty((3 * T, D), dtype=torch.bfloat16, device=DEV)
    tops.embed_fwd(ids, wte, wpe, e, T)
    pos = torch.arange(3 * T, device=DEV) % T
    assert torch.allclose(e.float(), (wte[ids.long()].float() + wpe[pos].float()), atol=2e-2, rtol=1e-2)
    de = _randn(3 * T, D, seed=39).bfloat16()
    gte, gpe = torch.zeros(Vv, D, device=DEV), torch.zeros(T, D, device=DEV)
    tops.embed_bwd(ids, de, gte, gpe, T)
    rte = torch.zeros(Vv, D, device=DEV).index_add_(0, ids.long(), de.float())
    rpe = torch.zeros(T, D, device=DEV).index_add_(0, pos, de.float())
    assert torch.allclose(gte, rte, atol=1e-3) and torch.allclose(gpe, rpe, atol=1e-3)


@pytest.mark.parametrize("t", [GgmlType.Q4_K, GgmlType.Q6_K])
@pytest.mark.parametrize("T,N,K,split", [(64, 384, 1024, 1), (40, 200, 512, 2), (130, 256, 768, 1), (7, 128, 2048, 4),
                                         (64, 4096, 4096, 0)])
def test_qgemm_fused_dequant(t, T, N, K, split):
    """Fused-dequant GEMM against the dequantized weights in fp32: plain store (fp32 and bf16) with bias, accumulation
    with and without K splits, ragged N, more than one token tile."""
    ops = _ops()
    W = _randn(N, K, seed=40, scale=0.02)
    w = _qweight(W, t)
    Wd = tc.dequantize(tc.quantize(W, t), t, (N, K))
    x = _randn(T, K, seed=41).bfloat16()
    bias = _randn(N, seed=42)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ref = x.float() @ Wd.t() + bias
    tol = 0.02 * ref.std().item()
    if split == 1:
        y = torch.full((T, N), 7.0, device=DEV)
        yb = torch.zeros((T, N), dtype=torch.bfloat16, device=DEV)
        ops.qgemm(w, x, T, out_f32=y, out_bf16=yb, bias=bias, epi=ops.QEPI_STORE, status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert (y - ref).abs().max().item() < 4 * tol, (y - ref).abs().max().item()
        assert torch.allclose(yb.float(), ref, atol=4 * tol + 2e-2, rtol=2e-2)
    r = _randn(T, N, seed=43)
    y = r.clone()
    ops.qgemm(w, x, T, out_f32=y, bias=bias, epi=ops.QEPI_ADD, split_k=split, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert (y - r - ref).abs().max().item() < 4 * tol, (y - r - ref).abs().max().item()
    y2 = r.clone()          # run-twice determinism does not hold for split K (atomics); a single split must repeat bit for bit
    if split == 1:
        ops.qgemm(w, x, T, out_f32=y2, bias=bias, epi=ops.QEPI_ADD, split_k=1, status=status)
        assert torch.equal(y, y2)


@pytest.mark.parametrize("T,F,K", [(64, 256, 512), (33, 448, 1024), (5, 64, 256)])
def test_qgemm_swiglu(T, F, K):
    """Gate/up projection with interleaved rows: the epilogue pairs adjacent accumulator lanes and writes silu(gate) * up."""
    ops = _ops()
    W = _randn(2 * F, K, seed=44, scale=0.05)
    Wi = torch.stack((W[:F], W[F:]), dim=1).reshape(2 * F, K)
    w = _qweight(Wi, GgmlType.Q4_K)
    Wd = tc.dequantize(tc.quantize(W, GgmlType.Q4_K), GgmlType.Q4_K, (2 * F, K))
    x = _randn(T, K, seed=45).bfloat16()
    gu = x.float() @ Wd.t()
    ref = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
    out = torch.zeros((T, F), dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.qgemm(w, x, T, out_bf16=out, ldo=F, epi=ops.QEPI_SWIGLU, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert torch.allclose(out.float(), ref, atol=0.04 * ref.std().item() + 1e-3, rtol=3e-2), (out.float() - ref).abs().max().item()


def test_slot_allreduce_single_rank():
    """The one-shot all-reduce with a world of one: a mat-vec or a fused-dequant GEMM leaves its result in the local
    partial buffer; the RMSNorm pushes each row into its slot, raises and awaits the row's flag, adds the slots into the
    residual stream, normalises the sum and leaves the partial rows zeroed.  Several rounds with different row counts, so
    both parities and the per-row device-side sequence numbers are exercised; the arg-max merge uses the same scheme."""
    from openagents_b200.parallel.symm import SymmHeap
    ops = _ops()
    N, K, rows = 256, 512, 64
    heap = SymmHeap(64 << 20, DEV)
    slots, slots_off = heap.alloc_tensor((2, 1, rows, N), torch.float32)
    part = torch.zeros((rows, N), device=DEV)
    W = _randn(N, K, seed=46, scale=0.05)
    w = _qweight(W, GgmlType.Q4_K)
    Wd = tc.dequantize(tc.quantize(W, GgmlType.Q4_K), GgmlType.Q4_K, (N, K))
    g = _randn(N, seed=47) * 0.1 + 1.0
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for rnd, nb in enumerate((1, 3, 40, 64, 2, 64)):
        x = _randn(nb, K, seed=48 + rnd)
        resid = _randn(nb, N, seed=60 + rnd)
        xres = resid.clone()
        if nb <= 4:
            xq, xd, xs = _alloc_q(nb, K)
            ops.quantize_x(x, xq, xd, xs)
            xin = _quant_x(x)[0]
            ops.matvec(w.wt, w.main, w.plane2, N, K, nb, xq=xq, xd=xd, xs16=xs, xf=x, epi=ops.EPI_STORE, y=part, ldy=N)
        else:
            xin = x.bfloat16().float()
            ops.qgemm(w, x.bfloat16(), nb, out_f32=part, ldo=N, epi=ops.QEPI_ADD, status=status)
        hf = torch.empty((nb, N), device=DEV)
        ops.rmsnorm(xres, g, 1e-5, hf=hf, slots=(heap.table, slots_off, rows, part))
        torch.cuda.synchronize()
        tot = resid + xin @ Wd.t()
        assert torch.allclose(xres, tot, atol=0.02 * tot.std().item(), rtol=1e-3), rnd
        ref = tot * torch.rsqrt(tot.pow(2).mean(-1, keepdim=True) + 1e-5) * g
        assert torch.allclose(hf, ref, atol=0.03, rtol=1e-2), rnd
        assert float(part[:nb].abs().max()) == 0.0          # left zeroed for the next projection
    assert int(status.item()) == 0 and heap.status() == (0, 0)
    # arg-max merge with one rank: the ids pass through unchanged, twice (both parities)
    merge, merge_off = heap.alloc_tensor((2, 1, 1024, 2), torch.float32)
    for rnd in range(3):
        ids = torch.randint(0, 1000, (70,), device=DEV, dtype=torch.int32)
        vals = _randn(70, seed=80 + rnd)
        want = ids.clone()
        ops.argmax_merge(ids, vals, 70, heap.table, merge_off, 1024)
        torch.cuda.synchronize()
        assert torch.equal(ids, want)
    assert heap.status() == (0, 0)


@pytest.mark.parametrize("B,T,H", [(2, 128, 3), (1, 320, 2), (3, 64, 1)])
def test_attn_train_forward_backward(B, T, H):
    """Training attention (causal, head size 64) against fp32 softmax attention and its autograd gradients, reading the
    fused QKV projection in place; run twice: the kernels use no atomics, so the bits must repeat."""
    from openagents_b200.ops import train_ops as tops
    hd, d = 64, H * 64
    qkv = (_randn(B * T, 3 * d, seed=70) * 0.8).bfloat16()
    d_o = (_randn(B * T, d, seed=71) * 0.5).bfloat16()
    o = torch.zeros((B * T, d), dtype=torch.bfloat16, device=DEV)
    lse = torch.zeros((B, H, T), device=DEV)
    tops.attn_train_fwd(qkv, o, lse, B, T, H, hd)
    q, k, v = (qkv.float().view(B, T, 3, H, hd)[:, :, i].permute(0, 2, 1, 3).clone().requires_grad_(True) for i in range(3))
    s = (q @ k.transpose(-1, -2)) / math.sqrt(hd)
    s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool, device=DEV), 1), float("-inf"))
    ref = torch.softmax(s, -1) @ v                                     # [B, H, T, hd]
    got = o.float().view(B, T, H, hd).permute(0, 2, 1, 3)
    assert torch.allclose(got, ref, atol=2e-2, rtol=2e-2), (got - ref).abs().max().item()
    assert torch.allclose(lse * math.log(2.0), torch.logsumexp(s, -1), atol=2e-3, rtol=1e-3)
    ref.backward(d_o.float().view(B, T, H, hd).permute(0, 2, 1, 3))
    dqkv = torch.zeros_like(qkv)
    dsum = torch.empty((B, H, T), device=DEV)
    tops.attn_train_bwd(qkv, o, d_o, lse, dsum, dqkv, B, T, H, hd)
    g = dqkv.float().view(B, T, 3, H, hd)
    for i, r in enumerate((q.grad, k.grad, v.grad)):
        mine = g[:, :, i].permute(0, 2, 1, 3)
        rel = (mine - r).norm().item() / r.norm().item()
        assert rel < 2e-2, (i, rel)
    again = torch.zeros_like(qkv)
    o2 = torch.zeros_like(o)
    tops.attn_train_fwd(qkv, o2, lse, B, T, H, hd)
    tops.attn_train_bwd(qkv, o2, d_o, lse, dsum, again, B, T, H, hd)
    assert torch.equal(o, o2) and torch.equal(dqkv, again)


@pytest.mark.parametrize("M,N,K", [(2304, 768, 2048), (200, 136, 100), (768, 3072, 4096), (50304, 768, 512)])
def test_gemm_mn_major_operands(M, N, K):
    """D = A^T B with both operands read as they lie in memory ([K][M] and [K][N]): the weight-gradient GEMM dW = dy^T x.
    Plain store, fp32 accumulation on top of existing contents, a K that is not a multiple of the 64-row K block."""
    ops = _ops()
    A = _randn(K, M, seed=90).bfloat16()
    B = _randn(K, N, seed=91).bfloat16()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ref = A.float().t() @ B.float()
    tol = 4e-3 * math.sqrt(K) + 1e-3
    out = torch.zeros((M, N), device=DEV)
    ops.gemm_bf16(A, B, M, N, K, out_f32=out, mn_major=True, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert (out - ref).abs().max().item() < tol, (out - ref).abs().max().item()
    acc = torch.full((M, N), 0.5, device=DEV)
    ops.gemm_bf16(A, B, M, N, K, out_f32=acc, accumulate=True, mn_major=True, status=status)
    assert (acc - ref - 0.5).abs().max().item() < tol
    # against the K-major path on explicit transposes
    out2 = torch.zeros((M, N), device=DEV)
    ops.gemm_bf16(A.t().contiguous(), B.t().contiguous(), M, N, (K + 7) // 8 * 8 if K % 8 == 0 else K, out_f32=out2, status=status) if K % 8 == 0 else None
    if K % 8 == 0:
        assert (out2 - out).abs().max().item() < tol


def test_stream_triad_probe():
    """The bandwidth probe's triad kernel computes a = b + 3 c (checked inside) and reports a plausible rate."""
    from openagents_b200.utils.bandwidth_probe import stream_triad_gbs
    assert stream_triad_gbs(DEV, n=1 << 24) > 200.0


@pytest.mark.parametrize("t,nb,hd", [(GgmlType.Q4_K, 1, 128), (GgmlType.Q4_K, 3, 64), (GgmlType.Q6_K, 4, 128), (GgmlType.Q8_0, 2, 64),
                                     (GgmlType.BF16, 1, 64)])
def test_matvec_with_rotary_and_cache_write(t, nb, hd):
    """The fused QKV projection with the rotary embedding and the paged-cache write in its epilogue equals the plain
    mat-vec followed by the rotary kernel (same sums, same table; the two compilations may contract the rotation into
    fused multiply-adds differently, hence a last-bit tolerance), including a position beyond the table, a
    token that writes no cache, a bias, and a matrix small enough for the 8-row CTAs."""
    ops = _ops()
    Hq, Hkv, K = 4, 2, 512
    N = (Hq + 2 * Hkv) * hd
    W = _randn(N, K, seed=90, scale=0.05)
    w = _qweight(W, t)
    bias = _randn(N, seed=91) * 0.1
    x = _randn(nb, K, seed=92)
    xq, xd, xs = _alloc_q(nb, K)
    ops.quantize_x(x, xq, xd, xs)
    pos = torch.tensor([5, 1023, 9000, 0][:nb], dtype=torch.int32, device=DEV)      # 9000 is beyond the table
    slot = torch.tensor([3, 17, -1, 40][:nb], dtype=torch.int32, device=DEV)         # -1 writes no cache
    tab = ops.rope_table(8192, hd, 500000.0, DEV)
    scale = 1.0 / math.sqrt(hd)
    # reference: two kernels
    y = torch.empty((nb, N), device=DEV)
    ops.matvec(w.wt, w.main, w.plane2, N, K, nb, xq=xq, xd=xd, xs16=xs, xf=x, epi=ops.EPI_STORE, bias=bias, y=y, ldy=N)
    kc0 = torch.zeros((4, Hkv, 16, hd), dtype=torch.float16, device=DEV)
    vc0 = torch.zeros_like(kc0)
    q0 = torch.zeros((nb, Hq * hd), device=DEV)
    ops.rope_kv(y, pos, slot, q0, None, kc0, vc0, Hq, Hkv, hd, 16, 500000.0, 0, scale, table=tab)
    # fused
    kc1, vc1, q1 = torch.zeros_like(kc0), torch.zeros_like(kc0), torch.zeros_like(q0)
    ops.matvec_rope_kv(w, nb, pos, slot, q1, kc1, vc1, Hq, Hkv, hd, 16, 500000.0, scale, xq=xq, xd=xd, xs16=xs, xf=x, bias=bias, table=tab)
    torch.cuda.synchronize()
    assert torch.allclose(q1, q0, atol=1e-6, rtol=1e-5) and torch.equal(vc1, vc0)
    assert torch.allclose(kc1.float(), kc0.float(), atol=2e-3, rtol=2e-3)
    assert float(q0.abs().max()) > 0 and float(kc0.abs().max()) > 0
    assert torch.equal(kc1 == 0, kc0 == 0)                    # exactly the same cache slots were written


def test_freivalds_arithmetic_on_the_device_is_exact():
    """The prime-field kernels of training verification against the host arithmetic: bit-identical mat-vec and product, a
    correct product verifies, a single wrong cell is caught by the random challenge, a compensated error only by the exact check."""
    import numpy as np
    from openagents_b200.control.verification import DEFAULT_MODULUS, freivalds_check_cuda, matmul_mod, matvec_mod
    ops = _ops()
    p = DEFAULT_MODULUS
    rng = np.random.default_rng(0)
    n, k, m = 70, 533, 45
    A, B = rng.integers(0, p, (n, k)), rng.integers(0, p, (k, m))
    A[0, :] = p - 1                                           # the largest residues: products near 2^62
    B[:, 0] = p - 1
    r = rng.integers(0, p, m)
    C = matmul_mod(A, B, p)
    dev = lambda a: torch.as_tensor(np.asarray(a, dtype=np.int64)).to(torch.int32).cuda()
    assert np.array_equal(ops.modp_matvec(dev(B), dev(r), p).cpu().numpy().astype(np.int64), matvec_mod(B, r, p))
    assert np.array_equal(ops.modp_matmul(dev(A), dev(B), p).cpu().numpy().astype(np.int64), C)
    assert freivalds_check_cuda(A, B, C, r, p, exact=True) == {"verified": True, "code": None, "mismatchedRows": 0, "mismatchedCells": 0}
    wrong = C.copy()
    wrong[3, 7] = (wrong[3, 7] + 1) % p
    got = freivalds_check_cuda(A, B, wrong, r, p)
    assert got["verified"] is False and got["mismatchedRows"] == 1 and got["code"] == "FreivaldsMismatch"
    # an error the challenge cannot see (it lies in the null space of r): only the exact product catches it
    r2 = r.copy()
    r2[5] = 0
    sneaky = C.copy()
    sneaky[9, 5] = (sneaky[9, 5] + 12345) % p
    assert freivalds_check_cuda(A, B, sneaky, r2, p)["verified"] is True
    ex = freivalds_check_cuda(A, B, sneaky, r2, p, exact=True)
    assert ex["verified"] is False and ex["mismatchedCells"] == 1
    assert freivalds_check_cuda(A, B[:-1], C, r, p)["code"] == "DimensionMismatch"
