"""Small single-kernel workloads for profiler captures.

    python -m openagents_b200.utils.profile_target <case> [launches]

Each case sets up one kernel on a problem that is larger than L2 but holds well under a gigabyte on
the device, launches it a few times and exits, so a capture with ``ncu -k regex:<kernel> -c 1`` ends
by itself in seconds.  Cases: qgemm64, qgemm_lm, gemm, matvec, attn_decode, attn_prefill, and
``step64`` / ``step1``: whole decode steps (batch 64 / 1, context 2048) of a 4-layer Llama-3-8B-shape
engine without graphs, for a per-kernel launch list; ``moe_step``: the same for a 2-layer gpt-oss-20b-shape
expert engine at batch 256.
"""
from __future__ import annotations

import math
import sys

import torch

from ..gguf import GgmlType
from ..ops import cuda_ops as ops
from .microbench import DEV, _rand_q


def main():
    case = sys.argv[1] if len(sys.argv) > 1 else "qgemm64"
    n = int(sys.argv[2]) if len(sys.argv) > 2 else 3
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    if case in ("qgemm64", "qgemm_lm"):
        N, K, t = (28672, 4096, GgmlType.Q4_K) if case == "qgemm64" else (128256, 4096, GgmlType.Q6_K)
        w = _rand_q(N, K, t)
        x = torch.randn(64, K, device=DEV).bfloat16()
        y = torch.zeros((64, N), device=DEV)
        fn = lambda: ops.qgemm(w, x, 64, y, N, epi=ops.QEPI_ADD, split_k=0, status=status)
    elif case == "gemm":
        M, N, K = 2048, 28672, 4096
        A, B = torch.randn(M, K, device=DEV).bfloat16(), torch.randn(N, K, device=DEV).bfloat16()
        out = torch.empty((M, N), dtype=torch.bfloat16, device=DEV)
        fn = lambda: ops.gemm_bf16(A, B, M, N, K, out_bf16=out, tile_n=256, status=status)
    elif case == "matvec":
        N, K = 14336, 4096
        w = _rand_q(2 * N, K, GgmlType.Q4_K)
        x = torch.randn(1, K, device=DEV)
        xq, xd, xs = torch.empty((1, K), dtype=torch.int8, device=DEV), torch.empty((1, K // 32), device=DEV), torch.empty((1, K // 16), device=DEV)
        ops.quantize_x(x, xq, xd, xs)
        oq, od, os16 = torch.empty((1, N), dtype=torch.int8, device=DEV), torch.empty((1, N // 32), device=DEV), torch.empty((1, N // 16), device=DEV)
        fn = lambda: ops.matvec(w.wt, w.main, w.plane2, N, K, 1, xq=xq, xd=xd, xs16=xs, epi=ops.EPI_SWIGLU_Q8, oq=oq, od=od, os16=os16)
    elif case == "attn_decode":
        B, ctx, Hq, Hkv, hd = 64, 2304, 32, 8, 128
        pages = (ctx + 15) // 16
        kc = torch.randn((B * pages + 1, Hkv, 16, hd), device=DEV).half()
        vc = torch.randn((B * pages + 1, Hkv, 16, hd), device=DEV).half()
        table = torch.arange(B * pages, dtype=torch.int32, device=DEV).view(B, pages) + 1
        lens = torch.full((B,), ctx, dtype=torch.int32, device=DEV)
        q = torch.randn(B, Hq * hd, device=DEV) / math.sqrt(hd)
        out = torch.empty((B, Hq * hd), dtype=torch.bfloat16, device=DEV)
        S = 4
        scratch = torch.empty(ops.attn_decode_scratch_floats(B, Hq, Hkv, hd, S), device=DEV)
        counters = torch.zeros(B * Hkv, dtype=torch.int32, device=DEV)
        fn = lambda: ops.attn_decode(q, kc, vc, table, lens, B, Hq, Hkv, hd, S=S, out_bf16=out, scratch=scratch, counters=counters)
    elif case == "attn_prefill":
        T, Hq, Hkv, hd = 2048, 32, 8, 128
        pages = T // 16
        kc = torch.randn((pages + 1, Hkv, 16, hd), device=DEV).half()
        vc = torch.randn((pages + 1, Hkv, 16, hd), device=DEV).half()
        table = torch.arange(pages, dtype=torch.int32, device=DEV).view(1, pages) + 1
        q = (torch.randn(T, Hq * hd, device=DEV) / math.sqrt(hd)).half()
        out = torch.empty((T, Hq * hd), dtype=torch.bfloat16, device=DEV)
        z, tl = torch.zeros(1, dtype=torch.int32, device=DEV), torch.full((1,), T, dtype=torch.int32, device=DEV)
        fn = lambda: ops.attn_prefill(q, kc, vc, table, pages, z, tl, tl, 1, T, Hq, Hkv, hd, out_bf16=out)
    elif case in ("step64", "step1"):
        from ..models.config import LLAMA3_8B
        from ..models.engine import LlamaEngine
        from ..models.qweight import RandomSource
        from ..models.weights import PLAN_Q4_K
        B, ctx = (64, 2048) if case == "step64" else (1, 2048)
        cfg = LLAMA3_8B.with_(n_layers=4)
        eng = LlamaEngine(cfg, RandomSource(cfg, PLAN_Q4_K, 0, DEV), device=DEV, max_batch=B, max_ctx=ctx + 64, max_tokens=2048)
        g = torch.Generator().manual_seed(1)
        for b in range(B):
            eng.begin(b)
            eng.forward_tokens([b], [torch.randint(0, cfg.vocab, (ctx,), generator=g).tolist()])
        ids = list(range(B))
        status = eng.status
        fn = lambda: eng.decode(ids, [5] * B, use_graph=False)
    elif case == "moe_step":
        from ..models.config import GPT_OSS_20B
        from ..models.moe_engine import MoEEngine
        from ..models.qweight import RandomSource
        from ..models.weights import PLAN_MOE
        B, ctx = 256, 128
        cfg = GPT_OSS_20B.with_(n_layers=2)
        eng = MoEEngine(cfg, RandomSource(cfg, PLAN_MOE, 0, DEV), device=DEV, max_batch=B, max_ctx=ctx + 64, max_tokens=4096)
        g = torch.Generator().manual_seed(1)
        for b0 in range(0, B, 32):
            ids = list(range(b0, b0 + 32))
            for b in ids:
                eng.begin(b)
            eng.forward_tokens(ids, [torch.randint(0, cfg.vocab, (ctx,), generator=g).tolist() for _ in ids])
        ids = list(range(B))
        status = eng.status
        fn = lambda: eng.decode(ids, [5] * B, use_graph=False)
    else:
        raise SystemExit(f"unknown case {case}")
    fn()                                  # warm-up outside the profiled range
    torch.cuda.synchronize()
    torch.cuda.profiler.start()           # honoured by `ncu --profile-from-start off`
    for _ in range(n):
        fn()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    assert int(status.item()) == 0
    print("ok", case)


if __name__ == "__main__":
    main()
