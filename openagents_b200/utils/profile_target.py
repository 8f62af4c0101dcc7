"""Small single-kernel workloads for profiler captures.

    python -m openagents_b200.utils.profile_target <case> [launches]

Each case sets up one kernel on a problem that is larger than L2 but holds well under a gigabyte on
the device, launches it a few times and exits, so a capture with ``ncu -k regex:<kernel> -c 1`` ends
by itself in seconds.  Cases: qgemm64, qgemm_lm, gemm, gemm_k768, matvec, attn_decode, attn_prefill, attn_prefill_tc05, and
``step64`` / ``step1``: whole decode steps (batch 64 / 1, context 2048) of a 4-layer Llama-3-8B-shape
engine without graphs, for a per-kernel launch list; ``moe_step``: the same for a 2-layer gpt-oss-20b-shape
expert engine at batch 256; ``moe_ffn``: one expert layer at 4096 tokens; ``gemm_ar64`` / ``gemm_ar2048``: the
row-parallel GEMM with its fused all-reduce epilogue; ``gemm_ag2048`` / ``gemm_rs2048``: the sequence-sharded prefill
pair (norm + all-gather push -> GEMM, GEMM -> reduce-scatter); ``zero_adamw``: the sharded optimizer step;
``attn_train_fwd`` / ``attn_train_bwd``: training attention at GPT-2-small's shape (16 x 1024 tokens, 12 heads of 64);
``gemm_mn``: the weight-gradient GEMM (both operands read token-major); ``norm_slots``: the RMSNorm that is the tensor-parallel
all-reduce, 64 rows of 4096 on a one-rank heap.
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
        y = torch.zeros((64, N // 2), dtype=torch.bfloat16, device=DEV) if case == "qgemm64" else torch.zeros((64, N), device=DEV)
        if case == "qgemm64":      # gate/up projection with the SwiGLU epilogue, the largest matrix of a layer
            fn = lambda: ops.qgemm(w, x, 64, out_bf16=y, ldo=N // 2, epi=ops.QEPI_SWIGLU, status=status)
        else:
            fn = lambda: ops.qgemm(w, x, 64, out_f32=y, epi=ops.QEPI_STORE, status=status)
    elif case in ("gemm", "gemm_k768"):
        M, N, K = (2048, 28672, 4096) if case == "gemm" else (16384, 3072, 768)      # prefill gate/up; GPT-2 feed-forward expansion
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
    elif case in ("attn_prefill", "attn_prefill_tc05"):
        T, Hq, Hkv, hd = 2048, 32, 8, 128
        pages = T // 16
        kc = torch.randn((pages + 1, Hkv, 16, hd), device=DEV).half()
        vc = torch.randn((pages + 1, Hkv, 16, hd), device=DEV).half()
        table = torch.arange(pages, dtype=torch.int32, device=DEV).view(1, pages) + 1
        q = (torch.randn(T, Hq * hd, device=DEV) / math.sqrt(hd)).half()
        out = torch.empty((T, Hq * hd), dtype=torch.bfloat16, device=DEV)
        z, tl = torch.zeros(1, dtype=torch.int32, device=DEV), torch.full((1,), T, dtype=torch.int32, device=DEV)
        if case == "attn_prefill":
            fn = lambda: ops.attn_prefill(q, kc, vc, table, pages, z, tl, tl, 1, T, Hq, Hkv, hd, out_bf16=out)
        else:
            fn = lambda: ops.attn_prefill_tc05(q, kc, vc, table, z, tl, tl, 1, T, Hq, Hkv, out_bf16=out, status=status)
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
    elif case == "moe_ffn":
        # one gpt-oss-20b-shape expert layer at 4096 tokens: fused router+dispatch, then the two grouped GEMMs
        from ..models.config import GPT_OSS_20B
        from ..models.moe_engine import MoEEngine
        from ..models.qweight import RandomSource
        from ..models.weights import PLAN_MOE
        cfg = GPT_OSS_20B.with_(n_layers=1, vocab=2048)
        eng = MoEEngine(cfg, RandomSource(cfg, PLAN_MOE, 0, DEV), device=DEV, max_batch=8, max_ctx=256, max_tokens=4096)
        T = 4096
        hb = torch.randn(T, cfg.d_model, device=DEV).bfloat16()
        eng.hf32[:T].copy_(hb.float())
        x = eng.x[:T]
        status = eng.status

        def fn():
            ops.moe_zero(eng.counts)
            eng._ffn_dense(0, eng.layers[0], T, x, hb, None, None)
    elif case in ("gemm_ar64", "gemm_ar2048"):
        # row-parallel down projection with the all-reduce fused into the epilogue (one-rank heap: the
        # reductions land in this GPU's own replica; on N ranks the same instructions go through NVSwitch)
        from ..parallel.tp import TPComm
        M = 64 if case == "gemm_ar64" else 2048
        N, K = 4096, 14336
        comm = TPComm(0, 1, DEV, heap_bytes=M * N * 4 + (1 << 20))
        xh, _ = comm.alloc_tensor((M, N), torch.float32)
        A, B = torch.randn(M, K, device=DEV).bfloat16(), torch.randn(N, K, device=DEV).bfloat16()
        fn = lambda: comm.gemm_allreduce(A, B, M, xh, status=status)
    elif case in ("gemm_ag2048", "gemm_rs2048"):
        # sequence-sharded prefill pair on a one-rank heap: norm + all-gather push -> QKV GEMM that waits for the
        # rows' owners tile by tile; output GEMM with the reduce-scatter in its epilogue
        from ..parallel.tp import TPComm
        M, d = 2048, 4096
        comm = TPComm(0, 1, DEV, heap_bytes=M * d * 8 + (1 << 20))
        xh, x_off = comm.alloc_tensor((M, d), torch.float32)
        hbf, hb_off = comm.alloc_tensor((M, d), torch.bfloat16)
        xh.normal_()
        gain = torch.ones(d, device=DEV)
        table = comm.heap.table
        if case == "gemm_ag2048":
            N = 6144
            B = torch.randn(N, d, device=DEV).bfloat16()
            out = torch.empty((M, N), device=DEV)
            epoch = [0]

            def fn():
                ops.rmsnorm_allgather(xh, gain, 1e-5, 0, M, hb_off, table)
                epoch[0] += 1
                ops.gemm_bf16(hbf, B, M, N, d, out_f32=out, status=status, sym=table, ag_rows_per_rank=M, ag_epoch=epoch[0])
        else:
            K = 4096
            A, B = torch.randn(M, K, device=DEV).bfloat16(), torch.randn(d, K, device=DEV).bfloat16()
            fn = lambda: ops.gemm_bf16(A, B, M, d, K, ldc=d, status=status, sym_mode=ops.SYM_RSCATTER_ROWS, sym=table,
                                       sym_off=x_off, rows_per_rank=M)
    elif case in ("attn_train_fwd", "attn_train_bwd"):
        from ..ops import train_ops as tops
        B, T, H, hd = 16, 1024, 12, 64
        qkv = (torch.randn(B * T, 3 * H * hd, device=DEV) * 0.5).bfloat16()
        o, d_o, dqkv = (torch.empty((B * T, H * hd), dtype=torch.bfloat16, device=DEV), (torch.randn(B * T, H * hd, device=DEV) * 0.1).bfloat16(),
                        torch.empty((B * T, 3 * H * hd), dtype=torch.bfloat16, device=DEV))
        lse, dsum = torch.empty((B, H, T), device=DEV), torch.empty((B, H, T), device=DEV)
        tops.attn_train_fwd(qkv, o, lse, B, T, H, hd)
        if case == "attn_train_fwd":
            fn = lambda: tops.attn_train_fwd(qkv, o, lse, B, T, H, hd)
        else:
            fn = lambda: tops.attn_train_bwd(qkv, o, d_o, lse, dsum, dqkv, B, T, H, hd)
    elif case == "gemm_mn":
        # dW = dY^T X of GPT-2-small's feed-forward expansion: 3072 x 768 over 16384 tokens, operands as stored
        M, N, K = 3072, 768, 16384
        A, B = torch.randn(K, M, device=DEV).bfloat16(), torch.randn(K, N, device=DEV).bfloat16()
        out = torch.empty((M, N), device=DEV)
        fn = lambda: ops.gemm_bf16(A, B, M, N, K, out_f32=out, status=status, mn_major=True)
    elif case == "norm_slots":
        from ..parallel.symm import SymmHeap
        rows, d = 64, 4096
        heap = SymmHeap(64 << 20, DEV)
        _, slots_off = heap.alloc_tensor((2, 1, rows, d), torch.float32)
        part, xres, gain = torch.randn(rows, d, device=DEV), torch.randn(rows, d, device=DEV), torch.ones(d, device=DEV)
        hb = torch.empty((rows, d), dtype=torch.bfloat16, device=DEV)
        fn = lambda: ops.rmsnorm(xres, gain, 1e-5, hb=hb, slots=(heap.table, slots_off, rows, part))
    elif case == "zero_adamw":
        # sharded AdamW step on GPT-2-small's 124M parameters, one-rank heap: reduce-scatter + norm, then
        # clip + AdamW + bf16 cast + all-gather push
        from ..ops import train_ops as tops
        from ..parallel.symm import SymmHeap
        n_par = 124_475_904
        heap = SymmHeap(n_par * 6 + (1 << 20), DEV)
        grads, goff = heap.alloc_tensor((n_par,), torch.float32)
        params, poff = heap.alloc_tensor((n_par,), torch.bfloat16)
        grads.normal_(0, 1e-3)
        gsh, master, m, v = (torch.zeros(n_par, device=DEV) for _ in range(4))
        master.normal_(0, 0.02)
        norm2 = torch.zeros(4, device=DEV)

        def fn():
            norm2.zero_()
            tops.zero_reduce_norm(heap.table, goff, 0, n_par, gsh, norm2)
            tops.zero_adamw_gather(heap.table, poff, 0, n_par, gsh, master, m, v, norm2, 6e-4, 0.9, 0.95, 1e-8, 0.1, 0.1, 0.05, 1.0, n_par)
    else:
        raise SystemExit(f"unknown case {case}")
    fn()                                  # warm-up outside the profiled range
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()           # honoured by `ncu --profile-from-start off`
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    assert int(status.item()) == 0
    print("ok", case, f"{e0.elapsed_time(e1) * 1000 / n:.1f} us per call (CUDA events, {n} calls back to back; not valid under a profiler)")


if __name__ == "__main__":
    main()
