"""Per-kernel timing against the measured roofline.

    python -m openagents_b200.utils.microbench [matvec|attn|gemm|all]

Each case is timed with CUDA events after warm-up, with a buffer larger than L2 written between
iterations so operands are read from HBM.  Fractions are "of measured": achieved bytes/s over the
copy bandwidth and achieved FLOP/s over the cuBLAS bf16 throughput recorded in MEASURED_PEAKS.json
(fallback 6650 GB/s and 1590 TFLOP/s when the file is absent).
"""
from __future__ import annotations

import json
import math
import os
import sys

import torch

from ..gguf import GgmlType
from ..gguf import torch_codecs as tc
from ..models.qweight import QWeight, RawTensor
from ..ops import cuda_ops as ops

DEV = "cuda"


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


_flush = None


def flush_l2():
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)
    _flush.fill_(1)


def timeit(fn, iters=20, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2] * 1e-3


def _rand_q(N, K, t):
    x = torch.randn(N, K, device=DEV) * 0.02
    return QWeight.from_raw(RawTensor(t, (N, K), tc.quantize(x, t)))


def bench_matvec(rows):
    hbm, _, tag = peaks()
    a = torch.zeros(32, device=DEV)
    b = torch.zeros(32, device=DEV)
    rows.append(f"event-pair floor (32-element add kernel): {timeit(lambda: ops.add_inplace(a, b))*1e6:6.1f} us")
    shapes = [("qkv", 6144, 4096, GgmlType.Q4_K, False), ("o", 4096, 4096, GgmlType.Q4_K, False),
              ("gate_up", 14336, 4096, GgmlType.Q4_K, True), ("down", 4096, 14336, GgmlType.Q4_K, False),
              ("lm_head", 128256, 4096, GgmlType.Q6_K, False)]
    for name, N, K, t, dual in shapes:
        w = _rand_q(N * (2 if dual else 1), K, t)
        for nb in (1, 4, 8):
            x = torch.randn(nb, K, device=DEV)
            xq = torch.empty((nb, K), dtype=torch.int8, device=DEV)
            xd = torch.empty((nb, K // 32), device=DEV)
            xs = torch.empty((nb, K // 16), device=DEV)
            ops.quantize_x(x, xq, xd, xs)
            y = torch.zeros((nb, N), device=DEV)
            oq, od, os16 = torch.empty((nb, N), dtype=torch.int8, device=DEV), torch.empty((nb, N // 32), device=DEV), torch.empty((nb, N // 16), device=DEV)
            if dual:
                fn = lambda: ops.matvec(w.wt, w.main, w.plane2, N, K, nb, xq=xq, xd=xd, xs16=xs, epi=ops.EPI_SWIGLU_Q8, oq=oq, od=od, os16=os16)
            else:
                fn = lambda: ops.matvec(w.wt, w.main, w.plane2, N, K, nb, xq=xq, xd=xd, xs16=xs, epi=ops.EPI_STORE, y=y, ldy=N)
            s = timeit(fn)
            gbs = w.nbytes() / s / 1e9
            rows.append(f"matvec {name:8s} N={N:6d} K={K:5d} {t.name} nb={nb}: {s*1e6:8.1f} us  {gbs:7.0f} GB/s  {gbs/hbm:5.2f} of {tag} HBM")


def bench_attn(rows):
    hbm, _, tag = peaks()
    Hq, Hkv, hd = 32, 8, 128
    for B, ctx in ((1, 2304), (8, 2304), (64, 2304)):
        pages = (ctx + 15) // 16
        n_pages = B * pages + 1
        kc = torch.randn((n_pages, Hkv, 16, hd), device=DEV).half()
        vc = torch.randn((n_pages, Hkv, 16, hd), device=DEV).half()
        table = (torch.arange(B * pages, dtype=torch.int32, device=DEV).view(B, pages) + 1)
        lens = torch.full((B,), ctx, dtype=torch.int32, device=DEV)
        q = torch.randn(B, Hq * hd, device=DEV) / math.sqrt(hd)
        out = torch.empty((B, Hq * hd), dtype=torch.bfloat16, device=DEV)
        for S in ((1, 4, 9, 18, 36) if B == 1 else (1, 2, 5) if B == 8 else (1, 2, 4)):
            scratch = torch.empty(ops.attn_decode_scratch_floats(B, Hq, Hkv, hd, S), device=DEV)
            counters = torch.zeros(B * Hkv, dtype=torch.int32, device=DEV)
            fn = lambda: ops.attn_decode(q, kc, vc, table, lens, B, Hq, Hkv, hd, S=S, out_bf16=out, scratch=scratch, counters=counters)
            s = timeit(fn)
            byts = 2 * B * ctx * Hkv * hd * 2
            rows.append(f"attn_decode B={B:3d} ctx={ctx} S={S:2d}: {s*1e6:8.1f} us  {byts/s/1e9:7.0f} GB/s  {byts/s/1e9/hbm:5.2f} of {tag} HBM")
    # prefill
    for T in (2048,):
        pages = (T + 15) // 16
        kc = torch.randn((pages + 1, Hkv, 16, hd), device=DEV).half()
        vc = torch.randn((pages + 1, Hkv, 16, hd), device=DEV).half()
        table = (torch.arange(pages, dtype=torch.int32, device=DEV).view(1, pages) + 1)
        q = (torch.randn(T, Hq * hd, device=DEV) / math.sqrt(hd)).half()
        out = torch.empty((T, Hq * hd), dtype=torch.bfloat16, device=DEV)
        z = torch.zeros(1, dtype=torch.int32, device=DEV)
        tl = torch.full((1,), T, dtype=torch.int32, device=DEV)
        fn = lambda: ops.attn_prefill(q, kc, vc, table, pages, z, tl, tl, 1, T, Hq, Hkv, hd, out_bf16=out)
        s = timeit(fn)
        fl = 4 * T * T * Hq * hd / 2
        _, tf, tag2 = peaks()
        rows.append(f"attn_prefill T={T}: {s*1e6:8.1f} us  {fl/s/1e12:6.1f} TFLOP/s (causal)  {fl/s/1e12/tf:5.2f} of {tag2} bf16")


def bench_gemm(rows):
    _, tf, tag = peaks()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for M, N, K in ((2048, 6144, 4096), (2048, 28672, 4096), (2048, 4096, 14336), (8192, 8192, 8192), (64, 6144, 4096),
                    (64, 28672, 4096), (16384, 2304, 768), (16384, 768, 3072), (16384, 3072, 768)):
        A = torch.randn(M, K, device=DEV).bfloat16()
        B = torch.randn(N, K, device=DEV).bfloat16()
        out = torch.empty((M, N), dtype=torch.bfloat16, device=DEV)
        for tile in (64, 128, 256):
            fn = lambda: ops.gemm_bf16(A, B, M, N, K, out_bf16=out, tile_n=tile, status=status)
            s = timeit(fn, iters=10)
            fl = 2.0 * M * N * K
            rows.append(f"gemm M={M:5d} N={N:5d} K={K:5d} tile_n={tile:3d}: {s*1e6:9.1f} us  {fl/s/1e12:7.1f} TFLOP/s  {fl/s/1e12/tf:5.2f} of {tag} bf16")
        ref = timeit(lambda: torch.matmul(A, B.t(), out=out), iters=10)
        rows.append(f"     torch.matmul (library reference)       : {ref*1e6:9.1f} us  {2.0*M*N*K/ref/1e12:7.1f} TFLOP/s")
    assert int(status.item()) == 0


def bench_qgemm(rows):
    """The projections of a Llama-3-8B layer (and the LM head) on the fused-dequant GEMM at decode batch sizes, judged
    against the copy bandwidth over the PACKED weight bytes.  Each timing is a CUDA graph over several different
    weight matrices (together larger than L2), so neither the host launch path nor a warm L2 is in the number.
    ``torch.matmul`` on a bf16 copy of the same matrix is the library reference (it reads 3.5x the bytes)."""
    hbm, _, tag = peaks()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    shapes = (("qkv", 6144, 4096, GgmlType.Q4_K, "add", 8), ("wo", 4096, 4096, GgmlType.Q4_K, "add", 8),
              ("gate_up", 28672, 4096, GgmlType.Q4_K, "swiglu", 4), ("down", 4096, 14336, GgmlType.Q4_K, "add", 6),
              ("lm_head", 128256, 4096, GgmlType.Q6_K, "store", 2))
    for name, N, K, t, mode, R in shapes:
        ws = [_rand_q(N, K, t) for _ in range(R)]
        for T in (16, 64):
            x = torch.randn(T, K, device=DEV).bfloat16()
            out = torch.zeros((T, N), device=DEV)
            outb = torch.zeros((T, N // 2), dtype=torch.bfloat16, device=DEV)

            def launch(w):
                if mode == "swiglu":
                    ops.qgemm(w, x, T, out_bf16=outb, ldo=N // 2, epi=ops.QEPI_SWIGLU, status=status)
                elif mode == "add":
                    ops.qgemm(w, x, T, out_f32=out, epi=ops.QEPI_ADD, status=status)
                else:
                    ops.qgemm(w, x, T, out_f32=out, epi=ops.QEPI_STORE, status=status)

            for w in ws[:2]:
                launch(w)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for w in ws:
                    launch(w)
            g.replay()
            torch.cuda.synchronize()
            ts = []
            for _ in range(5):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                g.replay()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1) * 1e-3 / R)
            s_ = sorted(ts)[len(ts) // 2]
            gbs = ws[0].nbytes() / s_ / 1e9
            rows.append(f"qgemm {name:8s} N={N:6d} K={K:5d} {t.name} {mode:6s} T={T:3d}: {s_*1e6:8.1f} us  {gbs:6.0f} GB/s packed "
                        f"({gbs/hbm:4.2f} of {tag} HBM)")
            stamps = getattr(ops.lib(), "b200_qgemm_stamps", None) if hasattr(ops, "lib") else None
            if stamps is not None:       # library built with B200_NVCC_DEFINES=QGEMM_STAMPS: CTA 0's MMA thread, summed over the launches above
                import ctypes
                buf = (ctypes.c_longlong * 4)()
                stamps(buf, 1)
                if buf[3]:
                    rows.append(f"      MMA thread of CTA 0: {buf[2] / buf[3]:7.0f} cycles per 256-wide K stage (16 MMAs) from first wait to "
                                f"retirement; waiting for operands {buf[0] / buf[3]:6.0f}, issuing {buf[1] / buf[3]:6.0f} cycles per stage")
        if name != "lm_head":
            Bs = [torch.randn(N, K, device=DEV).bfloat16() for _ in range(R)]
            A = torch.randn(64, K, device=DEV).bfloat16()
            ob = torch.empty((64, N), dtype=torch.bfloat16, device=DEV)
            g = torch.cuda.CUDAGraph()
            torch.matmul(A, Bs[0].t(), out=ob)
            torch.cuda.synchronize()
            with torch.cuda.graph(g):
                for B in Bs:
                    torch.matmul(A, B.t(), out=ob)
            g.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            rows.append(f"      torch.matmul on a bf16 copy, T= 64 (library reference): {e0.elapsed_time(e1) * 1e3 / R:8.1f} us")
            del Bs
        del ws
    assert int(status.item()) == 0


def bench_gemm_small(rows):
    """The four projections of a Llama-3-8B layer at a decode batch of 64 rows: weight-streaming GEMMs, judged
    against the copy bandwidth.  Each timing is a CUDA graph of 8 launches over 8 different weight matrices
    (together larger than L2), so that neither the host's launch path nor a warm L2 is in the number.
    ``store``: plain fp32 store (no split K); ``add``: accumulate into the output (split K allowed)."""
    hbm, _, tag = peaks()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    M, R = 64, 8
    shapes = (("qkv", 6144, 4096), ("wo", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336))
    if len(sys.argv) > 2 and sys.argv[2] == "ksweep":      # time against K at fixed N: intercept = per-launch cost, slope = per K block
        shapes = tuple((f"k{K}", 6144, K) for K in (64, 512, 1024, 2048, 4096, 8192))
    for name, N, K in shapes:
        A = torch.randn(M, K, device=DEV).bfloat16()
        Bs = [torch.randn(N, K, device=DEV).bfloat16() for _ in range(R)]
        out = torch.zeros((M, N), device=DEV)

        def timed(launch):
            for B in Bs[:2]:
                launch(B)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for B in Bs:
                    launch(B)
            g.replay()
            torch.cuda.synchronize()
            ts = []
            for _ in range(5):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                g.replay()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1) * 1e-3 / R)
            return sorted(ts)[len(ts) // 2]

        for mode in ("store", "add"):
            for tile in (0, 64, 128, 256):
                s = timed(lambda B: ops.gemm_bf16(A, B, M, N, K, out_f32=out, accumulate=(mode == "add"), tile_n=tile, status=status))
                gbs = N * K * 2 / s / 1e9
                rows.append(f"gemm64 {name:8s} N={N:5d} K={K:5d} {mode:5s} tile_n={tile:3d}: {s*1e6:7.1f} us  {gbs:6.0f} GB/s  {gbs/hbm:4.2f} of {tag} HBM")
        outb = torch.empty((M, N), dtype=torch.bfloat16, device=DEV)
        ref = timed(lambda B: torch.matmul(A, B.t(), out=outb))
        rows.append(f"       torch.matmul (library reference)              : {ref*1e6:7.1f} us  {N*K*2/ref/1e9:6.0f} GB/s")
    assert int(status.item()) == 0


def main():
    which = sys.argv[1] if len(sys.argv) > 1 else "all"
    rows = []
    if which in ("matvec", "all"):
        bench_matvec(rows)
    if which in ("attn", "all"):
        bench_attn(rows)
    if which in ("gemm", "all"):
        bench_gemm(rows)
    if which in ("qgemm", "all"):
        bench_qgemm(rows)
    if which in ("gemm64", "all"):
        bench_gemm_small(rows)
    print("\n".join(rows))


if __name__ == "__main__":
    main()
