"""Python faces of the sm_100a kernels (ctypes over ``libb200_cuda.so``).

Every function takes torch CUDA tensors, launches on the current torch stream and raises on a
non-zero return code.  There is no fallback: on a machine with a GPU a missing library is an error.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_long, c_size_t, c_void_p

import torch

from .. import _native

WT_Q4KR, WT_Q6KR, WT_Q8R, WT_BF16, WT_MXFP4R = 0, 1, 2, 3, 4
EPI_STORE, EPI_RESID, EPI_SWIGLU_Q8, EPI_SWIGLU_F32, EPI_ALLREDUCE = 0, 1, 2, 3, 4
SYM_NONE, SYM_ALLREDUCE, SYM_RSCATTER, SYM_RSCATTER_ROWS = 0, 1, 2, 3
EMB_F32, EMB_BF16, EMB_Q8R, EMB_Q6KR = 0, 1, 2, 3
ACT_NONE, ACT_GELU, ACT_SWIGLU_PAIR = 0, 1, 2

_P = c_void_p
_SIGS = {
    "b200_embedding": [_P, _P, c_int, c_int, c_int, _P, _P, c_int, c_int, _P],
    "b200_rmsnorm": [_P, _P, c_float, c_int, c_int, _P, _P, _P, _P, _P, _P, c_int, _P, c_long, c_size_t, c_int, _P, _P],
    "b200_rmsnorm_allgather": [_P, _P, c_float, c_int, c_int, c_int, c_size_t, _P, _P],
    "b200_quantize_x": [_P, c_int, c_int, _P, _P, _P, _P],
    "b200_rope_kv": [_P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_float, _P, c_int, _P],
    "b200_rope_table": [_P, c_int, c_int, c_float, _P],
    "b200_swiglu": [_P, c_int, c_int, _P, _P, c_int, _P],
    "b200_add_inplace": [_P, _P, c_size_t, _P],
    "b200_argmax": [_P, c_int, c_int, _P, _P, c_int, _P, _P],
    "b200_sample_topk": [_P, c_int, c_int, c_float, c_int, c_float, _P, _P, _P, _P],
    "b200_matvec_rope_kv": [c_int, _P, _P, c_int, c_int, _P, _P, _P, _P, _P, _P, _P, _P, c_int, _P, _P, _P, c_int, c_int, c_int,
                            c_int, c_float, c_float, _P],
    "b200_matvec": [c_int, _P, _P, c_int, c_int, c_int, _P, _P, _P, _P, c_int, _P, _P, _P, c_int, _P, _P, _P, _P,
                    c_size_t, c_int, _P],
    "b200_argmax_merge": [_P, _P, c_int, _P, c_size_t, c_int, _P],
    "b200_attn_decode": [_P, _P, _P, _P, c_int, c_int, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P, _P, _P,
                         _P, _P, _P, _P, _P],
    "b200_attn_prefill": [_P, _P, _P, _P, c_int, _P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P, _P, _P],
    "b200_attn_prefill_tc05": [_P, _P, _P, _P, c_int, c_int, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P, _P, _P, _P],
    "b200_gemm_bf16": [_P, _P, c_int, c_int, c_int, c_int, c_int, _P, _P, c_int, _P, _P, _P, c_int, c_int, c_int, c_int,
                       _P, c_int, _P, c_size_t, c_int, c_int, c_int, c_int, c_int, _P],
    "b200_moe_gemm": [_P, _P, c_int, c_int, c_int, c_int, c_int, c_int, _P, c_int, _P, c_int, _P, _P, _P, c_size_t, _P, _P],
    "b200_moe_route_dispatch": [_P, _P, _P, _P, c_int, c_int, c_int, c_int, c_int, c_int, c_size_t, c_size_t, c_size_t, c_size_t,
                                _P, _P, _P, _P, _P],
    "b200_moe_zero": [_P, c_int, _P],
    "b200_set_pdl": [c_int],
    "b200_set_prefetch": [c_int],
    "b200_dequant_bf16": [c_int, _P, _P, _P, c_size_t, c_int, _P],
    "b200_f32_to_bf16": [_P, _P, c_size_t, _P],
    "b200_transpose_bf16": [_P, _P, c_int, c_int, _P],
    "b200_qgemm": [c_int, _P, _P, c_int, c_int, _P, c_int, c_int, _P, _P, c_int, _P, c_int, c_int, _P, _P],
    "b200_decode_advance": [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, _P, _P, c_int, _P],
    "b200_modp_matvec": [_P, _P, _P, c_int, c_int, ctypes.c_uint, _P],
    "b200_modp_matmul": [_P, _P, _P, c_int, c_int, c_int, ctypes.c_uint, _P],
    "b200_count_mismatch": [_P, _P, c_size_t, _P, _P],
}

_lib = None


def lib():
    global _lib
    if _lib is None:
        L = _native.cuda()
        for name, args in _SIGS.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = c_int
        L.b200_attn_decode_scratch_floats.argtypes = [c_int, c_int, c_int, c_int, c_int]
        L.b200_attn_decode_scratch_floats.restype = c_size_t
        _lib = L
        if os.environ.get("B200_PDL", "1") == "0":      # debugging aid: fully serialised launches
            L.b200_set_pdl(0)
        if os.environ.get("B200_PREFETCH", "1") == "0":
            L.b200_set_prefetch(0)
    return _lib


def _p(t):
    return None if t is None else t.data_ptr()


def _sym(table):
    """ctypes pointer to a SymTable structure (or None)."""
    return None if table is None else ctypes.addressof(table)


def _st():
    return torch.cuda.current_stream().cuda_stream


def _check(rc: int, what: str):
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


def embedding(ids, out, emb_type, w, w2=None, vocab_lo=0, vocab_n=None):
    T, D = out.shape
    _check(lib().b200_embedding(_p(ids), _p(out), T, D, emb_type, _p(w), _p(w2), vocab_lo,
                                vocab_n if vocab_n is not None else 2 ** 31 - 1, _st()), "embedding")


def rmsnorm(x, g, eps, xq=None, xd=None, xs16=None, hb=None, hf=None, signal_sym=None, zero=None, slots=None):
    """``signal_sym``: symmetric-heap table; the kernel then ends by telling every rank that this rank has
    finished reading ``x`` (the handshake the fused all-reduce kernels check with ``wait_ready``).
    ``zero``: a contiguous fp32 tensor the kernel clears on the side (the output of a split-K GEMM that follows).
    ``slots``: ``(table, heap offset, rows, part)``: tensor parallel: ``part`` (fp32 [T, D], local) holds this rank's
    partial result of the row-parallel projection before this norm; the kernel all-reduces it through the per-rank slot
    tensor at ``heap offset`` ([2][world][rows][D] fp32 on every rank), adds the sum into ``x`` (in place), normalises
    it, and leaves ``part`` zeroed."""
    T, D = x.shape
    part = None
    if slots is not None:
        table, slot_off, slot_rows, part = slots
        mode = 2
    else:
        table, slot_off, slot_rows = signal_sym, 0, 0
        mode = 1 if signal_sym is not None else 0
    _check(lib().b200_rmsnorm(_p(x), _p(g), eps, T, D, _p(xq), _p(xd), _p(xs16), _p(hb), _p(hf), _sym(table), mode,
                              _p(zero), zero.numel() if zero is not None else 0, slot_off, slot_rows, _p(part), _st()), "rmsnorm")


def rmsnorm_allgather(x, g, eps, row0, n_rows, hb_off, sym):
    """Normalise rows [row0, row0 + n_rows) of ``x`` (fp32 [*, D]) and push them as bf16 into every rank's
    [*, D] tensor at byte offset ``hb_off`` of the symmetric heap; ends by bumping this rank's all-gather counter."""
    _check(lib().b200_rmsnorm_allgather(_p(x), _p(g), eps, row0, n_rows, x.shape[1], hb_off, _sym(sym), _st()), "rmsnorm_allgather")


def quantize_x(x, xq, xd, xs16):
    T, D = x.shape
    _check(lib().b200_quantize_x(_p(x), T, D, _p(xq), _p(xd), _p(xs16), _st()), "quantize_x")


def rope_kv(qkv, pos, slot, q_out, q_out_h, kc, vc, Hq, Hkv, hd, page_size, theta, style, q_scale, table=None):
    """``table``: optional (cos, sin) table from :func:`rope_table`; without it the angles are computed per call."""
    T = qkv.shape[0]
    _check(lib().b200_rope_kv(_p(qkv), _p(pos), _p(slot), _p(q_out), _p(q_out_h), _p(kc), _p(vc), T, Hq, Hkv, hd,
                              page_size, theta, style, q_scale, _p(table), 0 if table is None else table.shape[0], _st()),
           "rope_kv")


def rope_table(n_pos, hd, theta, device):
    """fp32 [n_pos][hd/2][2] table of (cos, sin), computed in double precision on the device."""
    tab = torch.empty((n_pos, hd // 2, 2), dtype=torch.float32, device=device)
    _check(lib().b200_rope_table(_p(tab), n_pos, hd, theta, _st()), "rope_table")
    return tab


def swiglu(gu, F, ob=None, of=None, zero_after=False):
    """``gu`` fp32 [T, 2F] holds (gate_i, up_i) in adjacent columns; writes silu(gate) * up; ``zero_after`` clears ``gu``."""
    T = gu.shape[0]
    _check(lib().b200_swiglu(_p(gu), T, F, _p(ob), _p(of), int(zero_after), _st()), "swiglu")


def add_inplace(x, y):
    _check(lib().b200_add_inplace(_p(x), _p(y), x.numel(), _st()), "add_inplace")


def argmax(logits, out_id, out_val=None, vocab_offset=0, scratch=None):
    T, V = logits.shape
    _check(lib().b200_argmax(_p(logits), T, V, _p(out_id), _p(out_val), vocab_offset, _p(scratch), _st()), "argmax")


def argmax_scratch(T, device):
    """Zeroed scratch that lets :func:`argmax` split each row over many blocks."""
    return torch.zeros(T * 4, dtype=torch.int32, device=device)


def sample_topk(logits, temperature, top_k, top_p, u, out_id, scratch):
    T, V = logits.shape
    _check(lib().b200_sample_topk(_p(logits), T, V, temperature, top_k, top_p, _p(u), _p(out_id), _p(scratch), _st()),
           "sample_topk")


def matvec(wt, w, w2, N, K, nb, xq=None, xd=None, xs16=None, xf=None, epi=EPI_STORE, bias=None, resid=None, y=None,
           ldy=0, oq=None, od=None, os16=None, sym=None, sym_off=0, wait_ready=False):
    """Quantized mat-vec for 1..8 tokens (see ``matvec.cu``).  The SwiGLU epilogues read ``w`` as 2N rows interleaved
    (gate_0, up_0, gate_1, ...)."""
    _check(lib().b200_matvec(wt, _p(w), _p(w2), N, K, nb, _p(xq), _p(xd), _p(xs16), _p(xf), epi, _p(bias), _p(resid),
                             _p(y), ldy, _p(oq), _p(od), _p(os16), _sym(sym), sym_off, int(wait_ready), _st()), "matvec")


def matvec_rope_kv(w, nb, pos, slot, q_out, kc, vc, Hq, Hkv, hd, page_size, theta, q_scale, xq=None, xd=None, xs16=None, xf=None,
                   bias=None, table=None):
    """The fused QKV projection of ``nb`` <= 8 tokens with the rotary embedding (adjacent-pair layout) and the paged-cache
    write in its epilogue: replaces ``matvec(..., EPI_STORE)`` + ``rope_kv`` on the small-batch decode path.  ``w``: a
    ``QWeight`` with (Hq + 2 Hkv) * hd rows."""
    _check(lib().b200_matvec_rope_kv(w.wt, _p(w.main), _p(w.plane2), w.K, nb, _p(xq), _p(xd), _p(xs16), _p(xf), _p(bias), _p(pos),
                                     _p(slot), _p(table), 0 if table is None else table.shape[0], _p(q_out), _p(kc), _p(vc), Hq, Hkv,
                                     hd, page_size, theta, q_scale, _st()), "matvec_rope_kv")


def argmax_merge(out_id, out_val, nb, sym, merge_off, rows):
    """Merge per-shard arg-max results across tensor-parallel ranks in one kernel (see ``decode_ops.cu``)."""
    _check(lib().b200_argmax_merge(_p(out_id), _p(out_val), nb, _sym(sym), merge_off, rows, _st()), "argmax_merge")


def attn_decode_scratch_floats(B, Hq, Hkv, hd, S):
    return lib().b200_attn_decode_scratch_floats(B, Hq, Hkv, hd, S)


def attn_decode(q, kc, vc, page_table, seq_lens, B, Hq, Hkv, hd, window=0, S=1, sinks=None, out_f32=None, out_bf16=None,
                oq=None, od=None, os16=None, scratch=None, counters=None, status=None):
    _check(lib().b200_attn_decode(_p(q), _p(kc), _p(vc), _p(page_table), page_table.shape[1], kc.shape[0], _p(seq_lens), _p(sinks),
                                  B, Hq, Hkv, hd, window, S, _p(out_f32), _p(out_bf16), _p(oq), _p(od), _p(os16),
                                  _p(scratch), _p(counters), _p(status), _st()), "attn_decode")


def attn_prefill(q, kc, vc, page_table, max_pages, q_start, q_len, ctx_len, n_seqs, max_q_len, Hq, Hkv, hd, window=0,
                 sinks=None, out_bf16=None, out_f32=None, lse=None):
    _check(lib().b200_attn_prefill(_p(q), _p(kc), _p(vc), _p(page_table), max_pages, _p(q_start), _p(q_len),
                                   _p(ctx_len), _p(sinks), n_seqs, max_q_len, Hq, Hkv, hd, window, _p(out_bf16),
                                   _p(out_f32), _p(lse), _st()), "attn_prefill")


def attn_prefill_tc05(q16, kc, vc, page_table, q_start, q_len, ctx_len, n_seqs, max_q_len, Hq, Hkv, window=0, sinks=None,
                      out_bf16=None, status=None):
    """Prefill attention on tcgen05 (head dim 128, fp16 q / cache, bf16 out); see ``attn_prefill_tc05.cu``."""
    _check(lib().b200_attn_prefill_tc05(_p(q16), _p(kc), _p(vc), _p(page_table), page_table.shape[1], kc.shape[0], _p(q_start),
                                        _p(q_len), _p(ctx_len), n_seqs, max_q_len, q16.shape[0], Hq, Hkv, window, _p(sinks),
                                        _p(out_bf16), _p(status), _st()), "attn_prefill_tc05")


def gemm_bf16(A, B, M, N, K, lda=None, ldb=None, out_f32=None, out_bf16=None, ldc=None, bias=None, resid_f32=None,
              resid_bf16=None, act=ACT_NONE, accumulate=False, tile_n=0, status=None, sym_mode=SYM_NONE, sym=None,
              sym_off=0, rows_per_rank=0, split_k=0, wait_ready=False, ag_rows_per_rank=0, ag_epoch=0, mn_major=False):
    """D[M][N] = A[M][K] @ B[N][K]^T with fused epilogue (see ``gemm_tc05.cu``).  ``ag_rows_per_rank`` > 0: the rows
    of A are all-gathered by push (``rmsnorm_allgather``) and each tile waits for its owners' counter to reach ``ag_epoch``.
    ``mn_major``: the operands are given as A [K][M] and B [K][N] (row strides ``lda`` / ``ldb``), i.e. D = A^T B: the weight
    gradient dW = dy^T x straight from dy and x, without transposed copies."""
    _check(lib().b200_gemm_bf16(_p(A), _p(B), M, N, K, lda or (M if mn_major else K), ldb or (N if mn_major else K), _p(out_f32), _p(out_bf16), ldc or N,
                                _p(bias), _p(resid_f32), _p(resid_bf16), act, int(accumulate), tile_n, split_k, _p(status),
                                sym_mode, _sym(sym), sym_off, rows_per_rank, int(wait_ready), ag_rows_per_rank, ag_epoch,
                                int(mn_major), _st()), "gemm_bf16")


def set_pdl(on: bool):
    """Turn programmatic dependent launch of the decode-path kernels on or off (on by default)."""
    _check(lib().b200_set_pdl(int(on)), "set_pdl")


def dequant_bf16(wt, w, w2, out, N, K):
    _check(lib().b200_dequant_bf16(wt, _p(w), _p(w2), _p(out), N, K, _st()), "dequant_bf16")


def f32_to_bf16(x, y):
    _check(lib().b200_f32_to_bf16(_p(x), _p(y), x.numel(), _st()), "f32_to_bf16")


def transpose_bf16(x, out):
    R, C = x.shape
    _check(lib().b200_transpose_bf16(_p(x), _p(out), R, C, _st()), "transpose_bf16")


def decode_advance(ids, out_ids, pos, slot, seq_lens, page_table, page_size, B, hist, step_counter, hist_cap):
    _check(lib().b200_decode_advance(_p(ids), _p(out_ids), _p(pos), _p(slot), _p(seq_lens), _p(page_table),
                                     page_table.shape[1], page_size, B, _p(hist), _p(step_counter), hist_cap, _st()),
           "decode_advance")


QEPI_STORE, QEPI_ADD, QEPI_SWIGLU = 0, 1, 2


def qgemm(w, x_bf16, T, out_f32=None, out_bf16=None, ldo=None, bias=None, epi=QEPI_STORE, split_k=0, status=None):
    """out[T][N] (+)= x[T][K] @ dequant(W)[N][K]^T with the dequantization inside the tcgen05 pipeline
    (``qgemm_tc05.cu``).  ``w`` is a QWeight in Q4_K-R or Q6_K-R; its packed planes are read as they are.
    ``QEPI_SWIGLU``: rows of ``w`` are (gate, up) pairs, ``out_bf16`` gets N/2 columns."""
    wt = {WT_Q4KR: 0, WT_Q6KR: 1}[w.wt]
    _check(lib().b200_qgemm(wt, _p(w.main), _p(w.plane2), w.N, w.K, _p(x_bf16), x_bf16.stride(0), T, _p(out_f32), _p(out_bf16),
                            ldo if ldo is not None else w.N, _p(bias), epi, split_k, _p(status), _st()), "qgemm")


# ---------------------------------------------------------------- mixture of experts
def moe_route_dispatch(h_bf16, h_f32, router_w, router_b, top_k, E_local, C, recv_x_off, recv_meta_off, recv_w_off, counts_off,
                       sym, topk_ids=None, topk_w=None, status=None):
    """Router + top-k + softmax + expert-parallel dispatch of ``h_bf16`` [T][d] (see ``moe.cu``); the router
    (fp32 weights) reads ``h_f32`` when given."""
    T, d = h_bf16.shape
    E = router_w.shape[0]
    _check(lib().b200_moe_route_dispatch(_p(h_bf16), _p(h_f32), _p(router_w), _p(router_b), T, d, E, top_k, E_local, C, recv_x_off,
                                         recv_meta_off, recv_w_off, counts_off, _p(topk_ids), _p(topk_w), _sym(sym),
                                         _p(status), _st()), "moe_route_dispatch")


def moe_gemm(A, B, groups, group_rows, N, K, counts, mode, out_bf16=None, ldc=0, meta=None, gate_w=None, sym=None,
             sym_off=0, status=None, lda=None, ldb=None):
    """Grouped expert GEMM (see ``gemm_tc05.cu``): mode 1 = gate/up with fused SwiGLU, mode 2 = down
    projection fused with the weighted combine into the source ranks' residual streams."""
    _check(lib().b200_moe_gemm(_p(A), _p(B), groups, group_rows, N, K, lda or K, ldb or K, _p(counts), mode, _p(out_bf16),
                               ldc, _p(meta), _p(gate_w), _sym(sym), sym_off, _p(status), _st()), "moe_gemm")


def moe_zero(t):
    _check(lib().b200_moe_zero(_p(t), t.numel(), _st()), "moe_zero")


# ---- exact arithmetic over a prime field (training verification): residues are int32 tensors with values in [0, p), p < 2^31
def modp_matvec(A, x, p: int):
    rows, cols = A.shape
    y = torch.empty(rows, dtype=torch.int32, device=A.device)
    _check(lib().b200_modp_matvec(_p(A), _p(x), _p(y), rows, cols, p, _st()), "modp_matvec")
    return y


def modp_matmul(A, B, p: int):
    n, k = A.shape
    m = B.shape[1]
    C = torch.empty((n, m), dtype=torch.int32, device=A.device)
    _check(lib().b200_modp_matmul(_p(A), _p(B), _p(C), n, k, m, p, _st()), "modp_matmul")
    return C


def count_mismatch(a, b) -> torch.Tensor:
    out = torch.zeros(1, dtype=torch.int32, device=a.device)
    _check(lib().b200_count_mismatch(_p(a), _p(b), a.numel(), _p(out), _st()), "count_mismatch")
    return out
