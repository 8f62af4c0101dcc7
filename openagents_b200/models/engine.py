"""Decoder engine for dense llama-family models on one GPU (or one tensor-parallel rank).

The engine owns the device weights, the paged fp16 KV cache and the activation workspaces, and
exposes two operations over packed token batches: ``forward_tokens`` (prefill chunks, many tokens
per sequence) and ``decode`` (one token per sequence, replayed from a CUDA graph).  The weights stay
in their packed GGUF block formats in device memory, once: up to 4 decode tokens take the quantized
mat-vec kernels (``dp4a``), up to 64 tokens the tcgen05 GEMM that expands the blocks inside its
pipeline, and longer chunks (prefill) expand one matrix at a time into a scratch buffer for the
bf16 tcgen05 GEMM.

The serve-side contract this implements is the reference's model-server description: GGUF load,
KV and prefix caches, continuous batching (docs/muse/muse-glimmer.md:110-126).
"""
from __future__ import annotations

import ctypes
import math
import os
from dataclasses import dataclass

import torch

from .. import _native
from ..ops import cuda_ops as ops
from .config import ModelConfig
from .qweight import QWeight, RawTensor, WeightSource
from ..utils.nvtx import nvtx_method

PAGE = 16
MATVEC_MAX_TOKENS = 8
QGEMM_MAX_TOKENS = 64      # token tile of the fused-dequant GEMM; also the row count of the tensor-parallel slots


class KVPool:
    """Host-side page bookkeeping (C++), shared by every layer's device cache."""

    def __init__(self, n_pages: int, page_size: int = PAGE):
        L = _native.host()
        if not getattr(L, "_b200_kv_ready", False):
            vp, i64, i32, u64 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_uint64
            P32 = ctypes.POINTER(ctypes.c_int32)
            sig = {"b200_kv_create": ([i32, i32], vp), "b200_kv_destroy": ([vp], None),
                   "b200_kv_free_pages": ([vp], i32), "b200_kv_total_pages": ([vp], i32), "b200_kv_retained_pages": ([vp], i32), "b200_kv_set_retention": ([vp, i32], None),
                   "b200_kv_prefix_hits": ([vp], u64), "b200_kv_prefix_lookups": ([vp], u64),
                   "b200_kv_seq_begin": ([vp, i64, P32, i64], i64), "b200_kv_seq_extend": ([vp, i64, i64], i32),
                   "b200_kv_seq_publish": ([vp, i64, P32, i64], None), "b200_kv_seq_len": ([vp, i64], i64),
                   "b200_kv_seq_n_pages": ([vp, i64], i32), "b200_kv_seq_pages": ([vp, i64, P32, i32], i32),
                   "b200_kv_seq_truncate": ([vp, i64, i64, P32, P32], i32), "b200_kv_seq_end": ([vp, i64], None),
                   "b200_kv_stage_decode": ([vp, vp, i32, i32, i32, vp, vp, vp, vp, vp], i32)}
            for n, (a, r) in sig.items():
                f = getattr(L, n)
                f.argtypes, f.restype = a, r
            L._b200_kv_ready = True
        self.L = L
        self.h = L.b200_kv_create(n_pages, page_size)
        self.page_size = page_size
        self.n_pages = n_pages
        # B200_KV_RETAIN=0: published pages leave the prefix index with their last holder, so that a repeated prompt takes the
        # very same compute path as the first time (bit-exact repeats); the default keeps them until the memory is needed
        if os.environ.get("B200_KV_RETAIN", "1") == "0":
            self.set_retention(False)

    def set_retention(self, on: bool):
        self.L.b200_kv_set_retention(self.h, int(bool(on)))

    @staticmethod
    def _arr(tokens):
        if tokens is None:
            return None, 0
        a = (ctypes.c_int32 * len(tokens))(*tokens)
        return a, len(tokens)

    def begin(self, seq_id: int, tokens=None) -> int:
        a, n = self._arr(tokens)
        r = self.L.b200_kv_seq_begin(self.h, seq_id, a, n)
        if r < 0:
            raise KeyError(f"sequence {seq_id} already exists")
        return r

    def extend(self, seq_id: int, n_new: int):
        r = self.L.b200_kv_seq_extend(self.h, seq_id, n_new)
        if r == -1:
            raise KeyError(f"unknown sequence {seq_id}")
        if r == -2:
            raise MemoryError("KV cache is out of pages")

    def publish(self, seq_id: int, tokens):
        a, n = self._arr(tokens)
        self.L.b200_kv_seq_publish(self.h, seq_id, a, n)

    def length(self, seq_id: int) -> int:
        return self.L.b200_kv_seq_len(self.h, seq_id)

    def n_pages_of(self, seq_id: int) -> int:
        return self.L.b200_kv_seq_n_pages(self.h, seq_id)

    def pages(self, seq_id: int) -> list[int]:
        n = self.L.b200_kv_seq_n_pages(self.h, seq_id)
        if n < 0:
            raise KeyError(f"unknown sequence {seq_id}")
        buf = (ctypes.c_int32 * max(n, 1))()
        self.L.b200_kv_seq_pages(self.h, seq_id, buf, n)
        return list(buf[:n])

    def stage_decode(self, seq_ids_ptr: int, B: int, max_pages: int, full_table: bool, pos_ptr: int, slot_ptr: int, ctx_ptr: int,
                     table_ptr: int) -> bool:
        """Grow ``B`` sequences by one token and fill the staging arrays (raw host pointers); returns
        whether any page-table row was rewritten."""
        dirty = ctypes.c_int32(0)
        r = self.L.b200_kv_stage_decode(self.h, seq_ids_ptr, B, max_pages, int(full_table), pos_ptr, slot_ptr, ctx_ptr, table_ptr,
                                        ctypes.addressof(dirty))
        if r == -1:
            raise KeyError("unknown sequence in the decode batch")
        if r == -2:
            raise MemoryError("KV cache is out of pages")
        if r == -3:
            raise ValueError("sequence exceeds the engine's max context")
        return bool(dirty.value)

    def truncate(self, seq_id: int, new_len: int):
        """Drop the tokens from ``new_len`` on.  Returns ``None``, or ``(src_page, dst_page)`` when the partly kept page
        was shared with another sequence and this one was given a page of its own: the caller must copy that page's
        K/V before writing to it."""
        src, dst = ctypes.c_int32(-1), ctypes.c_int32(-1)
        r = self.L.b200_kv_seq_truncate(self.h, seq_id, new_len, ctypes.byref(src), ctypes.byref(dst))
        if r == -2:
            raise MemoryError("KV cache is out of pages")
        if r < 0:
            raise ValueError("bad truncate")
        return (src.value, dst.value) if r == 1 else None

    def end(self, seq_id: int):
        self.L.b200_kv_seq_end(self.h, seq_id)

    @property
    def free_pages(self) -> int:
        return self.L.b200_kv_free_pages(self.h)

    @property
    def retained_pages(self) -> int:
        """Published pages no sequence holds any more: still in the prefix index, reclaimed (oldest first) when pages run short.
        They are counted in ``free_pages``."""
        return self.L.b200_kv_retained_pages(self.h)

    @property
    def prefix_stats(self) -> tuple[int, int]:
        return self.L.b200_kv_prefix_hits(self.h), self.L.b200_kv_prefix_lookups(self.h)

    def __del__(self):
        try:
            self.L.b200_kv_destroy(self.h)
        except Exception:
            pass


@dataclass
class _Layer:
    attn_norm: torch.Tensor
    wqkv: QWeight
    bqkv: torch.Tensor | None
    wo: QWeight
    bo: torch.Tensor | None
    sinks: torch.Tensor | None
    ffn_norm: torch.Tensor
    wgu: QWeight | None
    wdown: QWeight | None
    window: int


def _f32(src: WeightSource, name: str, device=None) -> torch.Tensor | None:
    if not src.has(name):
        return None
    x = src.get(name).to_float().contiguous()
    return x if device is None else x.to(device)


class LlamaEngine:
    ARCHS = ("llama",)

    def __init__(self, cfg: ModelConfig, src: WeightSource, device="cuda", max_batch: int = 64,
                 max_ctx: int = 4096, n_pages: int | None = None, tp_rank: int = 0, tp_world: int = 1,
                 max_tokens: int = 4096, comm=None, canaries: bool | None = None):
        if cfg.arch not in self.ARCHS:
            raise ValueError(f"{type(self).__name__} serves {self.ARCHS} models, not {cfg.arch!r}")
        self.cfg, self.device = cfg, torch.device(device)
        self.rank, self.world, self.comm = tp_rank, tp_world, comm
        self.canaries = (os.environ.get("B200_CANARY", "0") == "1") if canaries is None else bool(canaries)
        self._guards: dict[str, tuple[torch.Tensor, int]] = {}
        self._use_fence = os.environ.get("B200_TP_FENCE", "0") == "1"
        # Tensor-parallel decode: "slots" = the row-parallel projections keep their partial result local and the RMSNorm
        # that follows all-reduces it through per-rank slots (one kernel: push, per-row flags, sum, normalise; no barrier,
        # no handshake); "allreduce" = the older form (multimem.red into every replica from the projection's epilogue +
        # barrier), kept as a measurement aid and for weight types the fused-dequant GEMM does not take.
        self.tp_mode = os.environ.get("B200_TP_MODE", "slots")
        if cfg.n_kv_heads % tp_world or cfg.ffn % tp_world:
            raise ValueError("tensor-parallel degree must divide the KV heads and the FFN width")
        self.Hq, self.Hkv, self.hd = cfg.n_heads // tp_world, cfg.n_kv_heads // tp_world, cfg.head_dim
        self.F = cfg.ffn // tp_world
        self.d = cfg.d_model
        self.max_batch, self.max_tokens = max_batch, max_tokens
        self.max_pages = (max_ctx + PAGE - 1) // PAGE
        self.n_pages = n_pages if n_pages is not None else max_batch * self.max_pages + 1
        self.pool = KVPool(self.n_pages)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._load(src)
        self._alloc()
        self._graphs: dict[int, tuple] = {}
        self.launches_per_decode = 0
        # Up to this many decode tokens take the mat-vec path.  Measured on the 8B shape (ms per step, mat-vec / GEMM path):
        # 2 tokens 2.9 / 4.3, 4 tokens 4.0 / 4.3, 8 tokens 5.7 / 4.4: the mat-vec kernels scale with the token count, the
        # tensor-core path does not, and they cross between 4 and 5 tokens.
        self.small_path_tokens = min(MATVEC_MAX_TOKENS, int(os.environ.get("B200_SMALL_PATH_TOKENS", 4)))
        self.h2d_bytes = 0                              # host-to-device bytes copied by decode() so far
        self.prefill_tc05 = os.environ.get("B200_PREFILL_TC05", "1") == "1"     # tcgen05 prefill attention (head size 128)
        self.seq_shard = os.environ.get("B200_TP_SEQ_SHARD", "1") == "1"        # sequence-sharded tensor-parallel prefill
        self.fuse_rope = os.environ.get("B200_FUSE_ROPE", "1") == "1"          # small-batch path: rotary + cache write in the QKV mat-vec
        self.attn_target_ctas = int(os.environ.get("B200_ATTN_CTAS", 0))   # split-K attention: CTAs to aim for (0: built-in rule)

    # ------------------------------------------------------------------ weights
    def _shard_rows(self, r: RawTensor, per_head_rows: int | None = None) -> RawTensor:
        n = r.shape[0] // self.world
        return r.rows(self.rank * n, (self.rank + 1) * n)

    def _shard_cols(self, r: RawTensor) -> RawTensor:
        k = r.shape[1] // self.world
        return r.cols(self.rank * k, (self.rank + 1) * k) if self.world > 1 else r

    def _load(self, src: WeightSource):
        cfg, dev = self.cfg, self.device
        emb = src.get("token_embd.weight")
        self.emb = QWeight.from_raw(emb).to(dev)
        self.emb_type = {ops.WT_Q6KR: ops.EMB_Q6KR, ops.WT_Q8R: ops.EMB_Q8R, ops.WT_BF16: ops.EMB_BF16}.get(self.emb.wt)
        if self.emb_type is None:
            # Q4_K / MXFP4 tables are not gathered directly; keep them as bf16.
            x = emb.to_float().to(torch.bfloat16).contiguous().to(dev)
            self.emb = QWeight(ops.WT_BF16, x.shape[0], x.shape[1], x, None, emb.type)
            self.emb_type = ops.EMB_BF16
        self.layers: list[_Layer] = []
        for i in range(cfg.n_layers):
            p = f"blk.{i}."
            q, k, v = (self._shard_rows(src.get(p + n + ".weight")) for n in ("attn_q", "attn_k", "attn_v"))
            wqkv = QWeight.from_raw(RawTensor.cat_rows([q, k, v])).to(dev)
            bqkv = None
            if src.has(p + "attn_q.bias"):
                bqkv = torch.cat([self._shard_rows(src.get(p + n + ".bias")).to_float() for n in ("attn_q", "attn_k", "attn_v")]).contiguous().to(dev)
            wo = QWeight.from_raw(self._shard_cols(src.get(p + "attn_output.weight"))).to(dev)
            bo = _f32(src, p + "attn_output.bias", dev)
            sinks = _f32(src, p + "attn_sinks.weight", dev)
            if sinks is not None and self.world > 1:
                sinks = sinks[self.rank * self.Hq:(self.rank + 1) * self.Hq].contiguous()
            wgu, wdown = self._load_ffn(src, p, i)
            self.layers.append(_Layer(_f32(src, p + "attn_norm.weight", dev), wqkv, bqkv, wo, bo, sinks,
                                      _f32(src, p + "ffn_norm.weight", dev), wgu, wdown,
                                      cfg.sliding_window if cfg.layer_uses_window(i) else 0))
        self.out_norm = _f32(src, "output_norm.weight", dev)
        out = src.get("token_embd.weight" if cfg.tied_embeddings else "output.weight")
        self.V_local = out.shape[0] // self.world if out.shape[0] % self.world == 0 else out.shape[0]
        self.vocab_sharded = self.world > 1 and out.shape[0] % self.world == 0
        if self.vocab_sharded:
            out = out.rows(self.rank * self.V_local, (self.rank + 1) * self.V_local)
        self.wout = QWeight.from_raw(out).to(dev)
        torch.cuda.synchronize(dev)

    def _load_ffn(self, src: WeightSource, p: str, layer: int):
        """Gate and up projections as ONE matrix with interleaved rows (gate_0, up_0, gate_1, ...): every kernel that
        fuses SwiGLU pairs adjacent rows, so a single packed copy serves the mat-vec, the fused-dequant GEMM and the
        prefill GEMM."""
        g = self._shard_rows(src.get(p + "ffn_gate.weight"))
        u = self._shard_rows(src.get(p + "ffn_up.weight"))
        return (QWeight.from_raw(RawTensor.interleave_rows(g, u)).to(self.device),
                QWeight.from_raw(self._shard_cols(src.get(p + "ffn_down.weight"))).to(self.device))

    def weight_bytes(self) -> int:
        n = self.wout.nbytes()
        for l in self.layers:
            n += l.wqkv.nbytes() + l.wo.nbytes() + (l.wgu.nbytes() + l.wdown.nbytes() if l.wgu is not None else 0)
        return n

    # ------------------------------------------------------------------ workspaces
    _GUARD_BYTES, _GUARD_FILL = 256, 0xA5

    def _ws(self, name: str, shape, dtype, zero: bool = False) -> torch.Tensor:
        """One workspace tensor.  With canaries on (``B200_CANARY=1`` or ``canaries=True``) it sits between two 256-byte
        guard zones of a known byte, and ``check_canaries`` tells which guards a kernel has written into: the
        substitute for a memory checker on the engine's own buffers."""
        n = 1
        for v in shape:
            n *= int(v)
        if not self.canaries:
            return (torch.zeros if zero else torch.empty)(tuple(shape), dtype=dtype, device=self.device)
        G = self._GUARD_BYTES
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        body_bytes = (nbytes + G - 1) // G * G
        raw = torch.full((G + body_bytes + G,), self._GUARD_FILL, dtype=torch.uint8, device=self.device)
        body = raw[G: G + nbytes].view(dtype).view(*shape)
        if zero:
            body.zero_()
        self._guards[name] = (raw, nbytes)
        return body

    def check_canaries(self) -> list[str]:
        """Names of the workspaces whose guard zones no longer hold the fill byte (empty list: all intact, or canaries
        off).  ``name:before`` / ``name:after`` says on which side the stray write landed."""
        bad = []
        G = self._GUARD_BYTES
        torch.cuda.synchronize(self.device) if self.device.type == "cuda" else None
        for name, (raw, nbytes) in self._guards.items():
            if not bool((raw[:G] == self._GUARD_FILL).all()):
                bad.append(name + ":before")
            if not bool((raw[G + nbytes:] == self._GUARD_FILL).all()):
                bad.append(name + ":after")
        return bad

    def _alloc(self):
        dev, T = self.device, self.max_tokens
        f32 = dict(dtype=torch.float32, device=dev)
        d, qd, kvd, F = self.d, self.Hq * self.hd, self.Hkv * self.hd, self.F
        self.qkv_dim = qd + 2 * kvd
        self.kc = [torch.zeros((self.n_pages, self.Hkv, PAGE, self.hd), dtype=torch.float16, device=dev) for _ in self.layers]
        self.vc = [torch.zeros_like(k) for k in self.kc]
        if self.world > 1:   # the replicated residual stream receives peers' partial sums: symmetric heap
            # (+ world rows: the in-place all-gather that ends a sequence-sharded prefill moves whole row blocks)
            self.x, self.x_off = self.comm.alloc_tensor((T + self.world, d), torch.float32)
            self.hbfull, self.hbfull_off = self.comm.alloc_tensor((T + self.world, d), torch.bfloat16)
            self._ag_epoch = 0
        else:
            self.x = self._ws("x", (T, d), torch.float32)
        i8, i32, bf, f16, f32t = torch.int8, torch.int32, torch.bfloat16, torch.float16, torch.float32
        ws = self._ws
        self.qkv = ws("qkv", (T, self.qkv_dim), f32t)
        self.q32 = ws("q32", (max(self.max_batch, 1), qd), f32t)
        self.q16 = ws("q16", (T, qd), f16)
        self.hb = ws("hb", (T, max(d, qd, F)), bf)
        self.hb2 = ws("hb2", (T, F), bf)
        self.gu = ws("gu", (T, 2 * F), f32t)
        self.logits = ws("logits", (self.max_batch, self.V_local), f32t)
        kmax = max(d, qd, F)
        nb = MATVEC_MAX_TOKENS
        self.xq = ws("xq", (nb, kmax), i8)
        self.xd = ws("xd", (nb, kmax // 32 + 1), f32t)
        self.xs = ws("xs", (nb, kmax // 16 + 2), f32t)
        self.xf = ws("xf", (nb, kmax), f32t)
        # second activation set: a kernel never writes the buffers it is still reading
        self.fq = ws("fq", (nb, kmax), i8)
        self.fd = ws("fd", (nb, kmax // 32 + 1), f32t)
        self.fs = ws("fs", (nb, kmax // 16 + 2), f32t)
        self.ids = ws("ids", (T,), i32, zero=True)
        self.pos = ws("pos", (T,), i32, zero=True)
        self.slot = ws("slot", (T,), i32, zero=True)
        self.page_table = ws("page_table", (self.max_batch, self.max_pages), i32, zero=True)
        self.seq_lens = ws("seq_lens", (self.max_batch,), i32, zero=True)
        self.q_start = ws("q_start", (self.max_batch,), i32, zero=True)
        self.q_len = ws("q_len", (self.max_batch,), i32, zero=True)
        self.out_ids = ws("out_ids", (self.max_batch,), i32, zero=True)
        self.out_val = ws("out_val", (self.max_batch,), f32t, zero=True)
        self.max_splits = 64
        self.attn_scratch = ws("attn_scratch", (ops.attn_decode_scratch_floats(self.max_batch, self.Hq, self.Hkv, self.hd, self.max_splits),), f32t)
        self.attn_counters = ws("attn_counters", (self.max_batch * self.Hkv,), i32, zero=True)
        self.argmax_scratch = ops.argmax_scratch(self.max_batch, dev)
        self.rope_tab = ops.rope_table(self.max_pages * PAGE, self.hd, self.cfg.rope_theta, dev)
        wmax = max(max(l.wqkv.N * l.wqkv.K, l.wo.N * l.wo.K, *((l.wgu.N * l.wgu.K, l.wdown.N * l.wdown.K) if l.wgu is not None else ()))
                   for l in self.layers)
        # bf16 expansion space for prefill GEMMs: the largest layer matrix (the LM head too only when the fused-dequant GEMM
        # does not take its type).  Two buffers when the expansion of the next matrix runs beside the current GEMM.
        self._wscratch_elems = max(wmax, self.wout.N * self.wout.K if (self.wout.quantized and not self._qg(self.wout)) else 0)
        self._wbufs: list[torch.Tensor | None] = [None, None]
        self._pf = None                      # (weight, buffer index, ready event) of the expansion in flight on the side stream
        self._pf_stream = None
        self._pf_on = os.environ.get("B200_DEQUANT_OVERLAP", "1") == "1"
        order = [w for l in self.layers for w in (l.wqkv, l.wo, l.wgu, l.wdown) if w is not None and w.wt != ops.WT_BF16]
        self._pf_next = {id(a): b for a, b in zip(order, order[1:])}
        if self.world > 1:
            # one-shot all-reduce: slots [parity][rank][row][d] on every rank, and this rank's partial rows (local, kept
            # zeroed between uses: the projections accumulate into them)
            self.slot_rows = QGEMM_MAX_TOKENS
            self.slots, self.slots_off = self.comm.alloc_tensor((2, self.world, self.slot_rows, d), torch.float32)
            self.xpart = self._ws("xpart", (self.slot_rows, d), torch.float32, zero=True)
            row_par = [w for l in self.layers for w in (l.wo, l.wdown) if w is not None]
            self.slots_small = self.tp_mode == "slots"
            self.slots_dense = self.slots_small and all(self._qg(w) for w in row_par)
        else:
            self.slots_small = self.slots_dense = False
        self._slots_pending = False

    @staticmethod
    def _qg(w: QWeight) -> bool:
        """Whether the fused-dequant GEMM takes this weight."""
        return w is not None and w.wt in (ops.WT_Q4KR, ops.WT_Q6KR) and w.K % 256 == 0

    def scratch_bytes(self) -> int:
        return sum(b.numel() * 2 for b in self._wbufs if b is not None)

    def _wbuf(self, i: int, w: QWeight) -> torch.Tensor:
        if self._wbufs[i] is None:
            self._wbufs[i] = torch.empty(self._wscratch_elems, dtype=torch.bfloat16, device=self.device)
        return self._wbufs[i][: w.N * w.K].view(w.N, w.K)

    def _dense(self, w: QWeight) -> torch.Tensor:
        """bf16 [N][K] form of a weight for the bf16 tensor-core GEMM (prefill): the matrix itself when it is stored in
        bf16, else its expansion into a scratch buffer.  The expansion is memory-bound and the GEMM compute-bound, so while
        the GEMM on this matrix runs, the NEXT matrix of the layer walk is expanded into the other buffer on a side stream
        (events order the two; ``B200_DEQUANT_OVERLAP=0`` or a stream capture in progress falls back to one buffer in
        stream order)."""
        if w.wt == ops.WT_BF16:
            return w.main
        main = torch.cuda.current_stream(self.device)
        pf, self._pf = self._pf, None
        if pf is not None:
            main.wait_event(pf[2])                       # whatever the side stream was writing is complete before we go on
        overlap = self._pf_on and self.device.type == "cuda" and not torch.cuda.is_current_stream_capturing()
        if pf is not None and pf[0] is w:
            b, out = pf[1], self._wbuf(pf[1], w)
        else:
            b = 0
            out = w.dequant_into(self._wbuf(0, w))
        nxt = self._pf_next.get(id(w)) if overlap else None
        if nxt is not None:
            if self._pf_stream is None:
                self._pf_stream = torch.cuda.Stream(self.device)
            free = torch.cuda.Event()
            free.record(main)                            # the GEMM that last read the other buffer is before this point
            self._pf_stream.wait_event(free)
            with torch.cuda.stream(self._pf_stream):
                nxt.dequant_into(self._wbuf(1 - b, nxt))
                ready = torch.cuda.Event()
                ready.record(self._pf_stream)
            self._pf = (nxt, 1 - b, ready)
        return out

    @property
    def _slot_arg(self):
        return (self.comm.heap.table, self.slots_off, self.slot_rows, self.xpart)

    # ------------------------------------------------------------------ building blocks
    def _splits(self, B: int, ctx_pages: int) -> int:
        """Split-K factor of decode attention.  Measured on the 8B shape: a CTA should keep at least ~24
        pages (the merge of the partial results and each CTA's set-up are a fixed cost), small batches
        want just enough CTAs to cover the SMs once, and large batches run best at ~2000 CTAs (several
        waves even out the tail)."""
        if self.attn_target_ctas:                      # explicit override (benchmark sweeps)
            want = max(1, (self.attn_target_ctas + B * self.Hkv - 1) // (B * self.Hkv))
        else:
            rows = B * self.Hkv
            fill = (148 + rows - 1) // rows
            big = (2048 + rows - 1) // rows if rows >= 148 else 0
            want = min(max(1, ctx_pages // 24), max(fill, big))
        return max(1, min(self.max_splits, want, ctx_pages))

    @property
    def _sig(self):
        """Tensor-parallel only: peers add into this rank's residual stream from inside their row-parallel
        kernels, so every rank must have finished reading (or overwriting) it before anyone adds.  The
        RMSNorm that reads it signals when it is done and the row-parallel kernels check the signals just
        before their first remote add: a handshake inside kernels that run anyway, not a barrier launch."""
        if self.world > 1 and self._use_fence:      # measurement aid: the stand-alone barrier the handshake replaces
            self.comm.heap.barrier(ch=2)
            return None
        return self.comm.heap.table if self.world > 1 else None

    def _layers_small(self, nb: int, max_ctx_pages: int):
        """<= 8 tokens, one per sequence: quantized mat-vec path."""
        cfg, x = self.cfg, self.x[:nb]
        S = self._splits(nb, max_ctx_pages)
        qd = self.Hq * self.hd
        style = 0 if cfg.rope_style == "pairs" else 1
        n = 0
        slots = self.slots_small
        table = self.comm.heap.table if self.world > 1 else None
        for li, L in enumerate(self.layers):
            q8 = L.wqkv.quantized
            ops.rmsnorm(x, L.attn_norm, cfg.norm_eps, xq=self.xq if q8 else None, xd=self.xd, xs16=self.xs,
                        hf=None if q8 else self.xf, signal_sym=None if slots else self._sig,
                        slots=self._slot_arg if slots and li > 0 else None)
            if style == 0 and self.fuse_rope:      # rotary pairs are adjacent rows: rotate and write the cache in the epilogue
                ops.matvec_rope_kv(L.wqkv, nb, self.pos, self.slot, self.q32, self.kc[li], self.vc[li], self.Hq, self.Hkv, self.hd,
                                   PAGE, cfg.rope_theta, 1.0 / math.sqrt(self.hd), xq=self.xq, xd=self.xd, xs16=self.xs, xf=self.xf,
                                   bias=L.bqkv, table=self.rope_tab)
                n -= 1
            else:
                ops.matvec(L.wqkv.wt, L.wqkv.main, L.wqkv.plane2, L.wqkv.N, L.wqkv.K, nb, xq=self.xq, xd=self.xd,
                           xs16=self.xs, xf=self.xf, epi=ops.EPI_STORE, bias=L.bqkv, y=self.qkv, ldy=self.qkv_dim)
                ops.rope_kv(self.qkv[:nb], self.pos, self.slot, self.q32, None, self.kc[li], self.vc[li], self.Hq, self.Hkv,
                            self.hd, PAGE, cfg.rope_theta, style, 1.0 / math.sqrt(self.hd), table=self.rope_tab)
            oq8 = L.wo.quantized
            ops.attn_decode(self.q32, self.kc[li], self.vc[li], self.page_table, self.seq_lens, nb, self.Hq, self.Hkv,
                            self.hd, window=L.window, S=S, sinks=L.sinks, out_f32=None if oq8 else self.xf,
                            oq=self.xq if oq8 else None, od=self.xd, os16=self.xs, scratch=self.attn_scratch,
                            counters=self.attn_counters, status=self.status)
            if self.world == 1:
                ops.matvec(L.wo.wt, L.wo.main, L.wo.plane2, L.wo.N, L.wo.K, nb, xq=self.xq, xd=self.xd, xs16=self.xs,
                           xf=self.xf, epi=ops.EPI_RESID, bias=L.bo, resid=x, y=x, ldy=self.d)
            elif slots:      # partial result stays local; the norm below all-reduces it
                ops.matvec(L.wo.wt, L.wo.main, L.wo.plane2, L.wo.N, L.wo.K, nb, xq=self.xq, xd=self.xd, xs16=self.xs,
                           xf=self.xf, epi=ops.EPI_STORE, bias=L.bo if self.rank == 0 else None, y=self.xpart, ldy=self.d)
            else:
                self.comm.matvec_allreduce(L.wo, nb, self.xq, self.xd, self.xs, self.xf, x, self.d, bias=L.bo, wait_ready=not self._use_fence)
            g8 = L.wgu.quantized
            ops.rmsnorm(x, L.ffn_norm, cfg.norm_eps, xq=self.xq if g8 else None, xd=self.xd, xs16=self.xs,
                        hf=None if g8 else self.xf, signal_sym=None if slots else self._sig,
                        slots=self._slot_arg if slots else None)
            d8 = L.wdown.quantized and self.F % 32 == 0
            ops.matvec(L.wgu.wt, L.wgu.main, L.wgu.plane2, self.F, L.wgu.K, nb, xq=self.xq, xd=self.xd, xs16=self.xs,
                       xf=self.xf, epi=ops.EPI_SWIGLU_Q8 if d8 else ops.EPI_SWIGLU_F32, y=self.gu, ldy=self.F,
                       oq=self.fq, od=self.fd, os16=self.fs)
            if not d8 and L.wdown.quantized:
                ops.quantize_x(self.gu.view(-1)[: nb * self.F].view(nb, self.F), self.fq, self.fd, self.fs)
                n += 1
            if self.world == 1:
                ops.matvec(L.wdown.wt, L.wdown.main, L.wdown.plane2, L.wdown.N, L.wdown.K, nb, xq=self.fq, xd=self.fd,
                           xs16=self.fs, xf=self.gu, epi=ops.EPI_RESID, resid=x, y=x, ldy=self.d)
            elif slots:
                ops.matvec(L.wdown.wt, L.wdown.main, L.wdown.plane2, L.wdown.N, L.wdown.K, nb, xq=self.fq, xd=self.fd,
                           xs16=self.fs, xf=self.gu, epi=ops.EPI_STORE, y=self.xpart, ldy=self.d)
            else:
                self.comm.matvec_allreduce(L.wdown, nb, self.fq, self.fd, self.fs, self.gu, x, self.d, wait_ready=not self._use_fence)
            n += 8
        self._slots_pending = slots          # the last down projection's sum is taken by the final norm
        return n

    def _gemm(self, a_bf16, w: QWeight, M, out_f32=None, out_bf16=None, bias=None, resid_f32=None, ldc=None, accumulate=False):
        ops.gemm_bf16(a_bf16, self._dense(w), M, w.N, w.K, lda=a_bf16.stride(0), ldb=w.K, out_f32=out_f32,
                      out_bf16=out_bf16, ldc=ldc or w.N, bias=bias, resid_f32=resid_f32, accumulate=accumulate, status=self.status)

    def _seq_sharded(self, T: int, decode: bool) -> bool:
        """Tensor-parallel prefill keeps the residual stream sharded by rows (sequence parallel): each
        row-parallel GEMM reduce-scatters its partial sums to the rows' owners and each norm all-gathers the
        normalised rows into the next column-parallel GEMM, instead of all-reducing the whole stream twice
        a layer (an all-reduce delivers world x [T, d] fp32 to every GPU; the pair delivers about 1.5 x)."""
        return self.world > 1 and not decode and self.seq_shard and T >= 128 * self.world

    def _layers_dense(self, T: int, decode: bool, n_seqs: int, max_q: int, max_ctx_pages: int):
        """Any token count: tensor-core path.  Up to 64 tokens (decode batches, short chunks) the projections whose
        weights are Q4_K / Q6_K run on the fused-dequant GEMM, which streams the packed blocks; beyond that (prefill)
        every matrix is expanded into the shared scratch buffer and multiplied by the bf16 GEMM."""
        if self._seq_sharded(T, decode):
            return self._layers_seq_sharded(T, n_seqs, max_q)
        cfg, x = self.cfg, self.x[:T]
        qd = self.Hq * self.hd
        style = 0 if cfg.rope_style == "pairs" else 1
        hb_d = self.hb.view(-1)[: T * self.d].view(T, self.d)
        hb_q = self.hb.view(-1)[: T * qd].view(T, qd)
        hb_f = self.hb2[:T]                           # its own buffer: the fused gate/up GEMM reads hb_d while writing it
        qkv = self.qkv[:T]
        gu = self.gu[:T]
        S = self._splits(n_seqs, max_ctx_pages) if decode else 1
        n = 0
        fused = T <= QGEMM_MAX_TOKENS      # the fused-dequant GEMM's token tile
        slots = self.slots_dense and fused
        table = self.comm.heap.table if self.world > 1 else None
        sig = None if slots else self._sig
        split_qkv = T <= 64          # one row tile: let the QKV GEMM split K (the norm clears its output, the splits add)
        for li, L in enumerate(self.layers):
            ops.rmsnorm(x, L.attn_norm, cfg.norm_eps, hb=hb_d, signal_sym=sig, zero=qkv if split_qkv else None,
                        slots=self._slot_arg if slots and li > 0 else None)
            if fused and self._qg(L.wqkv):
                ops.qgemm(L.wqkv, hb_d, T, out_f32=qkv, bias=L.bqkv, epi=ops.QEPI_ADD, status=self.status)
            else:
                self._gemm(hb_d, L.wqkv, T, out_f32=qkv, bias=L.bqkv, accumulate=split_qkv)
            if decode:
                ops.rope_kv(qkv, self.pos, self.slot, self.q32, None, self.kc[li], self.vc[li], self.Hq, self.Hkv, self.hd,
                            PAGE, cfg.rope_theta, style, 1.0 / math.sqrt(self.hd), table=self.rope_tab)
                ops.attn_decode(self.q32, self.kc[li], self.vc[li], self.page_table, self.seq_lens, n_seqs, self.Hq,
                                self.Hkv, self.hd, window=L.window, S=S, sinks=L.sinks, out_bf16=hb_q,
                                scratch=self.attn_scratch, counters=self.attn_counters, status=self.status)
            else:
                ops.rope_kv(qkv, self.pos, self.slot, None, self.q16, self.kc[li], self.vc[li], self.Hq, self.Hkv, self.hd,
                            PAGE, cfg.rope_theta, style, 1.0 / math.sqrt(self.hd), table=self.rope_tab)
                if self.hd == 128 and self.prefill_tc05:     # 5th-generation tensor-core path
                    ops.attn_prefill_tc05(self.q16, self.kc[li], self.vc[li], self.page_table, self.q_start, self.q_len,
                                          self.seq_lens, n_seqs, max_q, self.Hq, self.Hkv, window=L.window, sinks=L.sinks,
                                          out_bf16=hb_q, status=self.status)
                else:
                    ops.attn_prefill(self.q16, self.kc[li], self.vc[li], self.page_table, self.max_pages, self.q_start,
                                     self.q_len, self.seq_lens, n_seqs, max_q, self.Hq, self.Hkv, self.hd, window=L.window,
                                     sinks=L.sinks, out_bf16=hb_q)
            self._row_parallel(hb_q, L.wo, T, x, L.bo, fused, slots, table)
            ops.rmsnorm(x, L.ffn_norm, cfg.norm_eps, hb=hb_d, hf=self._ffn_hf(T), signal_sym=sig,
                        slots=self._slot_arg if slots else None)
            n += 6 + self._ffn_dense(li, L, T, x, hb_d, hb_f, gu, fused, slots, table)
        if slots and not decode:
            # a short prefill chunk: the caller picks rows out of x, so fold the last all-reduce into it now
            ops.rmsnorm(x, None, cfg.norm_eps, slots=self._slot_arg)
            n += 1
        else:
            self._slots_pending = slots      # decode: the final norm takes the last sum
        return n

    @nvtx_method("tp.row_parallel(all_reduce)")
    def _row_parallel(self, a_bf16, w: QWeight, T: int, x, bias, fused: bool, slots: bool, table):
        """x += a W^T for a row-parallel projection (attention output, FFN down), summed over the tensor-parallel ranks."""
        if slots:        # this rank's partial sums stay local (K splits add into the zeroed rows); the next norm all-reduces them
            ops.qgemm(w, a_bf16, T, out_f32=self.xpart, ldo=self.d, bias=bias if self.rank == 0 else None, epi=ops.QEPI_ADD,
                      status=self.status)
        elif self.world == 1:
            if fused and self._qg(w):
                ops.qgemm(w, a_bf16, T, out_f32=x, ldo=self.d, bias=bias, epi=ops.QEPI_ADD, status=self.status)
            else:
                self._gemm(a_bf16, w, T, out_f32=x, bias=bias, resid_f32=x, ldc=self.d)
        else:
            self.comm.gemm_allreduce(a_bf16, self._dense(w), T, x, bias=bias, status=self.status, wait_ready=not self._use_fence)

    @nvtx_method("tp.prefill_layers(reduce_scatter+all_gather)")
    def _layers_seq_sharded(self, T: int, n_seqs: int, max_q: int):
        """Prefill with the residual stream sharded by rows over the tensor-parallel ranks.  Per layer:
        norm + all-gather push -> QKV GEMM (waits tile by tile for the rows' owners) -> attention on this
        rank's heads -> output GEMM with the reduce-scatter in its epilogue; the same pair around the
        feed-forward block.  Ends with an in-place all-gather of the residual rows, so that the caller
        finds the replicated stream the decode path works on."""
        cfg, W, table = self.cfg, self.world, self.comm.heap.table
        Tr = (T + W - 1) // W
        row0 = min(T, self.rank * Tr)
        nloc = min(T, row0 + Tr) - row0
        qd = self.Hq * self.hd
        style = 0 if cfg.rope_style == "pairs" else 1
        hbf = self.hbfull[:T]
        hb_q = self.hb.view(-1)[: T * qd].view(T, qd)
        hb_f = self.hb2[:T]
        qkv = self.qkv[:T]
        n = 0

        def norm_gather(gain):
            ops.rmsnorm_allgather(self.x, gain, cfg.norm_eps, row0, nloc, self.hbfull_off, table)
            self._ag_epoch += 1

        def gemm_scatter(a, w, bias=None):
            N, K = w.shape
            ops.gemm_bf16(a, w, T, N, K, lda=a.stride(0), ldb=K, ldc=self.d, bias=bias, status=self.status,
                          sym_mode=ops.SYM_RSCATTER_ROWS, sym=table, sym_off=self.x_off, rows_per_rank=Tr)

        for li, L in enumerate(self.layers):
            norm_gather(L.attn_norm)
            wq = self._dense(L.wqkv)
            ops.gemm_bf16(hbf, wq, T, L.wqkv.N, L.wqkv.K, lda=self.d, ldb=L.wqkv.K, out_f32=qkv, ldc=L.wqkv.N, bias=L.bqkv,
                          status=self.status, sym=table, ag_rows_per_rank=Tr, ag_epoch=self._ag_epoch)
            ops.rope_kv(qkv, self.pos, self.slot, None, self.q16, self.kc[li], self.vc[li], self.Hq, self.Hkv, self.hd,
                        PAGE, cfg.rope_theta, style, 1.0 / math.sqrt(self.hd), table=self.rope_tab)
            if self.hd == 128 and self.prefill_tc05:
                ops.attn_prefill_tc05(self.q16, self.kc[li], self.vc[li], self.page_table, self.q_start, self.q_len,
                                      self.seq_lens, n_seqs, max_q, self.Hq, self.Hkv, window=L.window, sinks=L.sinks,
                                      out_bf16=hb_q, status=self.status)
            else:
                ops.attn_prefill(self.q16, self.kc[li], self.vc[li], self.page_table, self.max_pages, self.q_start,
                                 self.q_len, self.seq_lens, n_seqs, max_q, self.Hq, self.Hkv, self.hd, window=L.window,
                                 sinks=L.sinks, out_bf16=hb_q)
            gemm_scatter(hb_q, self._dense(L.wo), bias=L.bo)
            norm_gather(L.ffn_norm)
            ops.gemm_bf16(hbf, self._dense(L.wgu), T, 2 * self.F, L.wgu.K, lda=self.d, ldb=L.wgu.K, out_bf16=hb_f,
                          ldc=self.F, act=ops.ACT_SWIGLU_PAIR, status=self.status, sym=table, ag_rows_per_rank=Tr,
                          ag_epoch=self._ag_epoch)
            n += 8
            gemm_scatter(hb_f, self._dense(L.wdown))
        # every rank's rows back into every replica (whole blocks of Tr rows; the tensor has world spare rows)
        self.comm.heap.all_gather(self.x_off + self.rank * Tr * self.d * 4, self.x_off, Tr * self.d * 4)
        return n + 1

    def _ffn_hf(self, T: int):
        """fp32 copy of the normalised hidden state, for feed-forward blocks that want one."""
        return None

    def _ffn_dense(self, li: int, L: _Layer, T: int, x, hb_d, hb_f, gu, fused: bool = False, slots: bool = False, table=None) -> int:
        """Feed-forward block on ``hb_d`` (normalised hidden, bf16); adds its output into ``x``.  The gate/up matrix has
        interleaved rows, so SwiGLU runs in the epilogue of its GEMM: no fp32 [T][2F] round trip."""
        n = 2
        if fused and self._qg(L.wgu) and (2 * self.F + 127) // 128 >= 74:
            ops.qgemm(L.wgu, hb_d, T, out_bf16=hb_f, ldo=self.F, epi=ops.QEPI_SWIGLU, status=self.status)
        elif fused and self._qg(L.wgu):
            # Few row tiles (a tensor-parallel shard): a tile per CTA would leave most SMs idle for the whole K loop, so K is
            # split, the partial sums add up in fp32 and a small kernel applies SwiGLU (and clears the buffer behind it).
            if not getattr(self, "_gu_zeroed", False):
                self.gu.zero_()
                self._gu_zeroed = True
            ops.qgemm(L.wgu, hb_d, T, out_f32=gu, ldo=2 * self.F, epi=ops.QEPI_ADD, status=self.status)
            ops.swiglu(gu, self.F, ob=hb_f, zero_after=True)
            n = 3
        else:
            ops.gemm_bf16(hb_d, self._dense(L.wgu), T, 2 * self.F, L.wgu.K, lda=hb_d.stride(0), ldb=L.wgu.K, out_bf16=hb_f,
                          ldc=self.F, act=ops.ACT_SWIGLU_PAIR, status=self.status)
        self._row_parallel(hb_f, L.wdown, T, x, None, fused, slots, table)
        return n

    def _head(self, rows: torch.Tensor, nb: int, greedy: bool = True):
        """Final norm + LM head on ``nb`` rows of fp32 hidden state -> logits (and arg-max ids)."""
        cfg = self.cfg
        n = 2
        slots = self._slot_arg if self._slots_pending else None     # tensor parallel: the last layer's sum is still in the slots
        self._slots_pending = False
        if nb <= MATVEC_MAX_TOKENS:
            q8 = self.wout.quantized
            ops.rmsnorm(rows, self.out_norm, cfg.norm_eps, xq=self.xq if q8 else None, xd=self.xd, xs16=self.xs,
                        hf=None if q8 else self.xf, slots=slots)
            ops.matvec(self.wout.wt, self.wout.main, self.wout.plane2, self.wout.N, self.wout.K, nb, xq=self.xq,
                       xd=self.xd, xs16=self.xs, xf=self.xf, epi=ops.EPI_STORE, y=self.logits, ldy=self.V_local)
        else:
            hb = self.hb.view(-1)[: nb * self.d].view(nb, self.d)
            ops.rmsnorm(rows, self.out_norm, cfg.norm_eps, hb=hb, slots=slots)
            if self._qg(self.wout):          # any row count: the kernel is launched once per 64 rows
                ops.qgemm(self.wout, hb, nb, out_f32=self.logits, ldo=self.V_local, epi=ops.QEPI_STORE, status=self.status)
            else:
                self._gemm(hb, self.wout, nb, out_f32=self.logits)
        if greedy:
            ops.argmax(self.logits[:nb], self.out_ids, self.out_val,
                       vocab_offset=self.rank * self.V_local if self.vocab_sharded else 0, scratch=self.argmax_scratch)
            n += 1
            if self.vocab_sharded:
                self.comm.argmax_merge(self.out_ids, self.out_val, nb)
        return n

    def _embed(self, T: int):
        ops.embedding(self.ids, self.x[:T], self.emb_type, self.emb.main, self.emb.plane2)

    # ------------------------------------------------------------------ host-side batch assembly
    def _stage_batch(self, seq_ids, new_tokens: list[list[int]]):
        """Extend the sequences' page lists and build ids/pos/slot/page-table for the new tokens."""
        ids, pos, slot, q_start, q_len, ctx = [], [], [], [], [], []
        table = torch.zeros((len(seq_ids), self.max_pages), dtype=torch.int32)
        # Check the whole batch before any sequence grows: a refused batch must leave the page lists as they were.
        if len(seq_ids) > self.max_batch or sum(len(t) for t in new_tokens) > self.max_tokens:
            raise ValueError("batch exceeds the engine's workspace")
        need = 0
        for sid, toks in zip(seq_ids, new_tokens):
            p0 = self.pool.length(sid)
            if p0 < 0:
                raise KeyError(f"unknown sequence {sid}")
            after = (p0 + len(toks) + PAGE - 1) // PAGE
            if after > self.max_pages:
                raise ValueError("sequence exceeds the engine's max context")
            need += max(0, after - self.pool.n_pages_of(sid))
        if need > self.pool.free_pages:
            raise MemoryError("KV cache is out of pages")
        for b, (sid, toks) in enumerate(zip(seq_ids, new_tokens)):
            p0 = self.pool.length(sid)
            self.pool.extend(sid, len(toks))
            pages = self.pool.pages(sid)
            table[b, : len(pages)] = torch.tensor(pages, dtype=torch.int32)
            q_start.append(len(ids))
            q_len.append(len(toks))
            ctx.append(p0 + len(toks))
            for i, t in enumerate(toks):
                p = p0 + i
                ids.append(t)
                pos.append(p)
                slot.append(pages[p // PAGE] * PAGE + p % PAGE)
        return ids, pos, slot, q_start, q_len, ctx, table

    def _upload(self, ids, pos, slot, q_start, q_len, ctx, table):
        T, B = len(ids), len(ctx)
        if getattr(self, "_stg", None) is not None:
            self._stg["last_batch"] = None        # the decode fast path must resend its page-table rows
        pin = lambda v: torch.tensor(v, dtype=torch.int32).pin_memory()
        self.ids[:T].copy_(pin(ids), non_blocking=True)
        self.pos[:T].copy_(pin(pos), non_blocking=True)
        self.slot[:T].copy_(pin(slot), non_blocking=True)
        self.q_start[:B].copy_(pin(q_start), non_blocking=True)
        self.q_len[:B].copy_(pin(q_len), non_blocking=True)
        self.seq_lens[:B].copy_(pin(ctx), non_blocking=True)
        self.page_table[:B].copy_(table.pin_memory(), non_blocking=True)

    # ------------------------------------------------------------------ public operations
    def begin(self, seq_id: int, prompt=None) -> int:
        """Open a sequence; returns how many prompt tokens are already cached (prefix reuse)."""
        return self.pool.begin(seq_id, list(prompt) if prompt is not None else None)

    def end(self, seq_id: int):
        self.pool.end(seq_id)

    def truncate(self, seq_id: int, new_len: int):
        """Drop the sequence's tokens from position ``new_len`` on (a cancelled turn, a rejected speculative tail).
        If the page that stays partly filled was shared through the prefix cache, the sequence gets a private copy of
        it, so writing the next tokens cannot touch another sequence's K/V."""
        cow = self.pool.truncate(seq_id, new_len)
        if cow is not None:
            src, dst = cow
            for k, v in zip(self.kc, self.vc):
                k[dst].copy_(k[src])
                v[dst].copy_(v[src])
        if getattr(self, "_stg", None) is not None:
            self._stg["last_batch"] = None        # page lists changed: the decode fast path must resend its rows

    @torch.no_grad()
    @nvtx_method("engine.prefill")
    def forward_tokens(self, seq_ids: list[int], new_tokens: list[list[int]], greedy: bool = True, all_positions: bool = False):
        """Append ``new_tokens[b]`` to sequence ``seq_ids[b]`` and return the logits of each
        sequence's last new token ([B, V] view, valid until the next call) and their arg-max.  ``all_positions``: the
        logits and arg-max of EVERY new token instead ([T, V], in feeding order): what verifying a speculated
        continuation needs; T is then limited by the logits workspace (``max_batch`` rows)."""
        B = len(seq_ids)
        staged = self._stage_batch(seq_ids, new_tokens)
        ids, pos, slot, q_start, q_len, ctx, table = staged
        T = len(ids)
        if T > self.max_tokens or B > self.max_batch or (all_positions and T > self.max_batch):
            raise ValueError("batch exceeds the engine's workspace")
        self._upload(*staged)
        self._embed(T)
        decode = all(n == 1 for n in q_len)
        pages = max((c + PAGE - 1) // PAGE for c in ctx)
        if decode and T <= self.small_path_tokens:
            self._layers_small(T, pages)
        else:
            self._layers_dense(T, decode, B, max(q_len), pages)
        if all_positions:
            self._head(self.x[:T], T, greedy)
            return self.logits[:T], self.out_ids[:T]
        if decode:
            rows = self.x[:B]
        else:
            last = torch.tensor([s + n - 1 for s, n in zip(q_start, q_len)], device=self.device)
            rows = self.x[:T].index_select(0, last).contiguous()
        self._head(rows, B, greedy)
        return self.logits[:B], self.out_ids[:B]

    # ---- graph-replayed decode
    def _capture(self, B: int, pages: int, advance: bool = False):
        g = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream())

        def body():
            self._embed(B)
            n = 1
            if B <= self.small_path_tokens:
                n += self._layers_small(B, pages)
            else:
                n += self._layers_dense(B, True, B, 1, pages)
            n += self._head(self.x[:B], B, True)
            if advance:
                ops.decode_advance(self.ids, self.out_ids, self.pos, self.slot, self.seq_lens, self.page_table, PAGE, B,
                                   self._hist, self._step, self._hist.numel() // B)
                n += 1
            return n

        if advance:   # the warm-up run must not move the real state: save and restore it
            saved = [t.clone() for t in (self.ids, self.pos, self.slot, self.seq_lens, self._step)]
        with torch.cuda.stream(s):
            body()  # warm-up outside capture: sets kernel attributes, allocates the scratch
        if advance:
            torch.cuda.synchronize()
            for t, v in zip((self.ids, self.pos, self.slot, self.seq_lens, self._step), saved):
                t.copy_(v)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=s):
            n = body()
        return g, n

    def _decode_staging(self):
        """Pinned host staging for decode steps, allocated once: per-step metadata goes from the page
        allocator (one native call for the whole batch) into these arrays and from there to the device
        in four small asynchronous copies; the page table moves only when a sequence took a new page
        or the batch changed."""
        if getattr(self, "_stg", None) is None:
            B, P = self.max_batch, self.max_pages
            pin = lambda *shape, dt=torch.int32: torch.zeros(shape, dtype=dt).pin_memory() if torch.cuda.is_available() else torch.zeros(shape, dtype=dt)
            self._stg = {"seq": pin(B, dt=torch.int64), "ids": pin(B), "pos": pin(B), "slot": pin(B), "ctx": pin(B), "table": pin(B, P),
                         "out": pin(B), "last_batch": None}
        return self._stg

    @torch.no_grad()
    @nvtx_method("engine.decode_step")
    def decode(self, seq_ids: list[int], tokens: list[int], use_graph: bool = True):
        """One decode step: append one token per sequence, return (logits view, arg-max ids)."""
        if not use_graph:
            return self.forward_tokens(seq_ids, [[t] for t in tokens])
        B = len(seq_ids)
        if B > self.max_batch:
            raise ValueError("batch exceeds the engine's workspace")
        st = self._decode_staging()
        batch = tuple(seq_ids)
        same = st["last_batch"] == batch
        if not same:
            st["seq"][:B] = torch.tensor(seq_ids, dtype=torch.int64)
        st["ids"][:B] = torch.tensor(tokens, dtype=torch.int32)
        dirty = self.pool.stage_decode(st["seq"].data_ptr(), B, self.max_pages, not same, st["pos"].data_ptr(), st["slot"].data_ptr(),
                                       st["ctx"].data_ptr(), st["table"].data_ptr())
        st["last_batch"] = batch
        pages = (int(st["ctx"][:B].max()) + PAGE - 1) // PAGE
        # Split count is baked into the captured launch; bucket the context length so a graph is
        # reused while the sequence grows.
        bucket = 1 << max(0, (pages - 1)).bit_length()
        key = (B, bucket)

        def upload():
            self.ids[:B].copy_(st["ids"][:B], non_blocking=True)
            self.pos[:B].copy_(st["pos"][:B], non_blocking=True)
            self.slot[:B].copy_(st["slot"][:B], non_blocking=True)
            self.seq_lens[:B].copy_(st["ctx"][:B], non_blocking=True)
            self.h2d_bytes += 16 * B
            if dirty or not same:     # otherwise the device rows are still those of the previous step
                self.page_table[:B].copy_(st["table"][:B], non_blocking=True)
                self.h2d_bytes += 4 * B * self.max_pages

        if key not in self._graphs:
            upload()
            self._graphs[key] = self._capture(B, bucket)
        upload()
        g, n = self._graphs[key]
        g.replay()
        self.launches_per_decode = n
        return self.logits[:B], self.out_ids[:B]

    @torch.no_grad()
    @nvtx_method("engine.decode_steps")
    def decode_steps(self, seq_ids: list[int], tokens: list[int], n_steps: int, on_replay=None):
        """``n_steps`` greedy decode steps with the autoregression kept on the device: one upload,
        ``n_steps`` graph replays (each ends by turning its arg-max into the next step's input),
        one read-back.  Returns the generated ids as an int32 tensor [n_steps, B] (on the device).
        ``on_replay(i)`` is called before replay ``i`` (benchmarks place their events there)."""
        B = len(seq_ids)
        staged = self._stage_batch(seq_ids, [[t] for t in tokens])
        ctx = staged[5]
        table = staged[6]
        for b, sid in enumerate(seq_ids):        # pages for every later step up front
            if (self.pool.length(sid) + n_steps - 1 + PAGE - 1) // PAGE > self.max_pages:
                raise ValueError("sequence exceeds the engine's max context")
            self.pool.extend(sid, n_steps - 1)
            pages = self.pool.pages(sid)
            if len(pages) > self.max_pages:
                raise ValueError("sequence exceeds the engine's max context")
            table[b, : len(pages)] = torch.tensor(pages, dtype=torch.int32)
        pages = max((c + n_steps + PAGE - 1) // PAGE for c in ctx)
        bucket = 1 << max(0, (pages - 1)).bit_length()
        key = ("loop", B, bucket)
        if getattr(self, "_hist", None) is None or self._hist.numel() < n_steps * B:
            self._hist = torch.zeros(max(n_steps * B, 4096), dtype=torch.int32, device=self.device)
            self._step = torch.zeros(1, dtype=torch.int32, device=self.device)
            self._graphs = {k: v for k, v in self._graphs.items() if not (isinstance(k, tuple) and k[0] == "loop")}
        if key not in self._graphs:
            self._upload(*staged)
            self._graphs[key] = self._capture(B, bucket, advance=True)
        self._upload(*staged)
        self._step.zero_()
        g, n = self._graphs[key]
        for i in range(n_steps):
            if on_replay is not None:
                on_replay(i)
            g.replay()
        self.launches_per_decode = n
        return self._hist[: n_steps * B].view(n_steps, B)

    def check_status(self):
        s = int(self.status.item())
        if s:
            raise RuntimeError(f"a kernel wait timed out (status {s})")

    @torch.no_grad()
    def generate(self, prompt: list[int], n_new: int, seq_id: int = 0, use_graph: bool = True):
        """Greedy generation for one sequence.  Returns (ids, per-step logits [n_new, V] on CPU)."""
        cached = self.begin(seq_id, prompt)
        logits, nxt = self.forward_tokens([seq_id], [list(prompt[cached:])])
        out, all_logits = [], []
        for _ in range(n_new):
            all_logits.append(logits[0].float().cpu().clone())
            tok = int(nxt[0].item())
            out.append(tok)
            logits, nxt = self.decode([seq_id], [tok], use_graph=use_graph)
        self.pool.publish(seq_id, list(prompt) + out)
        return out, torch.stack(all_logits)
