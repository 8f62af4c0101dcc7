"""GPT-2-shape causal LM for training: explicit forward and backward over the hand-written kernels.

Parameters live in one flat bf16 buffer (the working copy the GEMMs read) with one flat fp32
gradient buffer beside it; both sit in the symmetric heap so the sharded optimizer's collectives
can address them by offset.  Weight-decayed tensors (matrices, embeddings) come first in the flat
order, so "decay or not" is a single index comparison inside the optimizer kernel.

Linear layers run on the tcgen05 GEMM in its K-major x K-major form:
    forward   y  = x  W^T         A = x [M,K],     B = W  [N,K]
    backward  dx = dy W           A = dy [M,N],    B = W^T [K,N]   (transposed copy, refreshed per step)
              dW += dy^T x        both operands MN-major: dy [M,N] and x [M,K] are read as they lie in memory
                                  (the reduction runs over their rows); accumulated in fp32 in the epilogue
The attention core is this package's flash-attention kernel pair (``csrc/kernels/attn_train.cu``): the forward reads
the fused QKV projection in place and saves one log-sum-exp per row, the backward writes dQ, dK and dV straight into
the gradient of that projection.  No autograd graph is built anywhere in this file.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..models.config import ModelConfig
from ..models.weights import TensorSpec, tensor_specs
from ..ops import cuda_ops as ops
from ..ops import train_ops as tops

VOCAB_PAD = 128


def padded_vocab(v: int) -> int:
    return (v + VOCAB_PAD - 1) // VOCAB_PAD * VOCAB_PAD


@dataclass
class ParamSlot:
    name: str
    shape: tuple[int, ...]
    offset: int          # element offset into the flat buffers
    decay: bool

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


def param_layout(cfg: ModelConfig, align: int = 64) -> tuple[list[ParamSlot], int, int]:
    """Flat layout: decayed tensors first.  Returns (slots, total elements, decay_end)."""
    specs = tensor_specs(cfg)
    Vp = padded_vocab(cfg.vocab)

    def shape_of(s: TensorSpec):
        return (Vp, cfg.d_model) if s.name == "token_embd.weight" else tuple(s.shape)

    decayed = [s for s in specs if s.kind in ("matrix", "embed", "pos")]
    plain = [s for s in specs if s.kind not in ("matrix", "embed", "pos")]
    slots, off = [], 0
    for group, dec in ((decayed, True), (plain, False)):
        for s in group:
            sh = shape_of(s)
            n = 1
            for d in sh:
                n *= d
            slots.append(ParamSlot(s.name, sh, off, dec))
            off += (n + align - 1) // align * align
        if dec:
            decay_end = off
    return slots, off, decay_end


class GPT2Model:
    """Holds views into the flat buffers and runs forward/backward for one micro-batch."""

    def __init__(self, cfg: ModelConfig, params_bf16: torch.Tensor, grads_f32: torch.Tensor | None, slots: list[ParamSlot],
                 micro_batch: int, seq_len: int):
        """``grads_f32`` None: forward only (inference on the training kernels); no gradient views, no backward scratch."""
        self.cfg, self.B, self.T = cfg, micro_batch, seq_len
        self.M = micro_batch * seq_len
        self.dev = params_bf16.device
        self.Vp = padded_vocab(cfg.vocab)
        self.p, self.g = {}, {}
        for s in slots:
            self.p[s.name] = params_bf16[s.offset: s.offset + s.numel].view(*s.shape)
            if grads_f32 is not None:
                self.g[s.name] = grads_f32[s.offset: s.offset + s.numel].view(*s.shape)
        self.slots = slots
        d, f, M = cfg.d_model, cfg.ffn, self.M
        bf = dict(dtype=torch.bfloat16, device=self.dev)
        f32 = dict(dtype=torch.float32, device=self.dev)
        # fp32 copies of the small vectors the kernels read in fp32 (LayerNorm gains, biases)
        self.vec = {n: torch.empty(s.shape, **f32) for n, s in ((s.name, s) for s in slots) if len(s.shape) == 1}
        # transposed weight copies for dx = dy W
        self.wT = {s.name: torch.empty((s.shape[1], s.shape[0]), **bf) for s in slots
                   if len(s.shape) == 2 and s.name.startswith("blk.") and grads_f32 is not None}
        self.status = torch.zeros(1, dtype=torch.int32, device=self.dev)
        L = cfg.n_layers
        self.act = [dict(x_in=torch.empty((M, d), **bf), ln1=torch.empty((M, d), **bf), mean1=torch.empty(M, **f32),
                         rstd1=torch.empty(M, **f32), qkv=torch.empty((M, 3 * d), **bf), attn=torch.empty((M, d), **bf),
                         lse=torch.empty((micro_batch, cfg.n_heads, seq_len), **f32),
                         x_mid=torch.empty((M, d), **bf), ln2=torch.empty((M, d), **bf), mean2=torch.empty(M, **f32),
                         rstd2=torch.empty(M, **f32), h=torch.empty((M, f), **bf), a=torch.empty((M, f), **bf))
                    for _ in range(L)]
        self.x_out = torch.empty((M, d), **bf)
        self.lnf = torch.empty((M, d), **bf)
        self.meanf, self.rstdf = torch.empty(M, **f32), torch.empty(M, **f32)
        self.logits = torch.empty((M, self.Vp), **bf)
        self.loss_rows = torch.empty(M, **f32)
        self.kernel_launches = 0
        if grads_f32 is None:
            return
        # backward scratch
        self.dx = torch.empty((M, d), **bf)
        self.d_a = torch.empty((M, f), **bf)
        self.d_d = torch.empty((M, d), **bf)
        self.d_qkv = torch.empty((M, 3 * d), **bf)
        self.dsum = torch.empty((micro_batch, cfg.n_heads, seq_len), **f32)     # attention backward: rowsum(dO * O)
        self.tB = torch.empty(d * self.Vp, **bf)   # transposed tied embedding (dx of the LM head)
        self.kernel_launches = 0

    # ---- helpers
    def refresh_param_views(self, chunk=None):
        """Call after every optimizer step: fp32 vector copies and transposed matrices.  ``chunk``: only the views of one
        parameter chunk (``"rest"``: every vector; an int: that layer's transposed matrices), so that a chunked parameter
        all-gather can refresh each chunk's views right behind it."""
        if chunk is None or chunk == "rest":
            for n, v in self.vec.items():
                v.copy_(self.p[n])
        for n, t in self.wT.items():
            if chunk is None or (isinstance(chunk, int) and n.startswith(f"blk.{chunk}.")) or (chunk == "rest" and not n.startswith("blk.")):
                ops.transpose_bf16(self.p[n], t)
                self.kernel_launches += 1

    def _gemm(self, A, B, M, N, K, **kw):
        ops.gemm_bf16(A, B, M, N, K, status=self.status, **kw)
        self.kernel_launches += 1

    def _linear_fwd(self, x, wname, bname, out, resid=None):
        W = self.p[wname]
        N, K = W.shape
        self._gemm(x, W, x.shape[0], N, K, out_bf16=out, bias=self.vec[bname] if bname else None, resid_bf16=resid)

    def _linear_bwd(self, dy, x, wname, bname, dx_out):
        """dW += dy^T x, db += colsum(dy), dx_out = dy W (if requested)."""
        W = self.p[wname]
        N, K = W.shape
        M = dy.shape[0]
        self._gemm(dy, x, N, K, M, lda=dy.stride(0), ldb=x.stride(0), out_f32=self.g[wname], accumulate=True, mn_major=True)
        if bname:
            tops.bias_grad(dy, self.g[bname])
            self.kernel_launches += 1
        if dx_out is not None:
            self._gemm(dy, self.wT[wname], M, K, N, out_bf16=dx_out)

    # ---- forward + backward of one micro-batch; returns the mean loss (device scalar)
    def forward_backward(self, tokens: torch.Tensor, targets: torch.Tensor, loss_scale: float = 1.0, on_bucket=None, before_layer=None,
                         denom: float | None = None, backward: bool = True, row_scale_fn=None):
        """``backward=False``: forward only; returns a copy of the per-token losses ``-log p(target)`` [M] (0 where masked).
        ``row_scale_fn(loss_rows) -> (row_scale [M] fp32, reported loss)``: objectives that weight every token's log-likelihood
        gradient by a factor that depends on the losses themselves (preference optimisation): the losses are computed first
        with the logits left intact, the function runs on the device, then the gradient is written with those factors.
        ``denom``: with masked targets (negative ids contribute neither loss nor gradient) the caller passes the number of
        unmasked targets the loss is averaged over; the return value is then this micro-batch's share ``sum / denom``.
        ``on_bucket(i)`` is called right after the backward of layer ``i`` has been enqueued (its weight gradients are then
        final for this micro-batch) and ``on_bucket(None)`` at the very end (embeddings, norms and biases).
        ``before_layer("rest")`` is called before anything reads a parameter and ``before_layer(i)`` before layer ``i``'s
        forward (the trainer waits there for that chunk of the parameter all-gather)."""
        cfg, M, T, d = self.cfg, self.M, self.T, self.cfg.d_model
        H, hd = cfg.n_heads, cfg.head_dim
        ids = tokens.reshape(-1).to(torch.int32)
        tg = targets.reshape(-1).to(torch.int32)
        x = self.act[0]["x_in"]
        if before_layer is not None:
            before_layer("rest")
        tops.embed_fwd(ids, self.p["token_embd.weight"], self.p["position_embd.weight"], x, T)
        self.kernel_launches += 1
        for i, a in enumerate(self.act):
            pre = f"blk.{i}."
            x = a["x_in"]
            if before_layer is not None:
                before_layer(i)
            tops.layernorm_fwd(x, self.vec[pre + "attn_norm.weight"], self.vec[pre + "attn_norm.bias"], cfg.norm_eps,
                               a["ln1"], a["mean1"], a["rstd1"])
            self._linear_fwd(a["ln1"], pre + "attn_qkv.weight", pre + "attn_qkv.bias", a["qkv"])
            tops.attn_train_fwd(a["qkv"], a["attn"], a["lse"], self.B, T, H, hd)
            self._linear_fwd(a["attn"], pre + "attn_output.weight", pre + "attn_output.bias", a["x_mid"], resid=x)
            tops.layernorm_fwd(a["x_mid"], self.vec[pre + "ffn_norm.weight"], self.vec[pre + "ffn_norm.bias"],
                               cfg.norm_eps, a["ln2"], a["mean2"], a["rstd2"])
            self._linear_fwd(a["ln2"], pre + "ffn_up.weight", pre + "ffn_up.bias", a["h"])
            tops.gelu_fwd(a["h"], a["a"])
            nxt = self.act[i + 1]["x_in"] if i + 1 < len(self.act) else self.x_out
            self._linear_fwd(a["a"], pre + "ffn_down.weight", pre + "ffn_down.bias", nxt, resid=a["x_mid"])
            self.kernel_launches += 3
        tops.layernorm_fwd(self.x_out, self.vec["output_norm.weight"], self.vec["output_norm.bias"], cfg.norm_eps,
                           self.lnf, self.meanf, self.rstdf)
        wte = self.p["token_embd.weight"]
        self._gemm(self.lnf, wte, M, self.Vp, d, out_bf16=self.logits)
        if not backward:
            tops.ce_fused_rows(self.logits, tg, self.loss_rows, None, cfg.vocab)
            self.kernel_launches += 2
            return self.loss_rows.clone()
        if row_scale_fn is not None:
            tops.ce_fused_rows(self.logits, tg, self.loss_rows, None, cfg.vocab)
            row_scale, loss = row_scale_fn(self.loss_rows)
            tops.ce_fused_rows(self.logits, tg, self.loss_rows, row_scale.contiguous(), cfg.vocab)     # logits now hold dlogits
            self.kernel_launches += 3
        else:
            tops.ce_fused(self.logits, tg, self.loss_rows, loss_scale / M if denom is None else 1.0 / denom, cfg.vocab)     # logits now hold dlogits
            self.kernel_launches += 2
            loss = self.loss_rows.mean() if denom is None else self.loss_rows.sum() / denom

        # ---- backward
        dlog = self.logits
        # tied embedding: d wte += dlogits^T lnf ; d lnf = dlogits wte
        self._gemm(dlog, self.lnf, self.Vp, d, M, lda=self.Vp, ldb=d, out_f32=self.g["token_embd.weight"], accumulate=True, mn_major=True)
        wteT = self.tB[: d * self.Vp].view(d, self.Vp)
        ops.transpose_bf16(wte, wteT)
        self._gemm(dlog, wteT, M, d, self.Vp, out_bf16=self.d_d)
        tops.layernorm_bwd(self.d_d, self.x_out, self.vec["output_norm.weight"], self.meanf, self.rstdf, self.dx, False,
                           self.g["output_norm.weight"], self.g["output_norm.bias"])
        self.kernel_launches += 4
        for i in reversed(range(len(self.act))):
            a = self.act[i]
            pre = f"blk.{i}."
            # FFN branch: x_out = x_mid + down(gelu(up(ln2(x_mid))))
            self._linear_bwd(self.dx, a["a"], pre + "ffn_down.weight", pre + "ffn_down.bias", self.d_a)
            tops.gelu_bwd(a["h"], self.d_a)
            self._linear_bwd(self.d_a, a["ln2"], pre + "ffn_up.weight", pre + "ffn_up.bias", self.d_d)
            tops.layernorm_bwd(self.d_d, a["x_mid"], self.vec[pre + "ffn_norm.weight"], a["mean2"], a["rstd2"], self.dx,
                               True, self.g[pre + "ffn_norm.weight"], self.g[pre + "ffn_norm.bias"])
            # attention branch: x_mid = x_in + proj(attn(qkv(ln1(x_in))))
            self._linear_bwd(self.dx, a["attn"], pre + "attn_output.weight", pre + "attn_output.bias", self.d_d)
            tops.attn_train_bwd(a["qkv"], a["attn"], self.d_d, a["lse"], self.dsum, self.d_qkv, self.B, T, H, hd)
            self._linear_bwd(self.d_qkv, a["ln1"], pre + "attn_qkv.weight", pre + "attn_qkv.bias", self.d_d)
            tops.layernorm_bwd(self.d_d, a["x_in"], self.vec[pre + "attn_norm.weight"], a["mean1"], a["rstd1"], self.dx,
                               True, self.g[pre + "attn_norm.weight"], self.g[pre + "attn_norm.bias"])
            self.kernel_launches += 6
            if on_bucket is not None:
                on_bucket(i)
        tops.embed_bwd(ids, self.dx, self.g["token_embd.weight"], self.g["position_embd.weight"], T)
        self.kernel_launches += 1
        if on_bucket is not None:
            on_bucket(None)
        return loss
