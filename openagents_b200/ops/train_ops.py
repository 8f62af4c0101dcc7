"""Python faces of the training-path kernels (``csrc/kernels/train_ops.cu``, ``csrc/comm/zero_adamw.cu``)."""
from __future__ import annotations

from ctypes import c_float, c_int, c_size_t, c_void_p


from .. import _native
from .cuda_ops import _check, _p, _st, _sym

_P = c_void_p
_SIGS = {
    "b200_embed_fwd": [_P, _P, _P, _P, c_int, c_int, c_int, _P],
    "b200_embed_bwd": [_P, _P, _P, _P, c_int, c_int, c_int, _P],
    "b200_layernorm_fwd": [_P, _P, _P, c_float, _P, _P, _P, c_int, c_int, _P],
    "b200_layernorm_bwd": [_P, _P, _P, _P, _P, _P, c_int, _P, _P, c_int, c_int, _P],
    "b200_gelu_fwd": [_P, _P, c_size_t, _P],
    "b200_gelu_bwd": [_P, _P, c_size_t, _P],
    "b200_bias_grad": [_P, _P, c_int, c_int, _P],
    "b200_ce_fused": [_P, _P, _P, c_float, c_int, c_int, c_int, _P],
    "b200_ce_fused_rows": [_P, _P, _P, _P, c_int, c_int, c_int, c_int, _P],
    "b200_attn_train_fwd": [_P, _P, _P, c_int, c_int, c_int, c_int, _P],
    "b200_attn_train_bwd": [_P, _P, _P, _P, _P, _P, c_int, c_int, c_int, c_int, _P],
    "b200_zero_reduce_norm": [_P, c_size_t, c_size_t, c_size_t, _P, _P, _P],
    "b200_zero_adamw_gather": [_P, c_size_t, c_size_t, c_size_t, _P, _P, _P, _P, _P, c_float, c_float, c_float, c_float,
                               c_float, c_float, c_float, c_float, c_size_t, _P],
}
_lib = None


def lib():
    global _lib
    if _lib is None:
        L = _native.cuda()
        for n, a in _SIGS.items():
            f = getattr(L, n)
            f.argtypes, f.restype = a, c_int
        _lib = L
    return _lib


def embed_fwd(ids, wte, wpe, x, T):
    _check(lib().b200_embed_fwd(_p(ids), _p(wte), _p(wpe), _p(x), ids.numel(), T, x.shape[-1], _st()), "embed_fwd")


def embed_bwd(ids, dx, gwte, gwpe, T):
    _check(lib().b200_embed_bwd(_p(ids), _p(dx), _p(gwte), _p(gwpe), ids.numel(), T, dx.shape[-1], _st()), "embed_bwd")


def layernorm_fwd(x, g, b, eps, y, mean, rstd):
    rows, D = x.shape
    _check(lib().b200_layernorm_fwd(_p(x), _p(g), _p(b), eps, _p(y), _p(mean), _p(rstd), rows, D, _st()), "layernorm_fwd")


def layernorm_bwd(dy, x, g, mean, rstd, dx, dx_add, dgamma, dbeta):
    rows, D = x.shape
    _check(lib().b200_layernorm_bwd(_p(dy), _p(x), _p(g), _p(mean), _p(rstd), _p(dx), int(dx_add), _p(dgamma), _p(dbeta),
                                    rows, D, _st()), "layernorm_bwd")


def gelu_fwd(x, y):
    _check(lib().b200_gelu_fwd(_p(x), _p(y), x.numel(), _st()), "gelu_fwd")


def gelu_bwd(x, dy):
    _check(lib().b200_gelu_bwd(_p(x), _p(dy), x.numel(), _st()), "gelu_bwd")


def bias_grad(dy, gb):
    M, N = dy.shape
    _check(lib().b200_bias_grad(_p(dy), _p(gb), M, N, _st()), "bias_grad")


def ce_fused(logits, targets, loss, scale, V):
    M, ldl = logits.shape
    _check(lib().b200_ce_fused(_p(logits), _p(targets), _p(loss), scale, M, V, ldl, _st()), "ce_fused")


def ce_fused_rows(logits, targets, loss, row_scale, V):
    """Per-row losses only (``row_scale`` None: the logits are left untouched) or losses + gradients scaled row by row."""
    M, ldl = logits.shape
    _check(lib().b200_ce_fused_rows(_p(logits), _p(targets), _p(loss), _p(row_scale) if row_scale is not None else None,
                                    int(row_scale is not None), M, V, ldl, _st()), "ce_fused_rows")


def attn_train_fwd(qkv, o, lse, B, T, H, hd):
    """Causal attention forward on the fused projection output ``qkv`` [B*T, 3*H*hd] bf16 (read in place) ->
    ``o`` [B*T, H*hd] bf16 and ``lse`` [B, H, T] fp32 (see ``attn_train.cu``)."""
    _check(lib().b200_attn_train_fwd(_p(qkv), _p(o), _p(lse), B, T, H, hd, _st()), "attn_train_fwd")


def attn_train_bwd(qkv, o, d_o, lse, dsum, dqkv, B, T, H, hd):
    """Backward of :func:`attn_train_fwd`: ``dqkv`` [B*T, 3*H*hd] bf16 from ``d_o``; ``dsum`` [B, H, T] fp32 is working space."""
    _check(lib().b200_attn_train_bwd(_p(qkv), _p(o), _p(d_o), _p(lse), _p(dsum), _p(dqkv), B, T, H, hd, _st()), "attn_train_bwd")


def zero_reduce_norm(table, grad_off, lo, n, gshard, norm2):
    _check(lib().b200_zero_reduce_norm(_sym(table), grad_off, lo, n, _p(gshard), _p(norm2), _st()), "zero_reduce_norm")


def zero_adamw_gather(table, param_off, lo, n, gshard, master, m, v, norm2, lr, beta1, beta2, eps, wd, bc1, bc2,
                      max_norm, decay_end):
    _check(lib().b200_zero_adamw_gather(_sym(table), param_off, lo, n, _p(gshard), _p(master), _p(m), _p(v), _p(norm2),
                                        lr, beta1, beta2, eps, wd, bc1, bc2, max_norm, decay_end, _st()),
           "zero_adamw_gather")
