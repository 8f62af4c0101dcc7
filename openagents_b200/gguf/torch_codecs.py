"""Vectorised (torch) block codecs and the repack into the engine's device layouts.

These run on whatever device the input tensor lives on.  They are load/save-time code: a model is
quantized or repacked once, never inside a decode or training step.  ``quantize_*`` produce the
standard GGUF byte layout (bit-compatible with the C++ codecs); ``repack_*`` turn that layout into
the one the sm_100a kernels read:

* **Q4_K-R**: the 144-byte superblock keeps its 16-byte header; inside each 32-byte group the
  sixty-four 4-bit values are re-ordered so that word ``w`` holds elements ``8w..8w+7`` with element
  ``i`` at bit ``4*(i//2) + 16*(i%2)``.  ``(v >> 4s) & 0x000F000F`` then yields two *adjacent*
  elements as the mantissas of a bf16x2 pair, and ``v & 0x0F0F0F0F`` yields int8 lanes for ``dp4a``.
* **Q6_K-R**: per superblock 208 bytes ``[ql-r 128][qh-r 64][scales 16]`` plus a separate fp16 ``d``
  plane, with the low nibbles in the Q4_K-R word order and the high bit-pairs packed to match.
* **Q8_0-R**: an int8 plane in the activation byte order plus an fp16 scale plane.
* **MXFP4-R**: a nibble plane (Q4_K-R word order) plus an E8M0 exponent plane.

The activation byte order ("x8 order") places element ``i`` of every 8 at byte ``X8_POS[i]``.
"""
from __future__ import annotations

import torch

from .formats import GgmlType

# element i of each group of 8 sits at this byte / nibble slot
X8_ORDER = (0, 4, 1, 5, 2, 6, 3, 7)          # slot -> element
X8_POS = tuple(X8_ORDER.index(i) for i in range(8))  # element -> slot
_NIB_SHIFT = tuple(4 * (i // 2) + 16 * (i % 2) for i in range(8))


def _f16_bytes(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.float16).contiguous().view(torch.uint8)


def _round(x: torch.Tensor) -> torch.Tensor:
    return torch.round(x)  # half-to-even, as lrintf in the default rounding mode


# ------------------------------------------------------------------ standard GGUF layouts

def quantize_q8_0(x: torch.Tensor) -> torch.Tensor:
    xb = x.float().reshape(-1, 32)
    amax = xb.abs().amax(-1, keepdim=True)
    d = (amax / 127.0).to(torch.float16)
    df = d.float()
    inv = torch.where(df > 0, 1.0 / df, torch.zeros_like(df))
    q = _round(xb * inv).clamp_(-127, 127).to(torch.int8)
    return torch.cat((d.view(torch.uint8).reshape(-1, 2), q.view(torch.uint8)), dim=1).reshape(-1)


def _kquant_scales(xb: torch.Tensor, nmax: int):
    """xb: [nb, 8, 32] -> d, dmin (fp16-rounded fp32 [nb,1]), ls, lm (uint8 [nb, 8])."""
    lo = xb.amin(-1).clamp(max=0.0)
    hi = torch.maximum(xb.amax(-1), lo)
    scales = (hi - lo) / nmax
    mins = -lo
    d = (scales.amax(-1, keepdim=True) / 63.0).to(torch.float16).float()
    dmin = (mins.amax(-1, keepdim=True) / 63.0).to(torch.float16).float()
    ls = torch.where(d > 0, _round(scales / d), torch.zeros_like(scales)).clamp_(0, 63)
    lm = torch.where(dmin > 0, _round(mins / dmin), torch.zeros_like(mins)).clamp_(0, 63)
    return d, dmin, ls.to(torch.uint8), lm.to(torch.uint8)


def _pack_scale_min(ls: torch.Tensor, lm: torch.Tensor) -> torch.Tensor:
    q = torch.zeros(ls.shape[0], 12, dtype=torch.uint8, device=ls.device)
    q[:, 0:4] = (ls[:, 0:4] & 63) | ((ls[:, 4:8] >> 4) << 6)
    q[:, 4:8] = (lm[:, 0:4] & 63) | ((lm[:, 4:8] >> 4) << 6)
    q[:, 8:12] = (ls[:, 4:8] & 0xF) | ((lm[:, 4:8] & 0xF) << 4)
    return q


def _unpack_scale_min(q: torch.Tensor):
    q = q.to(torch.int32)
    ls = torch.cat(((q[:, 0:4] & 63), (q[:, 8:12] & 0xF) | ((q[:, 0:4] >> 6) << 4)), dim=1)
    lm = torch.cat(((q[:, 4:8] & 63), (q[:, 8:12] >> 4) | ((q[:, 4:8] >> 6) << 4)), dim=1)
    return ls, lm


def quantize_q4_k(x: torch.Tensor) -> torch.Tensor:
    xb = x.float().reshape(-1, 8, 32)
    d, dmin, ls, lm = _kquant_scales(xb, 15)
    a = (d * ls.float())[..., None]
    m = (dmin * lm.float())[..., None]
    L = torch.where(a > 0, _round((xb + m) / a), torch.zeros_like(xb)).clamp_(0, 15).to(torch.uint8)
    L = L.reshape(-1, 4, 2, 32)
    qs = (L[:, :, 0] | (L[:, :, 1] << 4)).reshape(-1, 128)
    head = torch.cat((_f16_bytes(d).reshape(-1, 2), _f16_bytes(dmin).reshape(-1, 2), _pack_scale_min(ls, lm)), dim=1)
    return torch.cat((head, qs), dim=1).reshape(-1)


def dequantize_q4_k(buf: torch.Tensor, n: int) -> torch.Tensor:
    b = buf.reshape(-1, 144)
    d = b[:, 0:2].contiguous().view(torch.float16).float()
    dmin = b[:, 2:4].contiguous().view(torch.float16).float()
    ls, lm = _unpack_scale_min(b[:, 4:16])
    qs = b[:, 16:].reshape(-1, 4, 32)
    L = torch.stack((qs & 0xF, qs >> 4), dim=2).reshape(-1, 8, 32).float()
    y = (d * ls.float())[..., None] * L - (dmin * lm.float())[..., None]
    return y.reshape(-1)[:n]


def quantize_q6_k(x: torch.Tensor) -> torch.Tensor:
    xb = x.float().reshape(-1, 16, 16)
    scales = xb.abs().amax(-1) / 31.0
    d = (scales.amax(-1, keepdim=True) / 127.0).to(torch.float16).float()
    s = torch.where(d > 0, _round(scales / d), torch.zeros_like(scales)).clamp_(0, 127)
    a = (d * s)[..., None]
    q = torch.where(a > 0, _round(xb / a), torch.zeros_like(xb)).clamp_(-32, 31) + 32
    L = q.to(torch.uint8).reshape(-1, 2, 4, 32)            # [nb, half, quarter, l]
    q1, q2, q3, q4 = L[:, :, 0], L[:, :, 1], L[:, :, 2], L[:, :, 3]
    ql = torch.cat(((q1 & 0xF) | ((q3 & 0xF) << 4), (q2 & 0xF) | ((q4 & 0xF) << 4)), dim=-1).reshape(-1, 128)
    qh = ((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6)).reshape(-1, 64)
    return torch.cat((ql, qh, s.to(torch.int8).view(torch.uint8), _f16_bytes(d).reshape(-1, 2)), dim=1).reshape(-1)


def _q6k_fields(buf: torch.Tensor):
    b = buf.reshape(-1, 210)
    ql = b[:, 0:128].reshape(-1, 2, 2, 32).to(torch.int32)   # [nb, half, which(l / l+32), l]
    qh = b[:, 128:192].reshape(-1, 2, 32).to(torch.int32)
    sc = b[:, 192:208].contiguous().view(torch.int8)
    d = b[:, 208:210].contiguous().view(torch.float16)
    q1 = (ql[:, :, 0] & 0xF) | (((qh >> 0) & 3) << 4)
    q2 = (ql[:, :, 1] & 0xF) | (((qh >> 2) & 3) << 4)
    q3 = (ql[:, :, 0] >> 4) | (((qh >> 4) & 3) << 4)
    q4 = (ql[:, :, 1] >> 4) | (((qh >> 6) & 3) << 4)
    L = torch.stack((q1, q2, q3, q4), dim=2).reshape(-1, 256)   # element order, values 0..63
    return L, sc, d


def dequantize_q6_k(buf: torch.Tensor, n: int) -> torch.Tensor:
    L, sc, d = _q6k_fields(buf)
    y = d.float()[:, :, None] * sc.float()[:, :, None] * (L.reshape(-1, 16, 16).float() - 32.0)
    return y.reshape(-1)[:n]


_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def quantize_mxfp4(x: torch.Tensor) -> torch.Tensor:
    xb = x.float().reshape(-1, 32)
    amax = xb.abs().amax(-1, keepdim=True)
    _, ex = torch.frexp(amax)
    e = torch.where(amax > 0, ex - 1 - 2 + 127, torch.zeros_like(ex)).clamp_(0, 254)
    v = xb * torch.exp2((127 - e).float())
    a = v.abs()
    # round-to-nearest-even onto {0, .5, 1, 1.5, 2, 3, 4, 6}
    bounds = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], device=x.device)
    code = torch.bucketize(a, bounds, right=False)            # a <= bound -> lower bucket
    tie_up = torch.tensor([0, 1, 0, 1, 0, 1, 0], device=x.device, dtype=torch.bool)  # ties to even mantissa
    is_tie = (a[..., None] == bounds).any(-1)
    idx = torch.bucketize(a, bounds, right=False).clamp(max=6)
    code = torch.where(is_tie & tie_up[idx], code + 1, code).clamp_(0, 7)
    code = (code | ((v < 0) | ((v == 0) & torch.signbit(v))).to(code.dtype) * 8).to(torch.uint8)
    qs = code[:, :16] | (code[:, 16:] << 4)
    return torch.cat((e.to(torch.uint8), qs), dim=1).reshape(-1)


def dequantize_mxfp4(buf: torch.Tensor, n: int) -> torch.Tensor:
    b = buf.reshape(-1, 17)
    s = torch.exp2(b[:, 0:1].float() - 127.0)
    lut = torch.tensor(_E2M1 + tuple(-v for v in _E2M1), device=buf.device)
    qs = b[:, 1:].long()
    y = torch.cat((lut[qs & 0xF], lut[qs >> 4]), dim=1) * s
    return y.reshape(-1)[:n]


def quantize(x: torch.Tensor, t: int) -> torch.Tensor:
    """fp32 tensor -> standard GGUF bytes (uint8, 1-D) on x's device."""
    t = GgmlType(t)
    if t == GgmlType.F32:
        return x.float().contiguous().view(torch.uint8).reshape(-1)
    if t == GgmlType.F16:
        return x.to(torch.float16).contiguous().view(torch.uint8).reshape(-1)
    if t == GgmlType.BF16:
        return x.to(torch.bfloat16).contiguous().view(torch.uint8).reshape(-1)
    return {GgmlType.Q8_0: quantize_q8_0, GgmlType.Q4_K: quantize_q4_k, GgmlType.Q6_K: quantize_q6_k,
            GgmlType.MXFP4: quantize_mxfp4}[t](x)


def dequantize(buf: torch.Tensor, t: int, shape) -> torch.Tensor:
    t = GgmlType(t)
    n = 1
    for s in shape:
        n *= int(s)
    buf = buf.reshape(-1)
    if t == GgmlType.F32:
        return buf.view(torch.float32).reshape(shape).clone()
    if t == GgmlType.F16:
        return buf.view(torch.float16).float().reshape(shape)
    if t == GgmlType.BF16:
        return buf.view(torch.bfloat16).float().reshape(shape)
    if t == GgmlType.Q8_0:
        b = buf.reshape(-1, 34)
        return (b[:, :2].contiguous().view(torch.float16).float() * b[:, 2:].contiguous().view(torch.int8).float()).reshape(shape)
    return {GgmlType.Q4_K: dequantize_q4_k, GgmlType.Q6_K: dequantize_q6_k,
            GgmlType.MXFP4: dequantize_mxfp4}[t](buf, n).reshape(shape)


# ------------------------------------------------------------------ engine layouts

def _pack_nibble_words(L: torch.Tensor) -> torch.Tensor:
    """L: [..., 8] values 0..15 (element order) -> int32 words [...] in the Q4_K-R bit order."""
    L = L.to(torch.int64)
    w = torch.zeros(L.shape[:-1], dtype=torch.int64, device=L.device)
    for i in range(8):
        w |= L[..., i] << _NIB_SHIFT[i]
    return _wrap_i32(w)


def _wrap_i32(w: torch.Tensor) -> torch.Tensor:
    """int64 holding a 32-bit pattern -> int32 with the same bits."""
    w = w & 0xFFFFFFFF
    return torch.where(w >= 2 ** 31, w - 2 ** 32, w).to(torch.int32)


def _words_to_bytes(w: torch.Tensor) -> torch.Tensor:
    return w.contiguous().view(torch.uint8)


def repack_q4_k(buf: torch.Tensor) -> torch.Tensor:
    """Standard Q4_K bytes -> Q4_K-R bytes (same size)."""
    b = buf.reshape(-1, 144)
    qs = b[:, 16:].reshape(-1, 4, 32)
    L = torch.stack((qs & 0xF, qs >> 4), dim=2).reshape(-1, 32, 8)     # [nb, word, elem]
    words = _pack_nibble_words(L)                                        # [nb, 32]
    return torch.cat((b[:, :16], _words_to_bytes(words).reshape(-1, 128)), dim=1).reshape(-1)


def unpack_q4_k_r(buf: torch.Tensor) -> torch.Tensor:
    """Inverse of ``repack_q4_k`` (used when a served model is saved back to GGUF)."""
    b = buf.reshape(-1, 144)
    w = b[:, 16:].contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF     # [nb, 32]
    L = torch.stack([(w >> _NIB_SHIFT[i]) & 0xF for i in range(8)], dim=-1)        # [nb, 32, 8]
    L = L.reshape(-1, 4, 2, 32).to(torch.uint8)
    qs = (L[:, :, 0] | (L[:, :, 1] << 4)).reshape(-1, 128)
    return torch.cat((b[:, :16], qs), dim=1).reshape(-1)


def repack_q6_k(buf: torch.Tensor):
    """Standard Q6_K bytes -> (main plane [nb*208] uint8, d plane [nb] fp16)."""
    L, sc, d = _q6k_fields(buf)                                          # L: [nb, 256]
    lo = _pack_nibble_words((L & 0xF).reshape(-1, 32, 8))                # [nb, 32] words
    hi2 = (L >> 4).reshape(-1, 16, 16).to(torch.int64)                   # 16 elements per T word
    t = torch.zeros(hi2.shape[:2], dtype=torch.int64, device=buf.device)
    # T word for 16 elements = two weight words; within a word, byte lane b of the "lo" extraction holds
    # element X8_ORDER[b] and of the "hi" extraction element X8_ORDER[4 + b].
    for word in range(2):
        for half in range(2):          # 0: lo extraction (shift 0), 1: hi extraction (shift 2)
            for lane in range(4):
                elem = X8_ORDER[4 * half + lane] + 8 * word
                t |= hi2[:, :, elem] << (8 * lane + 2 * half + 4 * word)
    tw = _wrap_i32(t)
    main = torch.cat((_words_to_bytes(lo).reshape(-1, 128), _words_to_bytes(tw).reshape(-1, 64),
                      sc.view(torch.uint8).reshape(-1, 16)), dim=1)
    return main.reshape(-1), d.reshape(-1).clone()


def repack_q8_0(buf: torch.Tensor):
    """Standard Q8_0 bytes -> (int8 plane in x8 order [n], fp16 scale plane [n/32])."""
    b = buf.reshape(-1, 34)
    d = b[:, :2].contiguous().view(torch.float16).reshape(-1).clone()
    q = b[:, 2:].reshape(-1, 4, 8)[:, :, list(X8_ORDER)]
    return q.reshape(-1).contiguous().view(torch.int8), d


def repack_mxfp4(buf: torch.Tensor):
    """Standard MXFP4 bytes -> (nibble plane [n/2] in Q4_K-R word order, E8M0 plane [n/32])."""
    b = buf.reshape(-1, 17)
    qs = b[:, 1:]
    L = torch.cat((qs & 0xF, qs >> 4), dim=1).reshape(-1, 4, 8)          # element order codes
    words = _pack_nibble_words(L)
    return _words_to_bytes(words).reshape(-1), b[:, 0].clone()


def to_x8_order(x: torch.Tensor) -> torch.Tensor:
    """Permute the last axis (multiple of 8) into the activation byte order."""
    sh = x.shape
    return x.reshape(*sh[:-1], sh[-1] // 8, 8)[..., list(X8_ORDER)].reshape(sh)
