"""Block-format ids and CPU quantize / dequantize entry points."""
from __future__ import annotations

import ctypes
import enum

import numpy as np

from .. import _native


class GgmlType(enum.IntEnum):
    F32 = 0
    F16 = 1
    Q8_0 = 8
    Q4_K = 12
    Q5_K = 13
    Q6_K = 14
    BF16 = 30
    MXFP4 = 39


GGML_TYPES = {t.name: t for t in GgmlType}


def _lib():
    lib = _native.host()
    if not getattr(lib, "_b200_quant_ready", False):
        lib.b200_type_info.argtypes = [ctypes.c_uint32, ctypes.POINTER(ctypes.c_uint32),
                                       ctypes.POINTER(ctypes.c_uint32)]
        lib.b200_type_info.restype = ctypes.c_int
        lib.b200_type_name.argtypes = [ctypes.c_uint32]
        lib.b200_type_name.restype = ctypes.c_char_p
        lib.b200_dequantize.argtypes = [ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64]
        lib.b200_dequantize.restype = ctypes.c_int
        lib.b200_quantize.argtypes = [ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64]
        lib.b200_quantize.restype = ctypes.c_int
        lib._b200_quant_ready = True
    return lib


def type_block(t: int) -> tuple[int, int]:
    """(elements per block, bytes per block)."""
    be, bb = ctypes.c_uint32(), ctypes.c_uint32()
    if _lib().b200_type_info(int(t), ctypes.byref(be), ctypes.byref(bb)) != 0:
        raise ValueError(f"unsupported ggml type {t}")
    return be.value, bb.value


def type_name(t: int) -> str:
    n = _lib().b200_type_name(int(t))
    if n is None:
        raise ValueError(f"unsupported ggml type {t}")
    return n.decode()


def tensor_nbytes(t: int, n_elems: int) -> int:
    be, bb = type_block(t)
    if n_elems % be:
        raise ValueError(f"{n_elems} elements is not a multiple of the {type_name(t)} block ({be})")
    return n_elems // be * bb


def quantize(x: np.ndarray, t: int) -> np.ndarray:
    """fp32 array -> packed bytes (uint8, 1-D).  The last axis must be a multiple of the block."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    be, _ = type_block(t)
    if x.shape[-1] % be:
        raise ValueError(f"row length {x.shape[-1]} is not a multiple of the {type_name(t)} block ({be})")
    out = np.empty(tensor_nbytes(t, x.size), dtype=np.uint8)
    if _lib().b200_quantize(int(t), x.ctypes.data, out.ctypes.data, x.size) != 0:
        raise ValueError("quantize failed")
    return out


def dequantize(buf, t: int, shape) -> np.ndarray:
    """Packed bytes -> fp32 array of ``shape`` (row-major, last axis contiguous)."""
    buf = np.ascontiguousarray(np.frombuffer(buf, dtype=np.uint8) if not isinstance(buf, np.ndarray) else buf.view(np.uint8).reshape(-1))
    n = int(np.prod(shape))
    if buf.size != tensor_nbytes(t, n):
        raise ValueError(f"buffer has {buf.size} bytes, expected {tensor_nbytes(t, n)}")
    out = np.empty(n, dtype=np.float32)
    if _lib().b200_dequantize(int(t), buf.ctypes.data, out.ctypes.data, n) != 0:
        raise ValueError("dequantize failed")
    return out.reshape(shape)
