"""GGUF reader and writer objects over the C++ implementation."""
from __future__ import annotations

import ctypes
import json
from dataclasses import dataclass

import numpy as np

from .. import _native
from .formats import GgmlType, dequantize, tensor_nbytes

_GV = {"u8": 0, "i8": 1, "u16": 2, "i16": 3, "u32": 4, "i32": 5, "f32": 6, "bool": 7,
       "str": 8, "u64": 10, "i64": 11, "f64": 12}
_NP_OF_GV = {0: np.uint8, 1: np.int8, 2: np.uint16, 3: np.int16, 4: np.uint32, 5: np.int32,
             6: np.float32, 10: np.uint64, 11: np.int64, 12: np.float64}


def _lib():
    lib = _native.host()
    if getattr(lib, "_b200_gguf_ready", False):
        return lib
    vp, u64, u32, cp = ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_char_p
    sig = {
        "b200_gguf_open": ([cp], vp), "b200_gguf_error": ([vp], cp), "b200_gguf_close": ([vp], None),
        "b200_gguf_version": ([vp], u32), "b200_gguf_alignment": ([vp], u64),
        "b200_gguf_meta_json": ([vp], cp), "b200_gguf_n_tensors": ([vp], u64),
        "b200_gguf_tensor_name": ([vp, u64], cp), "b200_gguf_tensor_type": ([vp, u64], u32),
        "b200_gguf_tensor_ndim": ([vp, u64], u32), "b200_gguf_tensor_dim": ([vp, u64, u32], u64),
        "b200_gguf_tensor_nbytes": ([vp, u64], u64), "b200_gguf_tensor_offset": ([vp, u64], u64),
        "b200_gguf_tensor_data": ([vp, u64], vp),
        "b200_gguf_writer_new": ([cp, u32], vp),
        "b200_gguf_writer_kv_u32": ([vp, cp, u32], None),
        "b200_gguf_writer_kv_i32": ([vp, cp, ctypes.c_int32], None),
        "b200_gguf_writer_kv_u64": ([vp, cp, u64], None),
        "b200_gguf_writer_kv_f32": ([vp, cp, ctypes.c_float], None),
        "b200_gguf_writer_kv_bool": ([vp, cp, ctypes.c_int], None),
        "b200_gguf_writer_kv_str": ([vp, cp, cp, u64], None),
        "b200_gguf_writer_kv_str_array": ([vp, cp, cp, ctypes.POINTER(u64), u64], None),
        "b200_gguf_writer_kv_array": ([vp, cp, u32, vp, u64, u32], None),
        "b200_gguf_writer_tensor": ([vp, cp, u32, u32, ctypes.POINTER(u64), vp], ctypes.c_int),
        "b200_gguf_writer_finish": ([vp], ctypes.c_int), "b200_gguf_writer_error": ([vp], cp),
        "b200_gguf_writer_free": ([vp], None),
    }
    for name, (args, res) in sig.items():
        fn = getattr(lib, name)
        fn.argtypes, fn.restype = args, res
    lib._b200_gguf_ready = True
    return lib


@dataclass
class GGUFTensor:
    """One tensor of an open file.  ``shape`` is row-major (slowest axis first), the reverse of
    the on-disk dimension order."""
    name: str
    type: GgmlType
    shape: tuple[int, ...]
    nbytes: int
    offset: int
    data: np.ndarray  # uint8 view into the mapping

    def to_float(self) -> np.ndarray:
        return dequantize(self.data, self.type, self.shape)


class GGUFFile:
    """A memory-mapped GGUF file.  Tensors are zero-copy views valid until ``close``."""

    def __init__(self, path: str):
        lib = _lib()
        self._lib = lib
        self._h = lib.b200_gguf_open(str(path).encode())
        err = lib.b200_gguf_error(self._h)
        if err:
            msg = err.decode()
            lib.b200_gguf_close(self._h)
            self._h = None
            raise ValueError(f"{path}: {msg}")
        self.path = str(path)
        self.version = lib.b200_gguf_version(self._h)
        self.alignment = lib.b200_gguf_alignment(self._h)
        self.metadata: dict = json.loads(lib.b200_gguf_meta_json(self._h).decode("utf-8", "replace"))
        self.tensors: dict[str, GGUFTensor] = {}
        for i in range(lib.b200_gguf_n_tensors(self._h)):
            nd = lib.b200_gguf_tensor_ndim(self._h, i)
            dims = [lib.b200_gguf_tensor_dim(self._h, i, d) for d in range(nd)]
            nbytes = lib.b200_gguf_tensor_nbytes(self._h, i)
            ptr = lib.b200_gguf_tensor_data(self._h, i)
            arr = np.ctypeslib.as_array((ctypes.c_uint8 * nbytes).from_address(ptr)) if nbytes else np.empty(0, np.uint8)
            name = lib.b200_gguf_tensor_name(self._h, i).decode()
            self.tensors[name] = GGUFTensor(name, GgmlType(lib.b200_gguf_tensor_type(self._h, i)),
                                            tuple(reversed(dims)), nbytes,
                                            lib.b200_gguf_tensor_offset(self._h, i), arr)

    @property
    def architecture(self) -> str:
        return self.metadata.get("general.architecture", "")

    def close(self):
        if self._h is not None:
            self.tensors.clear()
            self._lib.b200_gguf_close(self._h)
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class GGUFWriter:
    """Collects metadata and tensors, then writes the file atomically (temp name + rename)."""

    def __init__(self, path: str, alignment: int = 32):
        self._lib = _lib()
        self._h = self._lib.b200_gguf_writer_new(str(path).encode(), alignment)
        self._keep: list = []

    def add_meta(self, key: str, value, kind: str | None = None):
        lib, h, k = self._lib, self._h, key.encode()
        if key == "general.alignment":
            return
        if kind is None:
            if isinstance(value, bool):
                kind = "bool"
            elif isinstance(value, int):
                kind = "u32" if 0 <= value < 2**32 else ("u64" if value >= 0 else "i32")
            elif isinstance(value, float):
                kind = "f32"
            elif isinstance(value, str):
                kind = "str"
            elif isinstance(value, (list, tuple, np.ndarray)):
                kind = "array"
            else:
                raise TypeError(f"cannot infer GGUF type for {key}={value!r}")
        if kind == "u32":
            lib.b200_gguf_writer_kv_u32(h, k, int(value))
        elif kind == "i32":
            lib.b200_gguf_writer_kv_i32(h, k, int(value))
        elif kind == "u64":
            lib.b200_gguf_writer_kv_u64(h, k, int(value))
        elif kind == "f32":
            lib.b200_gguf_writer_kv_f32(h, k, float(value))
        elif kind == "bool":
            lib.b200_gguf_writer_kv_bool(h, k, int(bool(value)))
        elif kind == "str":
            b = value.encode()
            lib.b200_gguf_writer_kv_str(h, k, b, len(b))
        elif kind == "array":
            if len(value) and isinstance(value[0], str):
                parts = [s.encode() for s in value]
                lens = (ctypes.c_uint64 * len(parts))(*[len(p) for p in parts])
                lib.b200_gguf_writer_kv_str_array(h, k, b"".join(parts), lens, len(parts))
            else:
                arr = np.asarray(value)
                if arr.dtype.kind == "f":
                    arr, et = arr.astype(np.float32), _GV["f32"]
                elif arr.dtype.kind == "b":
                    arr, et = arr.astype(np.uint8), _GV["bool"]
                else:
                    arr, et = arr.astype(np.int32), _GV["i32"]
                arr = np.ascontiguousarray(arr)
                lib.b200_gguf_writer_kv_array(h, k, et, arr.ctypes.data, arr.size, arr.itemsize)
        else:
            raise ValueError(kind)

    def add_tensor_raw(self, name: str, t: int, shape, data: np.ndarray):
        """``data`` holds the packed bytes of a tensor of row-major ``shape``."""
        data = np.ascontiguousarray(data).view(np.uint8).reshape(-1)
        n = int(np.prod(shape))
        if data.size != tensor_nbytes(t, n):
            raise ValueError(f"{name}: {data.size} bytes given, {tensor_nbytes(t, n)} expected")
        self._keep.append(data)
        dims = (ctypes.c_uint64 * len(shape))(*reversed([int(s) for s in shape]))
        if self._lib.b200_gguf_writer_tensor(self._h, name.encode(), int(t), len(shape), dims, data.ctypes.data) != 0:
            raise ValueError(self._lib.b200_gguf_writer_error(self._h).decode())

    def add_tensor(self, name: str, x: np.ndarray, t: int = GgmlType.F32):
        from .formats import quantize
        self.add_tensor_raw(name, t, x.shape, quantize(x, t))

    def write(self):
        rc = self._lib.b200_gguf_writer_finish(self._h)
        err = self._lib.b200_gguf_writer_error(self._h)
        self._lib.b200_gguf_writer_free(self._h)
        self._h = None
        self._keep.clear()
        if rc != 0:
            raise IOError(err.decode() if err else "GGUF write failed")
