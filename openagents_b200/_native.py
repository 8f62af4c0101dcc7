"""Loading of the in-tree native libraries through ctypes.

``host()`` returns the C++ host library (GGUF, quantization, KV page allocator, digests) and works
on any machine.  ``cuda()`` returns the sm_100a kernel library; on a machine with a GPU a missing
or unbuildable library is an error, never a silent fallback.
"""
from __future__ import annotations

import ctypes
import os
import threading

from . import _build

_lock = threading.Lock()
_host = None
_cuda = None


def _load(kind: str) -> ctypes.CDLL:
    path = _build.host_lib_path() if kind == "host" else _build.cuda_lib_path()
    if os.environ.get("B200_NO_REBUILD") != "1" and _build.is_stale(kind):
        (_build.build_host if kind == "host" else _build.build_cuda)()
    if not path.exists():
        raise RuntimeError(f"native library {path} is missing; run `python -m openagents_b200._build`")
    return ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)


def host() -> ctypes.CDLL:
    global _host
    with _lock:
        if _host is None:
            _host = _load("host")
        return _host


def cuda() -> ctypes.CDLL:
    global _cuda
    with _lock:
        if _cuda is None:
            _cuda = _load("cuda")
        return _cuda


def cuda_available() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False
