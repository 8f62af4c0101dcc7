"""NVTX ranges around the phases a timeline should show: prefill, decode step, fused collectives, optimizer step.

Off unless ``B200_NVTX=1``: a range costs a host call on a path that otherwise only replays a CUDA graph, so the
marks are for profiling sessions, not for production serving.  Without CUDA the context manager does nothing.
"""
from __future__ import annotations

import contextlib
import os

_ON = os.environ.get("B200_NVTX", "0") == "1"


def enabled() -> bool:
    return _ON


@contextlib.contextmanager
def nvtx_range(name: str):
    if not _ON:
        yield
        return
    import torch
    if not torch.cuda.is_available():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


def nvtx_method(name: str):
    """Decorator form: the function runs inside a range called ``name``.  With the marks off it returns the function
    itself, so a decorated hot-path method costs nothing extra."""
    def wrap(fn):
        if not _ON:
            return fn
        import functools

        @functools.wraps(fn)
        def inner(*a, **kw):
            with nvtx_range(name):
                return fn(*a, **kw)
        return inner
    return wrap
