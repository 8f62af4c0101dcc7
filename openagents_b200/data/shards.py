"""Python face of the native token data set and batch loader (``csrc/data/token_data.cpp``).

The reference's training stack keeps its data code in a Rust crate (``psionic-data``: tokenizer, refinery,
trace-to-training conversion; docs/2026-06-10-cs336-a1-a2-psionic-training-audit.md:209,286-289) and feeds fixed-shape
token windows to the trainer.  Here: ``write_token_shard`` writes a shard, ``TokenDataset`` maps shards and serves
windows, ``BatchLoader`` prefetches ``[accum, micro_batch, seq_len]`` batches into pinned memory from worker threads.
The sampler is stateless (batch index -> windows), so a resumed run passes ``start_batch`` and continues the same stream.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import numpy as np
import torch

from .. import _native

_u64, _i64p, _vp, _cp = ctypes.c_uint64, ctypes.POINTER(ctypes.c_int64), ctypes.c_void_p, ctypes.c_char_p
_SIG = {
    "b200_tokds_open": ([ctypes.POINTER(_cp), ctypes.c_int, ctypes.c_int, ctypes.c_int], _vp),
    "b200_tokds_error": ([_vp], _cp), "b200_tokds_windows": ([_vp], _u64), "b200_tokds_tokens": ([_vp], _u64),
    "b200_tokds_close": ([_vp], None), "b200_tokds_read": ([_vp, _u64, _vp, _vp], ctypes.c_int64),
    "b200_tokds_permute": ([_u64, _u64, _u64, _u64], _u64),
    "b200_tok_shard_write": ([_cp, _vp, _u64, ctypes.c_int, _vp], ctypes.c_int),
    "b200_loader_create": ([_vp, ctypes.c_int, ctypes.c_int, ctypes.c_int, _u64, _u64, ctypes.c_int, ctypes.c_int], _vp),
    "b200_loader_error": ([_vp], _cp), "b200_loader_batches_per_epoch": ([_vp], _u64),
    "b200_loader_add_slot": ([_vp, _vp, _vp], ctypes.c_int), "b200_loader_start": ([_vp], ctypes.c_int),
    "b200_loader_next": ([_vp, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(_u64), ctypes.POINTER(ctypes.c_int64), ctypes.c_int], ctypes.c_int),
    "b200_loader_release": ([_vp, ctypes.c_int], ctypes.c_int), "b200_loader_destroy": ([_vp], None),
}
_ready = False


def _lib():
    global _ready
    lib = _native.host()
    if not _ready:
        for name, (args, res) in _SIG.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = args, res
        _ready = True
    return lib


def write_token_shard(path, tokens, mask=None, width: int | None = None) -> dict:
    """``tokens``: 1-D integer array.  ``mask``: optional 0/1 per token (1 = the token is a training target).
    ``width``: bytes per id (default 2 when every id fits, else 4)."""
    t = np.asarray(tokens)
    if t.ndim != 1 or (t.size and t.min() < 0):
        raise ValueError("tokens must be a 1-D array of non-negative ids")
    if width is None:
        width = 2 if (t.size == 0 or int(t.max()) < 65536) else 4
    if width == 2 and t.size and int(t.max()) >= 65536:
        raise ValueError("an id does not fit in 2 bytes")
    buf = np.ascontiguousarray(t.astype(np.uint16 if width == 2 else np.uint32))
    m = None
    if mask is not None:
        m = np.ascontiguousarray(np.asarray(mask).astype(np.uint8))
        if m.shape != t.shape:
            raise ValueError("mask and tokens differ in length")
    rc = _lib().b200_tok_shard_write(str(path).encode(), buf.ctypes.data, buf.size, width, m.ctypes.data if m is not None else None)
    if rc != 0:
        raise OSError(f"writing {path} failed ({rc})")
    return {"path": str(path), "tokens": int(buf.size), "bytesPerToken": width, "masked": mask is not None}


def permute(total: int, seed: int, epoch: int, pos: int) -> int:
    """Position ``pos`` of epoch ``epoch`` -> window index: a bijection of ``range(total)`` for every (seed, epoch)."""
    return int(_lib().b200_tokds_permute(total, seed, epoch, pos))


class TokenDataset:
    def __init__(self, paths, seq_len: int, raw_width: int = 0):
        """``raw_width``: 2 or 4 lets files without the shard header be read as plain dumps of ids of that width."""
        paths = [str(p) for p in ([paths] if isinstance(paths, (str, Path)) else paths)]
        arr = (_cp * len(paths))(*[p.encode() for p in paths])
        self._h = _lib().b200_tokds_open(arr, len(paths), seq_len, raw_width)
        self._free = _lib().b200_tokds_close               # bound now: module globals may be gone when __del__ runs at shutdown
        err = _lib().b200_tokds_error(self._h)
        if err:
            msg = err.decode()
            self.close()
            raise ValueError(msg)
        self.seq_len, self.paths = seq_len, paths
        self.windows, self.tokens = int(_lib().b200_tokds_windows(self._h)), int(_lib().b200_tokds_tokens(self._h))

    def __len__(self):
        return self.windows

    def window(self, i: int):
        """(inputs, targets, unmasked targets) of window ``i``; masked targets are -1."""
        tok, tgt = torch.empty(self.seq_len, dtype=torch.int64), torch.empty(self.seq_len, dtype=torch.int64)
        n = _lib().b200_tokds_read(self._h, i, tok.data_ptr(), tgt.data_ptr())
        if n < 0:
            raise IndexError(i)
        return tok, tgt, int(n)

    def close(self):
        if getattr(self, "_h", None):
            self._free(self._h)
            self._h = None

    def __del__(self):
        self.close()


class BatchLoader:
    """Iterator of ``(tokens, targets, n_valid, batch_index)``; ``tokens`` / ``targets`` are int64
    ``[accum, micro_batch, seq_len]`` views of a slot of the ring (pinned when CUDA is there) and stay valid until the
    next call to ``next``.  Rank ``rank`` of ``world`` gets rows ``rank, rank + world, ...`` of each global batch, so the
    union over ranks of batch ``b`` is the same set of windows whatever the world size's factorisation into ranks x rows."""

    def __init__(self, ds: TokenDataset, accum: int, micro_batch: int, rank: int = 0, world: int = 1, seed: int = 0, start_batch: int = 0,
                 shuffle: bool = True, slots: int = 3, threads: int = 2, pin: bool | None = None, timeout_s: float = 60.0):
        self.ds, self.shape, self.timeout_ms = ds, (accum, micro_batch, ds.seq_len), int(timeout_s * 1000)
        rows = accum * micro_batch
        lib = _lib()
        self._h = lib.b200_loader_create(ds._h, rows, rank, world, seed, start_batch, int(shuffle), threads)
        self._free = lib.b200_loader_destroy
        err = lib.b200_loader_error(self._h)
        if err:
            msg = err.decode()
            self.close()
            raise ValueError(msg)
        pin = torch.cuda.is_available() if pin is None else pin
        self._bufs = []
        for _ in range(max(2, slots)):
            tok = torch.empty(self.shape, dtype=torch.int64, pin_memory=pin)
            tgt = torch.empty(self.shape, dtype=torch.int64, pin_memory=pin)
            lib.b200_loader_add_slot(self._h, tok.data_ptr(), tgt.data_ptr())
            self._bufs.append((tok, tgt))
        self.batches_per_epoch = int(lib.b200_loader_batches_per_epoch(self._h))
        self._held = None
        self.next_batch = start_batch
        lib.b200_loader_start(self._h)

    def next(self):
        lib = _lib()
        if self._held is not None:
            lib.b200_loader_release(self._h, self._held)
            self._held = None
        slot, batch, valid = ctypes.c_int(), _u64(), ctypes.c_int64()
        rc = lib.b200_loader_next(self._h, ctypes.byref(slot), ctypes.byref(batch), ctypes.byref(valid), self.timeout_ms)
        if rc != 0:
            raise TimeoutError("the loader produced no batch in time") if rc == 1 else RuntimeError("loader not started")
        self._held = slot.value
        self.next_batch = batch.value + 1
        tok, tgt = self._bufs[slot.value]
        return tok, tgt, int(valid.value), int(batch.value)

    __next__ = next

    def __iter__(self):
        return self

    def state(self) -> dict:
        """What a checkpoint stores to continue the stream."""
        return {"next_batch": self.next_batch}

    def close(self):
        if getattr(self, "_h", None):
            self._free(self._h)
            self._h = None

    def __del__(self):
        self.close()
