"""Byte-level BPE over the native trainer and encoder (``csrc/data/bpe.cpp``).

The reference's training audit lists a BPE trainer among the CS336 A1 lanes of its data crate
(docs/2026-06-10-cs336-a1-a2-psionic-training-audit.md:209; the homework workload
apps/openagents.com/workers/api/src/cs336-a1-homework-workload.ts:132-169 pins 24 merges over a byte stream).  With
``pieces="none"`` the trainer reproduces that loop exactly (``oracle.cs336.bpe_train``); with ``pieces="gpt2-bytes"`` the
text is first split into word-like pieces so that merges never cross a word boundary.
"""
from __future__ import annotations

import ctypes
import json

import numpy as np

from .. import _native

_MODES = {"none": 0, "gpt2-bytes": 1}
_vp, _u64 = ctypes.c_void_p, ctypes.c_uint64
_SIG = {
    "b200_bpe_split": ([_vp, _u64, ctypes.c_int, _vp, _u64], ctypes.c_int64),
    "b200_bpe_train_text": ([_vp, _u64, ctypes.c_int, ctypes.c_int], _vp), "b200_bpe_train_error": ([_vp], ctypes.c_char_p),
    "b200_bpe_n_merges": ([_vp], ctypes.c_int), "b200_bpe_get_merges": ([_vp, _vp], None), "b200_bpe_train_free": ([_vp], None),
    "b200_bpe_encoder": ([_vp, ctypes.c_int], _vp), "b200_bpe_encode": ([_vp, _vp, _u64, ctypes.c_int, _vp, _u64], ctypes.c_int64),
    "b200_bpe_encoder_free": ([_vp], None),
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


def split_pieces(data: bytes, pieces: str = "gpt2-bytes") -> list[bytes]:
    buf = np.frombuffer(data, dtype=np.uint8)
    ends = np.empty(max(1, len(data)), dtype=np.uint64)
    n = _lib().b200_bpe_split(buf.ctypes.data if len(data) else None, len(data), _MODES[pieces], ends.ctypes.data, ends.size)
    out, at = [], 0
    for e in ends[:n].tolist():
        out.append(data[at:e])
        at = e
    return out


class ByteBpe:
    """Ids 0..255 are bytes, id 256 + k is merge k.  ``special`` tokens get ids after the merges and are matched verbatim."""

    def __init__(self, merges: list[tuple[int, int]], pieces: str = "gpt2-bytes", special: list[str] | None = None):
        self.merges, self.pieces, self.special = [tuple(m) for m in merges], pieces, list(special or [])
        arr = np.asarray(self.merges, dtype=np.int32).reshape(-1, 2)
        self._h = _lib().b200_bpe_encoder(arr.ctypes.data if len(arr) else None, len(arr))
        self._free = _lib().b200_bpe_encoder_free          # bound now: module globals may be gone when __del__ runs at shutdown
        if not self._h:
            raise ValueError("a merge names an id that does not exist yet")
        self.vocab: list[bytes] = [bytes([i]) for i in range(256)]
        for a, b in self.merges:
            self.vocab.append(self.vocab[a] + self.vocab[b])
        self.special_ids = {s: len(self.vocab) + i for i, s in enumerate(self.special)}
        self.vocab_size = len(self.vocab) + len(self.special)

    @classmethod
    def train(cls, data: bytes, n_merges: int, pieces: str = "gpt2-bytes", special: list[str] | None = None) -> "ByteBpe":
        lib = _lib()
        buf = np.frombuffer(data, dtype=np.uint8)
        h = lib.b200_bpe_train_text(buf.ctypes.data if len(data) else None, len(data), n_merges, _MODES[pieces])
        try:
            err = lib.b200_bpe_train_error(h)
            if err:
                raise ValueError(err.decode())
            n = lib.b200_bpe_n_merges(h)
            out = np.empty((n, 2), dtype=np.int32)
            if n:
                lib.b200_bpe_get_merges(h, out.ctypes.data)
        finally:
            lib.b200_bpe_train_free(h)
        return cls([tuple(r) for r in out.tolist()], pieces, special)

    def _encode_plain(self, data: bytes) -> list[int]:
        if not data:
            return []
        buf = np.frombuffer(data, dtype=np.uint8)
        out = np.empty(len(data), dtype=np.int32)                 # never more ids than bytes
        n = _lib().b200_bpe_encode(self._h, buf.ctypes.data, len(data), _MODES[self.pieces], out.ctypes.data, out.size)
        return out[:n].tolist()

    def encode(self, text: str | bytes) -> list[int]:
        data = text.encode("utf-8") if isinstance(text, str) else text
        if not self.special:
            return self._encode_plain(data)
        out, pos = [], 0
        marks = sorted(self.special, key=len, reverse=True)
        while pos < len(data):
            hit, at = None, len(data)
            for s in marks:
                i = data.find(s.encode(), pos)
                if i != -1 and i < at:
                    hit, at = s, i
            out += self._encode_plain(data[pos:at])
            if hit is None:
                break
            out.append(self.special_ids[hit])
            pos = at + len(hit.encode())
        return out

    def decode_bytes(self, ids) -> bytes:
        inv = {v: k.encode() for k, v in self.special_ids.items()}
        return b"".join(self.vocab[i] if i < len(self.vocab) else inv[i] for i in ids)

    def decode(self, ids) -> str:
        return self.decode_bytes(ids).decode("utf-8", errors="replace")

    def to_json(self) -> str:
        return json.dumps({"schema": "b200.byte_bpe.v1", "pieces": self.pieces, "merges": [list(m) for m in self.merges], "special": self.special})

    @classmethod
    def from_json(cls, s: str) -> "ByteBpe":
        o = json.loads(s)
        if o.get("schema") != "b200.byte_bpe.v1":
            raise ValueError("not a byte-BPE file")
        return cls([tuple(m) for m in o["merges"]], o["pieces"], o.get("special"))

    def __del__(self):
        if getattr(self, "_h", None):
            self._free(self._h)
            self._h = None
