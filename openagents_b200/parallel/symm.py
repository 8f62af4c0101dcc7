"""Symmetric heap: one buffer per rank, mapped into every rank, plus an NVSwitch multicast mapping.

``torch.distributed`` is the plumbing: its symmetric-memory allocator creates the CUDA VMM
allocation, exchanges the handles over the process group and binds the multicast object.  Nothing
here moves data; the kernels in ``csrc/comm`` and the fused kernels do, addressing the heap by byte
offset (the same offset means the same tensor on every rank).

Communication in the reference is HTTPS + JSON (no collective library; the multi-device training
evidence averages uploaded gradients on the operator side:
apps/openagents.com/docs/2026-06-11-cs336-a1-multi-device-real-gradient-evidence.md:66-74).
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from .. import _native

MAX_RANKS = 8
CONTROL_BYTES = 4096


class SymTable(ctypes.Structure):
    _fields_ = [("world", ctypes.c_int), ("rank", ctypes.c_int), ("use_mc", ctypes.c_int),
                ("wait_ns", ctypes.c_ulonglong), ("base", ctypes.c_void_p * MAX_RANKS), ("mc_base", ctypes.c_void_p)]


_sig_ready = False


def _lib():
    global _sig_ready
    L = _native.cuda()
    if not _sig_ready:
        P, sz, i = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
        for name, args in {"b200_sym_barrier": [P, i, P], "b200_sym_all_reduce_f32": [P, sz, sz, i, P],
                           "b200_sym_all_gather": [P, sz, sz, sz, i, P], "b200_sym_reduce_scatter_f32": [P, sz, sz, sz, i, P],
                           "b200_sym_all_to_all": [P, sz, sz, sz, i, P], "b200_sym_wait_unset_flag": [P, i, P]}.items():
            f = getattr(L, name)
            f.argtypes, f.restype = args, ctypes.c_int
        _sig_ready = True
    return L


def _check(rc, what):
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")


class SymmHeap:
    """A symmetric allocation of ``nbytes`` (plus a control block) shared by the ranks of ``group``.

    ``multicast=None`` uses NVSwitch multicast when the allocation supports it; ``False`` forces
    plain peer loads/stores (used by the failure-handling tests, which must not leave a dead rank
    bound to a multicast object).
    """

    def __init__(self, nbytes: int, device, group=None, wait_s: float = 2.0, multicast: bool | None = None):
        self.device = torch.device(device)
        self.group = group if group is not None else (dist.group.WORLD if dist.is_initialized() else None)
        self.world = dist.get_world_size(self.group) if self.group is not None else 1
        self.rank = dist.get_rank(self.group) if self.group is not None else 0
        if self.world > MAX_RANKS:
            raise ValueError(f"at most {MAX_RANKS} ranks")
        total = CONTROL_BYTES + ((nbytes + 255) // 256) * 256
        self.nbytes = total
        self.table = SymTable()
        self.table.world, self.table.rank = self.world, self.rank
        self.table.wait_ns = int(wait_s * 1e9)
        if self.world == 1:
            self.buf = torch.zeros(total, dtype=torch.uint8, device=self.device)
            self.table.base[0] = self.buf.data_ptr()
            self.table.use_mc, self.table.mc_base = 0, None
            self._hdl = None
        else:
            import torch.distributed._symmetric_memory as symm_mem
            self.buf = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
            self._hdl = symm_mem.rendezvous(self.buf, self.group)
            ptrs = list(self._hdl.buffer_ptrs)
            for r in range(self.world):
                self.table.base[r] = ptrs[r]
            mc = int(self._hdl.multicast_ptr or 0)
            want_mc = (multicast is not False) and os.environ.get("B200_SYMM_MULTICAST", "1") != "0"
            self.table.use_mc = 1 if (mc and want_mc) else 0
            self.table.mc_base = mc if self.table.use_mc else None
            self.buf.zero_()
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)
        self._top = CONTROL_BYTES

    @property
    def uses_multicast(self) -> bool:
        return bool(self.table.use_mc)

    def alloc(self, nbytes: int, align: int = 256) -> int:
        """Bump-allocate; every rank must call in the same order so offsets agree."""
        off = (self._top + align - 1) // align * align
        if off + nbytes > self.nbytes:
            raise MemoryError("symmetric heap exhausted")
        self._top = off + nbytes
        return off

    def tensor(self, off: int, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nb = n * torch.empty((), dtype=dtype).element_size()
        return self.buf[off: off + nb].view(dtype).view(*shape)

    def alloc_tensor(self, shape, dtype):
        n = 1
        for s in shape:
            n *= int(s)
        off = self.alloc(n * torch.empty((), dtype=dtype).element_size())
        return self.tensor(off, shape, dtype), off

    def status(self) -> tuple[int, int]:
        """(last error code, number of timed-out waits) from the local control block."""
        ctl = self.buf[:CONTROL_BYTES].view(torch.int32)
        torch.cuda.synchronize(self.device)
        return int(ctl[96].item()), int(ctl[97].item())   # after flag[32], epoch[32], ticket[32]

    def _stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    # ---- stand-alone collectives (kernels in csrc/comm/collectives.cu)
    def barrier(self, ch: int = 1):
        _check(_lib().b200_sym_barrier(ctypes.addressof(self.table), ch, self._stream()), "sym_barrier")

    def all_reduce_f32(self, off: int, n: int, ch: int = 1):
        _check(_lib().b200_sym_all_reduce_f32(ctypes.addressof(self.table), off, n, ch, self._stream()), "sym_all_reduce")

    def all_gather(self, src_off: int, dst_off: int, nbytes: int, ch: int = 1):
        _check(_lib().b200_sym_all_gather(ctypes.addressof(self.table), src_off, dst_off, nbytes, ch, self._stream()), "sym_all_gather")

    def reduce_scatter_f32(self, in_off: int, out_off: int, n: int, ch: int = 1):
        _check(_lib().b200_sym_reduce_scatter_f32(ctypes.addressof(self.table), in_off, out_off, n, ch, self._stream()), "sym_reduce_scatter")

    def all_to_all(self, src_off: int, dst_off: int, nbytes: int, ch: int = 1):
        _check(_lib().b200_sym_all_to_all(ctypes.addressof(self.table), src_off, dst_off, nbytes, ch, self._stream()), "sym_all_to_all")

    def wait_unset_flag(self, ch: int = 15):
        """Launch a kernel that waits on a flag nothing sets; it gives up after the heap's wait
        limit and records a timeout in the control block (see ``status``)."""
        _check(_lib().b200_sym_wait_unset_flag(ctypes.addressof(self.table), ch, self._stream()), "sym_wait_unset_flag")
