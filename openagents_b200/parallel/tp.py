"""Tensor-parallel communicator of the serving engine.

The residual stream is replicated on every rank and lives in the symmetric heap.  A row-parallel
projection (attention output, FFN down) adds its partial result straight into every replica from
inside the kernel that computed it (``multimem.red`` through NVSwitch, or one ``red`` per peer), and
the same kernel ends with the cross-rank barrier: there is no separate all-reduce launch.

Topology naming follows the reference's serving contracts, which list ``tensor_sharded`` among the
typed topologies (docs/teardowns/2026-07-21-buzz-teardown.md:660-681).
"""
from __future__ import annotations

import torch

from ..ops import cuda_ops as ops
from .symm import SymmHeap


class TPComm:
    def __init__(self, rank: int, world: int, device, heap_bytes: int = 1 << 30, multicast: bool | None = None,
                 wait_s: float = 2.0, group=None):
        """``group``: the process group of ONE tensor-parallel replica (default: all ranks); ``rank`` / ``world`` are the
        position and size within it."""
        self.rank, self.world, self.device = rank, world, torch.device(device)
        self.heap = SymmHeap(heap_bytes, device, group=group, wait_s=wait_s, multicast=multicast)
        if (self.heap.rank, self.heap.world) != (rank, world):
            raise ValueError(f"rank {rank}/{world} does not match the group's {self.heap.rank}/{self.heap.world}")
        self._merge = None

    def alloc_tensor(self, shape, dtype):
        return self.heap.alloc_tensor(shape, dtype)

    def offset_of(self, t: torch.Tensor) -> int:
        return t.data_ptr() - self.heap.buf.data_ptr()

    # row-parallel mat-vec with the all-reduce fused into its epilogue
    def matvec_allreduce(self, w, nb, xq, xd, xs, xf, x, ldy, bias=None, wait_ready=False):
        """``wait_ready``: every rank's reader of ``x`` signals when it is done (``ops.rmsnorm(..., signal_sym=)``)
        and this kernel checks the signals before its first remote add, instead of a barrier launch in between."""
        ops.matvec(w.wt, w.main, w.plane2, w.N, w.K, nb, xq=xq, xd=xd, xs16=xs, xf=xf, epi=ops.EPI_ALLREDUCE,
                   bias=bias, y=x, ldy=ldy, sym=self.heap.table, sym_off=self.offset_of(x), wait_ready=wait_ready)

    # row-parallel GEMM with the all-reduce fused into its epilogue
    def gemm_allreduce(self, a_bf16, w_dense, M, x, bias=None, status=None, wait_ready=False):
        N, K = w_dense.shape
        ops.gemm_bf16(a_bf16, w_dense, M, N, K, lda=a_bf16.stride(0), ldb=K, ldc=x.stride(0), bias=bias, status=status,
                      sym_mode=ops.SYM_ALLREDUCE, sym=self.heap.table, sym_off=self.offset_of(x), wait_ready=wait_ready)

    def argmax_merge(self, out_ids: torch.Tensor, out_val: torch.Tensor, nb: int):
        """Global arg-max over vocabulary shards in one kernel: every rank stores its per-row (value, id) into its slot
        on every rank, raises its flag, waits for the others' and picks the best pair (lowest id on ties) from identical
        data."""
        if self._merge is None:
            self._merge_rows = 1024
            self._merge, self._merge_off = self.heap.alloc_tensor((2, self.world, self._merge_rows, 2), torch.float32)
        if nb > self._merge_rows:
            raise ValueError("argmax_merge handles up to 1024 rows")
        ops.argmax_merge(out_ids, out_val, nb, self.heap.table, self._merge_off, self._merge_rows)
