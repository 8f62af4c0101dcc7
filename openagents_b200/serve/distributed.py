"""Serving on several GPUs of one node: rank 0 runs the HTTP server and the scheduler, the other ranks follow.

Tensor- and expert-parallel engines need every rank to make the SAME engine calls in the same order (their kernels
meet in collectives, and every rank keeps its own copy of the page allocator, which stays identical because it sees
identical calls).  ``LeaderBackend`` wraps rank 0's backend and announces each call (``begin`` / ``step`` /
``forward`` / ``publish`` / ``end``) to the followers before making it; ``follower_loop`` receives the
announcements and replays them on its own backend.  Announcements travel over a ``gloo`` process group (host
memory, a few hundred bytes per decode step); the data path between the GPUs is the engine's own kernels.

The reference's server takes ``--backend`` and a mesh-coordination flag
(apps/pylon/docs/2026-06-09-pylon-qwen35-local-inference-roadmap.md:137-160) and names the sharded topologies
``tensor_sharded`` and ``sparse_expert`` (docs/teardowns/2026-07-21-buzz-teardown.md:660-681).
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from .backend import Backend


def _announce(group, msg):
    box = [msg]
    dist.broadcast_object_list(box, src=0, group=group)
    return box[0]


class LeaderBackend(Backend):
    """Rank 0's face of a multi-rank engine: same interface, every call mirrored on the followers."""

    def __init__(self, inner: Backend, group):
        self.inner, self.group, self.cfg = inner, group, inner.cfg
        self.name = inner.name

    def _call(self, op: str, *args):
        _announce(self.group, (op, args))
        return getattr(self.inner, op)(*args)

    def begin(self, seq_id, prompt):
        return self._call("begin", seq_id, list(prompt))

    def forward(self, seq_ids, new_tokens):
        return self._call("forward", list(seq_ids), [list(t) for t in new_tokens])

    def step(self, seq_ids, new_tokens, params, uniforms):
        out = self._call("step", list(seq_ids), [list(t) for t in new_tokens], list(params), list(uniforms))
        self.last_d2h_bytes = getattr(self.inner, "last_d2h_bytes", 0)
        return out

    def publish(self, seq_id, tokens):
        return self._call("publish", seq_id, list(tokens))

    def end(self, seq_id):
        return self._call("end", seq_id)

    @property
    def supports_verify(self):
        return self.inner.supports_verify

    def verify(self, seq_id, tokens):
        return self._call("verify", seq_id, list(tokens))

    def truncate(self, seq_id, new_len):
        return self._call("truncate", seq_id, new_len)

    @property
    def supports_score(self):
        return self.inner.supports_score

    def score(self, seq_id, tokens, targets):
        return self._call("score", seq_id, list(tokens), list(targets))

    def seq_len(self, seq_id):
        return self.inner.seq_len(seq_id)          # host-side bookkeeping, identical on every rank

    def shutdown(self):
        _announce(self.group, ("stop", ()))

    @property
    def max_context(self):
        return self.inner.max_context

    def kv_stats(self):
        return self.inner.kv_stats()

    def topology(self):
        return self.inner.topology()


def follower_loop(backend: Backend, group) -> int:
    """Replay rank 0's calls until it says stop.  An exception raised by a call is swallowed here exactly when rank 0's
    identical call raised too (same inputs, same allocator state); the leader reports it to the client."""
    n = 0
    while True:
        op, args = _announce(group, None)
        if op == "stop":
            return n
        try:
            getattr(backend, op)(*args)
        except Exception:      # noqa: BLE001 - mirrored failure (out of pages, context limit): rank 0 handles it
            pass
        n += 1


def _rank_main(rank: int, world: int, args, port: int):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    control = dist.new_group(backend="gloo")
    from ..parallel.tp import TPComm
    comm = TPComm(rank, world, dev, heap_bytes=int(os.environ.get("B200_SERVE_HEAP_MB", "1024")) << 20)
    par = dict(device=dev, comm=comm, control_group=control)
    par.update(dict(tp_rank=rank, tp_world=world) if args.tp > 1 else dict(ep_rank=rank, ep_world=world))
    try:
        if rank == 0:
            from .server import run_server
            try:
                run_server(args, **par)
            finally:
                _announce(control, ("stop", ()))
        else:
            from .backend import CudaBackend
            for p in args.model:
                b = CudaBackend.from_gguf(p, device=dev, max_num_seqs=args.max_num_seqs, max_ctx=args.max_ctx, comm=comm,
                                          **{k: v for k, v in par.items() if k.endswith(("rank", "world"))})
            follower_loop(b, control)
    finally:
        dist.destroy_process_group()


def launch_ranks(args):
    """One process per GPU (``--tp N`` or ``--ep N``); returns when rank 0's server stops."""
    import socket
    import torch.multiprocessing as mp
    world = max(args.tp, args.ep)
    if len(args.model) != 1:
        raise SystemExit("--tp / --ep serve one model")
    if torch.cuda.device_count() < world:
        raise SystemExit(f"--tp/--ep {world} needs {world} GPUs, found {torch.cuda.device_count()}")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_rank_main, args=(world, args, port), nprocs=world, join=True)
