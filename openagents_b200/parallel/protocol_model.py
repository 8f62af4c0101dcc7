"""Exhaustive interleaving checks of the cross-GPU flag protocols, on the host.

The kernels in ``csrc/comm`` and the fused kernels synchronise ranks through a few words of peer-visible memory.
No sanitizer can watch those protocols on the GPUs this code runs on, so each of them is restated here as a small
set of per-rank programs of atomic steps over shared state, and EVERY interleaving of 2 to 3 ranks is enumerated
(breadth-first over reachable states).  A model passes when no reachable state violates its safety assertions and
every terminal state is a completed run (no deadlock).  Each model also takes *mutations*, deliberate bugs (drop a
release, reuse a parity too early, wait for too few arrivals), and the tests require that every mutation is caught:
a check that cannot fail proves nothing.

This follows the reference's discipline for its own concurrent protocols: bounded models checked exhaustively, each
with must-fail mutations alongside the must-pass configuration (specs/run-tlc.sh:6-18, 36-60).

Models:

* ``slot_allreduce``   per-row one-shot all-reduce of decode (``rmsnorm_kernel`` mode 2, ``sym_row_signal`` /
                       ``sym_row_wait``): push own partial row into slot (parity, rank) on every rank, release the
                       row's flag everywhere, wait for world x seq arrivals, read all slots.
* ``allgather_counters`` the prefill all-gather consumed tile by tile (``sym_signal_rows`` / ``sym_wait_rows``):
                       monotonic per-owner counters compared with a host-side epoch.
* ``epoch_barrier``    the flag barrier (``sym_barrier_thread``): arrivals accumulate in one word, each rank waits for
                       world x (epoch + 1) and then advances its private epoch.
* ``moe_parity``       the expert-parallel dispatch counters of two parities: layer L claims slots in parity L & 1
                       while parity 1 - (L & 1) is cleared for layer L + 1.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass


@dataclass
class Result:
    ok: bool
    states: int
    violation: str | None = None

    def __bool__(self):
        return self.ok


def explore(init, programs, step, done, max_states: int = 2_000_000) -> Result:
    """Breadth-first search over interleavings.  ``init``: hashable shared state; ``programs``: number of ranks;
    ``step(state, pcs, r)`` returns ``None`` when rank r is blocked, the string of a violated assertion, or
    ``(state', pc')``; ``done(pcs)`` tells whether every rank has finished."""
    start = (init, tuple(0 for _ in range(programs)))
    seen = {start}
    q = deque([start])
    while q:
        state, pcs = q.popleft()
        moved = False
        for r in range(programs):
            out = step(state, pcs, r)
            if out is None:
                continue
            if isinstance(out, str):
                return Result(False, len(seen), out)
            moved = True
            nstate, npc = out
            nxt = (nstate, pcs[:r] + (npc,) + pcs[r + 1:])
            if nxt not in seen:
                if len(seen) >= max_states:
                    return Result(False, len(seen), "state space exceeds the bound")
                seen.add(nxt)
                q.append(nxt)
        if not moved and not done(pcs):
            return Result(False, len(seen), f"deadlock at pcs {pcs}")
    return Result(True, len(seen))


# ---------------------------------------------------------------------------------------------------- slot all-reduce
def slot_allreduce(world: int = 2, rounds: int = 3, mutation: str | None = None) -> Result:
    """One row.  Shared state: slots[rank_of_memory][parity][writer] = round number written there (0 = never),
    flag[rank_of_memory] = arrivals.  Per round k (1-based) rank r executes:
        push   : for every destination d: slots[d][k & 1][r] = k       (one atomic step per destination)
        signal : for every destination d: flag[d] += 1                 (release: ordered after the pushes)
        wait   : until flag[r] >= world * k
        read   : every slots[r][k & 1][w] must equal k  (a stale or overwritten slot is a violation)
    Mutations: ``single_buffer`` (parity always 0), ``signal_before_push`` (the release is dropped: the flag may pass the
    data), ``wait_for_one`` (target k instead of world * k)."""
    W = world
    n_push, n_sig = W, W
    per_round = n_push + n_sig + 2

    def parity(k):
        return 0 if mutation == "single_buffer" else k & 1

    slots0 = tuple(tuple(tuple(0 for _ in range(W)) for _ in range(2)) for _ in range(W))
    init = (slots0, tuple(0 for _ in range(W)))

    def step(state, pcs, r):
        slots, flag = state
        pc = pcs[r]
        if pc >= rounds * per_round:
            return None
        k, ph = pc // per_round + 1, pc % per_round
        order = list(range(n_push + n_sig))
        if mutation == "signal_before_push":          # signals are not ordered after the pushes
            order = list(range(n_push, n_push + n_sig)) + list(range(n_push))
        if ph < n_push + n_sig:
            op = order[ph]
            if op < n_push:
                d = op
                s = [list(map(list, x)) for x in slots]
                s[d][parity(k)][r] = k
                slots = tuple(tuple(tuple(y) for y in x) for x in s)
            else:
                d = op - n_push
                f = list(flag)
                f[d] += 1
                flag = tuple(f)
            return (slots, flag), pc + 1
        if ph == n_push + n_sig:                      # wait
            target = k if mutation == "wait_for_one" else W * k
            if flag[r] < target:
                return None
            return state, pc + 1
        for w in range(W):                            # read
            if slots[r][parity(k)][w] != k:
                return f"rank {r} round {k}: slot of writer {w} holds round {slots[r][parity(k)][w]}"
        return state, pc + 1

    return explore(init, W, step, lambda pcs: all(p >= rounds * per_round for p in pcs))


# ---------------------------------------------------------------------------------------------------- all-gather counters
def allgather_counters(world: int = 2, rounds: int = 2, mutation: str | None = None) -> Result:
    """Rank r owns row block r of a tensor replicated on every rank.  Per all-gather e (1-based) rank r: writes its block
    into every rank's copy (value e), then bumps counter[d][r] on every rank d; the consumer on rank r waits, for each
    owner o, until counter[r][o] >= e and then reads block o, which must hold e.  Between the consumer and the next
    all-gather's push sits a kernel that ends with the cross-rank barrier (the reduce-scatter GEMM): it is what keeps a
    fast rank from overwriting a block a slow rank has not read yet.  Mutations: ``no_wait`` (the consumer reads without
    waiting), ``counter_first`` (the counter is bumped before the data is written), ``no_barrier`` (the kernel in
    between does not synchronise the ranks)."""
    W = world
    per_round = 2 * W + 2 * W + 1      # W pushes, W bumps, for each owner: wait, read; then the barrier
    data0 = tuple(tuple(0 for _ in range(W)) for _ in range(W))       # data[rank_of_memory][owner]
    init = (data0, data0, tuple(0 for _ in range(W)))

    def step(state, pcs, r):
        data, ctr, bar = state
        pc = pcs[r]
        if pc >= rounds * per_round:
            return None
        e, ph = pc // per_round + 1, pc % per_round
        if ph < 2 * W:
            op = ph
            if mutation == "counter_first":
                op = ph + W if ph < W else ph - W
            d = op % W
            if op < W:
                x = [list(t) for t in data]
                x[d][r] = e
                data = tuple(tuple(t) for t in x)
            else:
                x = [list(t) for t in ctr]
                x[d][r] += 1
                ctr = tuple(tuple(t) for t in x)
            return (data, ctr, bar), pc + 1
        if ph < 4 * W:
            o, what = (ph - 2 * W) // 2, (ph - 2 * W) % 2
            if what == 0:
                if mutation != "no_wait" and ctr[r][o] < e:
                    return None
                return state, pc + 1
            if data[r][o] != e:
                return f"rank {r} all-gather {e}: block of owner {o} holds {data[r][o]}"
            return state, pc + 1
        if mutation == "no_barrier":
            return state, pc + 1
        b = list(bar)                                 # arrive, then wait for everyone's arrival of this round
        if b[r] == e - 1:
            b[r] += 1
            return (data, ctr, tuple(b)), pc
        if any(x < e for x in bar):
            return None
        return state, pc + 1

    return explore(init, W, step, lambda pcs: all(p >= rounds * per_round for p in pcs))


# ---------------------------------------------------------------------------------------------------- epoch barrier
def epoch_barrier(world: int = 2, rounds: int = 3, mutation: str | None = None) -> Result:
    """Per barrier b (0-based) rank r: arrive (flag[d] += 1 for every rank d), wait until flag[r] >= world * (b + 1), then
    check that every rank has at least STARTED barrier b (nobody is still before its arrival).  Mutations:
    ``stale_epoch`` (the private epoch is not advanced, so the second barrier falls through), ``arrive_self_only`` (the
    arrival is not sent to the peers: deadlock)."""
    W = world
    per_round = W + 2
    init = (tuple(0 for _ in range(W)),)

    def step(state, pcs, r):
        (flag,) = state
        pc = pcs[r]
        if pc >= rounds * per_round:
            return None
        b, ph = pc // per_round, pc % per_round
        if ph < W:
            d = ph
            if mutation == "arrive_self_only" and d != r:
                return state, pc + 1
            f = list(flag)
            f[d] += 1
            return (tuple(f),), pc + 1
        if ph == W:
            epoch = 0 if mutation == "stale_epoch" else b
            if flag[r] < W * (epoch + 1):
                return None
            return state, pc + 1
        for o in range(W):          # everyone has arrived at barrier b: its first arrival step is behind it
            if pcs[o] < b * per_round + 1 and o != r:
                return f"rank {r} left barrier {b} before rank {o} reached it"
        return state, pc + 1

    return explore(init, W, step, lambda pcs: all(p >= rounds * per_round for p in pcs))


# ---------------------------------------------------------------------------------------------------- MoE parity counters
def moe_parity(world: int = 2, layers: int = 3, mutation: str | None = None) -> Result:
    """Per layer L rank r: claim a slot on every rank's counter of parity L & 1 (count[d][p] += 1), barrier (all claims of
    the layer are in), clear its counter of the OTHER parity for the next layer (the engine does this while the grouped
    GEMMs of layer L are still to read the counts), read its own counter of parity p (must equal world), barrier (the
    layer's closing barrier: peers start layer L + 1 only after it).  Mutations: ``one_parity`` (a single counter: the
    clear for the next layer wipes the counts the GEMMs are about to read), ``no_closing_barrier`` (layer L + 1 claims may
    land before the clear)."""
    W = world
    per_layer = W + 1 + 1 + 1 + 1     # claims, barrier A, read, clear, barrier B
    init = (tuple((0, 0) for _ in range(W)), tuple(0 for _ in range(W)), tuple(0 for _ in range(W)))

    def step(state, pcs, r):
        count, bar_a, bar_b = state
        pc = pcs[r]
        if pc >= layers * per_layer:
            return None
        L, ph = pc // per_layer, pc % per_layer
        p = 0 if mutation == "one_parity" else L & 1
        if ph < W:
            d = ph
            c = [list(x) for x in count]
            c[d][p] += 1
            return (tuple(tuple(x) for x in c), bar_a, bar_b), pc + 1
        if ph == W:                                   # barrier A: arrive then wait, folded into two visits
            a = list(bar_a)
            if a[r] == 2 * L:                         # not yet arrived at this layer's barrier A
                a[r] += 1
                return (count, tuple(a), bar_b), pc
            if any(x < 2 * L + 1 for x in bar_a):
                return None
            a[r] += 1
            return (count, tuple(a), bar_b), pc + 1
        if ph == W + 1:
            c = [list(x) for x in count]
            c[r][p if mutation == "one_parity" else 1 - p] = 0
            return (tuple(tuple(x) for x in c), bar_a, bar_b), pc + 1
        if ph == W + 2:
            if count[r][p] != W:
                return f"rank {r} layer {L}: counter of parity {p} reads {count[r][p]}, expected {W}"
            return state, pc + 1
        if mutation == "no_closing_barrier":
            return state, pc + 1
        b = list(bar_b)
        if b[r] == 2 * L:
            b[r] += 1
            return (count, bar_a, tuple(b)), pc
        if any(x < 2 * L + 1 for x in bar_b):
            return None
        b[r] += 1
        return (count, bar_a, tuple(b)), pc + 1

    return explore(init, W, step, lambda pcs: all(p >= layers * per_layer for p in pcs))


MODELS = {
    "slot_allreduce": (slot_allreduce, ("single_buffer", "signal_before_push", "wait_for_one")),
    "allgather_counters": (allgather_counters, ("no_wait", "counter_first", "no_barrier")),
    "epoch_barrier": (epoch_barrier, ("stale_epoch", "arrive_self_only")),
    "moe_parity": (moe_parity, ("one_parity", "no_closing_barrier")),
}


def run_all(world: int = 2) -> dict:
    """Every model unmutated (must pass) and with each mutation (must fail)."""
    out = {}
    for name, (fn, muts) in MODELS.items():
        base = fn(world=world)
        out[name] = {"pass": bool(base), "states": base.states, "violation": base.violation,
                     "mutations": {m: (lambda r: {"caught": not r.ok, "violation": r.violation})(fn(world=world, mutation=m)) for m in muts}}
    return out


if __name__ == "__main__":
    import json
    print(json.dumps(run_all(), indent=1))
