"""An exhaustively checked model of the batch loader's slot ring (``csrc/data/token_data.cpp``).

The loader is a small concurrent protocol: worker threads claim batch numbers in order, each waits until the slot its batch maps
to is FREE and expects exactly that batch, fills it outside the lock and marks it READY; the consumer takes batches strictly in
order, holds a slot while the GPU copy reads it, and releases it, which advances the slot's expected batch by the ring size.  The
thread sanitizer (``tests/test_native_sanitizers.py``) checks the implementation for data races on the runs it happens to see; this
model checks the protocol itself on EVERY interleaving of a bounded configuration with the explicit-state checker of
``control.protocol_specs``:

* safety: the consumer receives batches in order, each exactly once; a slot is never filled while the consumer holds it or
  before it has been taken; two workers never fill the same slot at once;
* liveness (under weak fairness of workers and consumer): every batch is eventually delivered;
* two deliberately broken variants (a worker that ignores which batch the slot expects; a release that does not advance it) must
  produce a counterexample, which shows that the properties can tell a broken ring from a working one.
"""
from __future__ import annotations

from ..control.protocol_specs import Model, check, check_leads_to

FREE, FILLING, READY, HELD = 0, 1, 2, 3


def loader_ring(n_slots: int = 2, n_workers: int = 2, n_batches: int = 5, ignore_expect: bool = False, release_keeps_expect: bool = False) -> Model:
    """State: (next_fill, next_take, slots, workers, delivered).  ``slots[i] = (state, expect, holds)``: ``holds`` is the batch whose
    data sits in the slot (None when empty).  ``workers[w]`` = batch claimed and not yet done (None when idle), plus its phase."""
    init = (0, 0, tuple((FREE, i, None) for i in range(n_slots)), tuple((None, 0) for _ in range(n_workers)), ())

    def claim(w):
        def act(s):
            nf, nt, slots, workers, out = s
            if workers[w][0] is None and nf < n_batches:
                yield (nf + 1, nt, slots, workers[:w] + ((nf, 0),) + workers[w + 1:], out)
        return act

    def begin_fill(w):
        def act(s):
            nf, nt, slots, workers, out = s
            b, phase = workers[w]
            if b is None or phase != 0:
                return
            i = b % n_slots
            st, expect, holds = slots[i]
            if st == FREE and (ignore_expect or expect == b):
                yield (nf, nt, slots[:i] + ((FILLING, expect, b),) + slots[i + 1:], workers[:w] + ((b, 1),) + workers[w + 1:], out)
        return act

    def end_fill(w):
        def act(s):
            nf, nt, slots, workers, out = s
            b, phase = workers[w]
            if b is None or phase != 1:
                return
            i = b % n_slots
            st, expect, holds = slots[i]
            yield (nf, nt, slots[:i] + ((READY, expect, holds),) + slots[i + 1:], workers[:w] + ((None, 0),) + workers[w + 1:], out)
        return act

    def take(s):
        nf, nt, slots, workers, out = s
        if nt >= n_batches:
            return
        i = nt % n_slots
        st, expect, holds = slots[i]
        if st == READY and expect == nt:
            yield (nf, nt + 1, slots[:i] + ((HELD, expect, holds),) + slots[i + 1:], workers, out + (holds,))

    def release(s):
        nf, nt, slots, workers, out = s
        for i, (st, expect, holds) in enumerate(slots):
            if st == HELD:
                yield (nf, nt, slots[:i] + ((FREE, expect if release_keeps_expect else expect + n_slots, None),) + slots[i + 1:], workers, out)

    actions = {"take": take, "release": release}
    for w in range(n_workers):
        actions[f"claim{w}"], actions[f"begin_fill{w}"], actions[f"end_fill{w}"] = claim(w), begin_fill(w), end_fill(w)

    def in_order(s):
        return s[4] == tuple(range(len(s[4])))

    def one_filler_per_slot(s):
        filling = [b % n_slots for b, phase in s[3] if b is not None and phase == 1]
        return len(filling) == len(set(filling))

    def fill_only_free(a, b):        # a slot that turns FILLING was FREE just before: never READY (data not yet taken) or HELD (being read)
        return all(not (tb[0] == FILLING and ta[0] != FILLING) or ta[0] == FREE for ta, tb in zip(a[2], b[2]))

    return Model([init], actions, {"delivered_in_order_exactly_once": in_order, "one_filler_per_slot": one_filler_per_slot}, {"fill_only_free_slots": fill_only_free})


def check_loader_ring(n_slots: int = 2, n_workers: int = 2, n_batches: int = 5) -> dict:
    """Safety and liveness of the ring, and the two mutations that must fail."""
    good = loader_ring(n_slots, n_workers, n_batches)
    fair = list(good.actions)
    out = {"safety": check(good),
           "every_batch_is_delivered": check_leads_to(good, lambda s: True, lambda s: len(s[4]) == n_batches, fair),
           "mutation_worker_ignores_expected_batch": check(loader_ring(n_slots, n_workers, n_batches, ignore_expect=True)),
           "mutation_release_keeps_expected_batch": check_leads_to(loader_ring(n_slots, n_workers, n_batches, release_keeps_expect=True),
                                                                   lambda s: True, lambda s: len(s[4]) == n_batches, fair)}
    return out
