"""Bounded, exhaustively checked models of the three control-plane protocols, with must-fail mutations.

The reference keeps TLA+ specifications of its fleet-delegation supervisor, its approval protocol and its
session/thread mapping, and a runner that requires four configurations to pass and four deliberately broken
variants to produce a counterexample (specs/run-tlc.sh:6-18, 36-60; specs/khala-fleet-delegate/
FleetDelegateSupervisor.tla; specs/approval-protocol/ApprovalProtocol.tla; specs/session-thread-mapping/
SessionThreadMapping.tla; specs/mutations/*).  ``tlc`` is a Java tool; this module gives the same guarantees with
a small explicit-state checker:

* a model is a set of named guarded actions over an immutable state (``Model``);
* ``check`` enumerates every reachable state breadth-first and evaluates state invariants on each state and action
  properties on each transition;
* ``check_leads_to`` verifies ``[](P => <>Q)`` under weak fairness of a chosen set of actions: it searches the part of
  the graph where Q does not hold for a strongly connected component (a single state with the implicit stuttering
  step counts) that a fair behaviour could stay in forever, i.e. one in which every fair action is either disabled
  somewhere or taken inside the component.

``run_all`` runs the four passing configurations and the four mutations with the constants of the reference's
``.cfg`` files and reports each outcome; ``tests/test_protocol_specs.py`` requires pass / violation respectively.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Hashable, Iterable


@dataclass
class Model:
    """``actions``: name -> function(state) yielding successor states (an empty iteration = disabled)."""
    init: list
    actions: dict[str, Callable[[Hashable], Iterable[Hashable]]]
    invariants: dict[str, Callable[[Hashable], bool]] = field(default_factory=dict)
    action_props: dict[str, Callable[[Hashable, Hashable], bool]] = field(default_factory=dict)


@dataclass
class Outcome:
    ok: bool
    states: int
    violated: str | None = None
    trace: list | None = None

    def __bool__(self):
        return self.ok


def _graph(m: Model, max_states: int):
    """Reachable states with their labelled edges and BFS parents.  Raises if the bound is exceeded."""
    parent: dict = {}
    edges: dict = {}
    q = deque()
    for s in m.init:
        if s not in parent:
            parent[s] = None
            q.append(s)
    while q:
        s = q.popleft()
        out = []
        for name, act in m.actions.items():
            for t in act(s):
                out.append((name, t))
                if t not in parent:
                    if len(parent) >= max_states:
                        raise RuntimeError("state space exceeds the bound")
                    parent[t] = (s, name)
                    q.append(t)
        edges[s] = out
    return parent, edges


def _trace(parent, s):
    path = []
    while s is not None:
        p = parent[s]
        path.append((p[1] if p else "init", s))
        s = p[0] if p else None
    return path[::-1]


def check(m: Model, max_states: int = 500_000) -> Outcome:
    """Safety: every invariant on every reachable state, every action property on every reachable transition."""
    parent, edges = _graph(m, max_states)
    for s in parent:
        for name, inv in m.invariants.items():
            if not inv(s):
                return Outcome(False, len(parent), f"invariant {name}", _trace(parent, s))
    for s, out in edges.items():
        for _, t in out:
            for name, prop in m.action_props.items():
                if not prop(s, t):
                    return Outcome(False, len(parent), f"action property {name}", _trace(parent, s) + [("step", t)])
    return Outcome(True, len(parent))


def check_leads_to(m: Model, p: Callable, q: Callable, fair: list[str], max_states: int = 500_000) -> Outcome:
    """Liveness ``[](p => <>q)`` under weak fairness of the actions named in ``fair`` (stuttering allowed otherwise)."""
    parent, edges = _graph(m, max_states)
    # states from which a not-q run can start: reachable inside the not-q subgraph from a state with p and not q
    start = [s for s in parent if p(s) and not q(s)]
    region = set(start)
    dq = deque(start)
    while dq:
        s = dq.popleft()
        for _, t in edges[s]:
            if not q(t) and t not in region:
                region.add(t)
                dq.append(t)
    # Tarjan over the region
    index, low, on, stack, comps = {}, {}, set(), [], []
    counter = [0]
    for root in region:
        if root in index:
            continue
        work = [(root, iter([t for _, t in edges[root] if t in region]))]
        index[root] = low[root] = counter[0]
        counter[0] += 1
        stack.append(root)
        on.add(root)
        while work:
            v, it = work[-1]
            advanced = False
            for w in it:
                if w not in index:
                    index[w] = low[w] = counter[0]
                    counter[0] += 1
                    stack.append(w)
                    on.add(w)
                    work.append((w, iter([t for _, t in edges[w] if t in region])))
                    advanced = True
                    break
                if w in on:
                    low[v] = min(low[v], index[w])
            if advanced:
                continue
            work.pop()
            if work:
                u = work[-1][0]
                low[u] = min(low[u], low[v])
            if low[v] == index[v]:
                comp = set()
                while True:
                    w = stack.pop()
                    on.discard(w)
                    comp.add(w)
                    if w == v:
                        break
                comps.append(comp)
    for comp in comps:
        # a behaviour may stay in `comp` forever (moving along its internal edges or stuttering); it is fair iff every
        # fair action is disabled in some state of comp or is taken on an edge inside comp
        fair_ok = True
        for a in fair:
            disabled_somewhere = any(not any(n == a for n, _ in edges[s]) for s in comp)
            taken_inside = any(n == a and t in comp for s in comp for n, t in edges[s])
            if not (disabled_somewhere or taken_inside):
                fair_ok = False
                break
        if fair_ok:
            s = next(iter(comp))
            return Outcome(False, len(parent), "temporal property (a fair behaviour never reaches the goal)", _trace(parent, s))
    return Outcome(True, len(parent))


# ------------------------------------------------------------------------------------------------ approval protocol
def approval_protocol(requests=("r1", "r2"), mutation: str | None = None) -> Model:
    """A harness asks for approval of tool calls; a turn interrupt or a superseding request advances the turn epoch,
    and an approve may only be applied to a request issued in the current epoch
    (specs/approval-protocol/ApprovalProtocol.tla:27-32; mutation ``stale_forgery`` drops that guard,
    specs/mutations/approval-stale-forgery/ApprovalStaleForgery.tla:27-30).
    State: (status per request, response per request, epoch, epoch recorded per request)."""
    n = len(requests)
    init = (("never",) * n, ("none",) * n, 0, (0,) * n)

    def put(t, i, v):
        return t[:i] + (v,) + t[i + 1:]

    def issue(s):
        st, rs, ep, re = s
        for i in range(n):
            if st[i] == "never":
                yield (put(st, i, "requested"), rs, ep, put(re, i, ep))

    def approve(s):
        st, rs, ep, re = s
        for i in range(n):
            if st[i] == "requested" and (mutation == "stale_forgery" or re[i] == ep):
                yield (put(st, i, "approved"), put(rs, i, "approve"), ep, re)

    def reject(s):
        st, rs, ep, re = s
        for i in range(n):
            if st[i] == "requested" and re[i] == ep:
                yield (put(st, i, "rejected"), put(rs, i, "reject"), ep, re)

    def closer(status, resp):
        def act(s):
            st, rs, ep, re = s
            for i in range(n):
                if st[i] == "requested":
                    yield (put(st, i, status), put(rs, i, resp), ep + 1, re)
        return act

    closed = ("approved", "rejected", "interrupted", "superseded")
    return Model(
        init=[init],
        actions={"issue": issue, "approve": approve, "reject": reject, "interrupt": closer("interrupted", "interrupt"),
                 "supersede": closer("superseded", "supersede")},
        invariants={
            "NoLostApprovals": lambda s: all(st in ("requested", "never") or r != "none" for st, r in zip(s[0], s[1])),
            "NoDuplicateApprovalResponses": lambda s: all(r == "none" or st in closed for st, r in zip(s[0], s[1])),
        },
        action_props={
            # an approve is only ever applied to a request whose recorded epoch is the current one
            "NoStaleApproveApplication": lambda s, t: all(not (s[1][i] != "approve" and t[1][i] == "approve") or s[3][i] == s[2]
                                                          for i in range(n)),
        })


def approval_liveness(requests=("r1", "r2")) -> Outcome:
    """Every issued request eventually closes, given that closing actions are not postponed forever."""
    m = approval_protocol(requests)
    # the four closing actions are one fair disjunction in the specification: model them as one action
    closing = [m.actions[k] for k in ("approve", "reject", "interrupt", "supersede")]
    m.actions = {"issue": m.actions["issue"], "close": lambda s: (t for a in closing for t in a(s))}
    worst = Outcome(True, 0)
    for i in range(len(requests)):
        o = check_leads_to(m, lambda s, i=i: s[0][i] == "requested", lambda s, i=i: s[0][i] != "requested", ["issue", "close"])
        if not o:
            return o
        worst = o
    return worst


# ------------------------------------------------------------------------------------------- session / thread mapping
def session_thread_mapping(sessions=("s1", "s2"), threads=("t1", "t2"), mutation: str | None = None) -> Model:
    """A desktop session is bound to at most one agent thread and back; bindings are persisted after the fact, and a
    crash followed by a reload must rebuild BOTH directions from what was persisted
    (specs/session-thread-mapping/SessionThreadMapping.tla:24-75).  Mutation ``reload_drops_reverse``: the reload
    restores only session -> thread (specs/mutations/session-crash-divergence/SessionCrashDivergence.tla:38-48).
    State: (thread of each session, session of each thread, persisted pairs, pending pairs, crashed)."""
    ns, nt = len(sessions), len(threads)
    init = ((None,) * ns, (None,) * nt, frozenset(), frozenset(), False)

    def put(t, i, v):
        return t[:i] + (v,) + t[i + 1:]

    def bind(s):
        st, ts, per, pend, crashed = s
        if crashed:
            return
        for a in range(ns):
            for b in range(nt):
                if st[a] is None and ts[b] is None:
                    if mutation == "reload_drops_reverse":     # the mutated model persists at once, as its source does
                        yield (put(st, a, b), put(ts, b, a), per | {(a, b)}, pend, False)
                    else:
                        yield (put(st, a, b), put(ts, b, a), per, pend | {(a, b)}, False)

    def persist(s):
        st, ts, per, pend, crashed = s
        if crashed:
            return
        for (a, b) in pend:
            if st[a] == b and ts[b] == a:
                yield (st, ts, per | {(a, b)}, pend - {(a, b)}, False)

    def archive(s):
        st, ts, per, pend, crashed = s
        if crashed or mutation == "reload_drops_reverse":
            return
        for a in range(ns):
            if st[a] is not None:
                b = st[a]
                yield (put(st, a, None), put(ts, b, None), per - {(a, b)}, pend - {(a, b)}, False)

    def crash(s):
        if not s[4]:
            yield s[:4] + (True,)

    def reload(s):
        st, ts, per, pend, crashed = s
        if not crashed:
            return
        by_s, by_t = {}, {}
        for (a, b) in per:
            by_s.setdefault(a, []).append(b)
            by_t.setdefault(b, []).append(a)
        if any(len(v) > 1 for v in by_s.values()) or any(len(v) > 1 for v in by_t.values()):
            return
        nst = tuple(by_s[a][0] if a in by_s else None for a in range(ns))
        nts = ((None,) * nt if mutation == "reload_drops_reverse" else tuple(by_t[b][0] if b in by_t else None for b in range(nt)))
        yield (nst, nts, per, frozenset(), False)

    def no_orphan(s):
        st, ts = s[0], s[1]
        return (all(st[a] is None or ts[st[a]] == a for a in range(ns)) and
                all(ts[b] is None or st[ts[b]] == b for b in range(nt)))

    def no_double(s):
        st, ts = s[0], s[1]
        live_t = [x for x in st if x is not None]
        live_s = [x for x in ts if x is not None]
        return len(live_t) == len(set(live_t)) and len(live_s) == len(set(live_s))

    def persisted_consistent(s):
        st, ts, per = s[0], s[1], s[2]
        if s[4]:                                   # between crash and reload the in-memory maps are not consulted
            return True
        ok = all(st[a] == b and ts[b] == a for (a, b) in per)
        return ok and len({a for a, _ in per}) == len(per) and len({b for _, b in per}) == len(per)

    return Model(init=[init], actions={"bind": bind, "persist": persist, "archive": archive, "crash": crash, "reload": reload},
                 invariants={"NoOrphanThreadBinding": no_orphan, "NoDoubleBind": no_double,
                             "PersistedMappingConsistent": persisted_consistent})


# ---------------------------------------------------------------------------------------- fleet delegation supervisor
def fleet_delegate(supervisors=("s1", "s2"), work=("w1", "w2"), capacity: int = 1, claim_ttl: int = 2, max_releases: int = 1,
                   mutation: str | None = None) -> Model:
    """Racing supervisors claim work units of a fleet run under one supervisor lease; claims expire or are released a
    bounded number of times; an operator can pause, resume and drain; a reconciler closes a run and may revive a closed
    run for new backlog, but never one the OPERATOR closed (specs/khala-fleet-delegate/FleetDelegateSupervisor.tla:
    52-57, 79-90, 172-190).  Mutations: ``paused_claim`` (a claim is accepted while the run is paused,
    specs/mutations/fleet-paused-claim/FleetPausedClaim.tla:26-33), ``operator_revive`` (the revive guard ignores who
    closed the run, specs/mutations/fleet-operator-revive/FleetOperatorRevive.tla:55-59).
    State: (run state, who set it, claim state per unit, holder per unit, ttl per unit, releases per unit, active set,
    terminal set, lease holder, paused-claim seen, operator-closed run revived, operator intervened)."""
    nw = len(work)
    live = ("claimed", "in_progress", "closeout")
    init = ("running", "none", ("none",) * nw, (None,) * nw, (0,) * nw, (0,) * nw, frozenset(), frozenset(), None, False, False, False)

    def put(t, i, v):
        return t[:i] + (v,) + t[i + 1:]

    def claimable(s):
        claims, rel, terminal = s[2], s[5], s[7]
        return [w for w in range(nw) if claims[w] not in live and w not in terminal and rel[w] <= max_releases]

    def open_claims(s):
        return [w for w in range(nw) if s[2][w] in ("claimed", "in_progress")]

    def acquire(s):
        if s[0] == "running" and s[8] is None:
            for sup in supervisors:
                yield s[:8] + (sup,) + s[9:]

    def release_sup(s):
        if s[8] is not None and s[0] in ("completed", "stopped"):
            yield s[:8] + (None,) + s[9:]

    def try_claim(s):
        run, src, claims, holders, ttl, rel, active, terminal, lease, forged, revived, interv = s
        if lease is None:
            return
        allowed = run == "running" or (mutation == "paused_claim" and run == "paused")
        if not allowed or len(open_claims(s)) >= capacity:
            return
        for w in claimable(s):
            yield (run, src, put(claims, w, "claimed"), put(holders, w, lease), put(ttl, w, claim_ttl), rel, active, terminal, lease,
                   forged or run == "paused", revived, interv)

    def dispatch(s):
        run, claims, active = s[0], s[2], s[6]
        if run != "running":
            return
        for w in range(nw):
            if claims[w] == "claimed" and w not in active:
                yield s[:2] + (put(claims, w, "in_progress"),) + s[3:6] + (active | {w},) + s[7:]

    def complete(s):
        claims, ttl, active, terminal = s[2], s[4], s[6], s[7]
        for w in active:
            yield s[:2] + (put(claims, w, "closeout"), s[3], put(ttl, w, 0), s[5], active - {w}, terminal | {w}) + s[8:]

    def release_claim(s):
        claims, holders, ttl, rel, active = s[2], s[3], s[4], s[5], s[6]
        for w in open_claims(s):
            if rel[w] < max_releases:
                yield s[:2] + (put(claims, w, "released"), put(holders, w, None), put(ttl, w, 0), put(rel, w, rel[w] + 1), active - {w}) + s[7:]

    def expire(s):
        claims, holders, ttl, rel, active = s[2], s[3], s[4], s[5], s[6]
        for w in open_claims(s):
            if ttl[w] == 0:
                yield s[:2] + (put(claims, w, "expired"), put(holders, w, None), ttl, put(rel, w, rel[w] + 1), active - {w}) + s[7:]

    def tick(s):
        ttl = s[4]
        if any(x > 0 for x in ttl):
            yield s[:4] + (tuple(x - 1 if x > 0 else x for x in ttl),) + s[5:]

    def operator(frm, to):
        def act(s):
            if s[0] in frm:
                yield (to, "operator") + s[2:11] + (True,)
        return act

    def reconcile_close(s):
        run, active, terminal = s[0], s[6], s[7]
        if run in ("running", "draining") and not claimable(s) and not active:
            yield ("completed" if len(terminal) == nw else "stopped", "operator" if run == "draining" else "reconcile") + s[2:]

    def drain_complete(s):
        if s[0] == "draining" and not s[6]:
            yield ("stopped", "operator") + s[2:11] + (True,)

    def revive(s):
        run, src = s[0], s[1]
        auto = run in ("completed", "stopped") and (mutation == "operator_revive" or src != "operator")
        if auto and claimable(s):
            yield ("running", "reconcile") + s[2:10] + (s[10] or src == "operator", s[11])

    return Model(
        init=[init],
        actions={"acquire_supervisor": acquire, "release_supervisor": release_sup, "try_claim": try_claim, "dispatch": dispatch,
                 "complete": complete, "release_claim": release_claim, "expire_claim": expire, "tick": tick,
                 "pause": operator(("running",), "paused"), "resume": operator(("paused",), "running"),
                 "drain": operator(("running", "paused"), "draining"), "reconcile_close": reconcile_close,
                 "drain_complete": drain_complete, "revive": revive},
        invariants={
            "ActiveAssignmentsNeverExceedAdvertisedCapacity": lambda s: len(s[6]) <= capacity,
            "ClaimUniquenessUnderRacingSupervisors": lambda s: all(s[2][w] not in live or s[3][w] in supervisors for w in range(nw)),
            "PausedRunsClaimNothing": lambda s: not s[9],
            "SupervisorReviveHonorsAutoRevivableGuard": lambda s: not s[10],
        })


_FLEET_FAIR = ["acquire_supervisor", "try_claim", "dispatch", "complete", "expire_claim", "tick", "reconcile_close", "drain_complete",
               "revive", "release_supervisor"]


def fleet_liveness() -> Outcome:
    """With one supervisor, one unit, a ttl of one and no releases: unless an operator steps in, the run ends closed with
    nothing active or open; and a draining run always ends (FleetDelegateSupervisorLiveness.cfg)."""
    m = fleet_delegate(("s1",), ("w1",), capacity=1, claim_ttl=1, max_releases=0)

    def settled(s):
        return s[11] or (s[0] in ("completed", "stopped") and not s[6] and not any(c in ("claimed", "in_progress") for c in s[2]))

    o = check_leads_to(m, lambda s: True, settled, _FLEET_FAIR)
    if not o:
        return o
    return check_leads_to(m, lambda s: s[0] == "draining", lambda s: s[0] in ("completed", "stopped"), _FLEET_FAIR)


def run_all() -> dict[str, Outcome]:
    """The four configurations that must pass and the four mutations that must be caught."""
    out = {
        "fleet_delegate.safety": check(fleet_delegate()),
        "fleet_delegate.liveness": fleet_liveness(),
        "approval_protocol": check(approval_protocol()),
        "approval_protocol.liveness": approval_liveness(),
        "session_thread_mapping": check(session_thread_mapping()),
        "session_thread_mapping.reload": check_leads_to(session_thread_mapping(), lambda s: s[4], lambda s: not s[4], ["reload"]),
        "mutation.fleet_paused_claim": check(fleet_delegate(mutation="paused_claim")),
        "mutation.fleet_operator_revive": check(fleet_delegate(mutation="operator_revive")),
        "mutation.approval_stale_forgery": check(approval_protocol(mutation="stale_forgery")),
        "mutation.session_crash_divergence": check(session_thread_mapping(mutation="reload_drops_reverse")),
    }
    return out
