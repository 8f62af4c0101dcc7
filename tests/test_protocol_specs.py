"""The control-plane protocol models: four configurations pass, four deliberate bugs are caught with the expected
property, and the liveness check itself can fail (it reports a fair non-progressing behaviour when fairness is withdrawn)."""
from openagents_b200.control import protocol_specs as ps


def test_passing_configurations_and_mutations():
    out = ps.run_all()
    for name, o in out.items():
        if name.startswith("mutation."):
            assert not o.ok and o.trace, name
        else:
            assert o.ok, (name, o.violated, o.trace)
    assert out["mutation.fleet_paused_claim"].violated == "invariant PausedRunsClaimNothing"
    assert out["mutation.fleet_operator_revive"].violated == "invariant SupervisorReviveHonorsAutoRevivableGuard"
    assert out["mutation.approval_stale_forgery"].violated == "action property NoStaleApproveApplication"
    assert out["mutation.session_crash_divergence"].violated == "invariant NoOrphanThreadBinding"
    assert out["fleet_delegate.safety"].states > 1000       # two racing supervisors, two units: a real state space


def test_counterexample_trace_starts_at_init_and_ends_in_the_bad_state():
    o = ps.check(ps.approval_protocol(mutation="stale_forgery"))
    assert o.trace[0][0] == "init"
    names = [a for a, _ in o.trace]
    # the forged approve needs a request issued in an old epoch: issue, issue, close one by interrupt/supersede, approve the other
    assert names.count("issue") == 2 and any(n in ("interrupt", "supersede") for n in names)


def test_liveness_check_can_fail():
    m = ps.session_thread_mapping()
    assert ps.check_leads_to(m, lambda s: s[4], lambda s: not s[4], ["reload"])
    o = ps.check_leads_to(m, lambda s: s[4], lambda s: not s[4], [])          # nobody is obliged to reload: may stay crashed
    assert not o.ok and "temporal" in o.violated
    # a draining fleet run ends only because completion and drain_complete are fair
    f = ps.fleet_delegate(("s1",), ("w1",), 1, 1, 0)
    assert not ps.check_leads_to(f, lambda s: s[0] == "draining", lambda s: s[0] in ("completed", "stopped"), ["tick"]).ok


def test_larger_bounds_still_hold():
    assert ps.check(ps.approval_protocol(("a", "b", "c")))
    assert ps.check(ps.session_thread_mapping(("s1", "s2", "s3"), ("t1", "t2")))
    assert ps.check(ps.fleet_delegate(("s1", "s2"), ("w1", "w2", "w3"), capacity=2, claim_ttl=1, max_releases=1), max_states=2_000_000)
