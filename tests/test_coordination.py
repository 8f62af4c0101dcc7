"""NIP-TRN records, commit authority, mesh election, reactor lanes (CPU)."""
import json

import pytest

from openagents_b200.control import coordination as co


def _window():
    return co.training_window("net.alpha", "window.000042", 42, "ckpt-041", planned_local_steps=64, policy="policy-7",
                              min_participants=2, min_weight_fraction=0.8)


def test_trn_events_have_required_tags_and_no_tensors():
    net = co.network_contract("net.alpha", "Alpha", "gov-3")
    node = co.node_record("net.alpha", "node-1", ["miner", "validator"])
    w = _window()
    r = co.training_receipt(w, "trainer1", 64, 1_048_576, "artifact.1", "sha256:ab")
    v = co.validator_verdict(w, "receipt-0", "trainer1", "accepted")
    a = co.artifact_locator(w, "artifact.1", "local_update", "ab" * 32, "https://cdn.example/a.safetensors", update_format="pseudo_gradient")
    for ev in (net, node, w, r, v, a):
        assert co.check_event(ev) == []
        assert json.loads(ev["content"])["schema"] == 1
    assert co.first_tag(w, "aggregation_rule") == "weighted_avg"
    assert co.first_tag(r, "base_checkpoint") == "ckpt-041"
    assert ["cap", "accelerator", "8xb200"] in node["tags"]
    with pytest.raises(co.TrnError):
        co._event(co.KIND_RECEIPT, {"gradients": [1, 2]}, [])
    bad = {"kind": co.KIND_WINDOW, "content": "{}", "tags": [["d", "w"]]}
    assert "missing_tag:network" in co.check_event(bad) and "content_schema" in co.check_event(bad)
    with pytest.raises(co.TrnError):
        co.validator_verdict(w, "r", "t", "maybe")


def test_aggregate_window_applies_verdicts_base_and_quorum():
    w = _window()
    rs = [co.training_receipt(w, f"t{i}", 64, n, f"art.{i}", "sha256:00") for i, n in enumerate((1000, 3000, 500))]
    for i, r in enumerate(rs):
        r["id"] = f"rid{i}"
    stale = co.training_receipt(co.training_window("net.alpha", "window.000042", 42, "ckpt-040", 64, "p"), "t9", 64, 800, "art.9", "sha256:00")
    stale["id"] = "rid9"
    vs = [co.validator_verdict(w, "rid0", "t0", "accepted"), co.validator_verdict(w, "rid1", "t1", "accepted"),
          co.validator_verdict(w, "rid2", "t2", "rejected", "loss_regression"), co.validator_verdict(w, "rid9", "t9", "accepted")]
    agg = co.aggregate_window(w, rs + [stale], vs)
    assert [a["trainer"] for a in agg["admitted"]] == ["t0", "t1"]
    assert agg["admitted_weight_total"] == "4000" and agg["normalized_weights"] == [0.25, 0.75]
    assert not agg["quorum_met"]                       # 4000 / 5300 < 0.8
    agg2 = co.aggregate_window(w, rs[:2], vs)
    assert agg2["quorum_met"] and agg2["promotion_state"] == "candidate"


def test_commit_authority_terms_and_leases():
    ca = co.CommitAuthority()
    assert ca.claim("a", 0) and ca.term == 1 and ca.may_commit("a", 1, 10)
    assert not ca.claim("b", 100)                       # lease still held
    assert ca.claim("a", 20_000) and ca.term == 1       # renewal keeps the term
    assert ca.claim("b", 60_000) and ca.term == 2 and not ca.may_commit("a", 1, 60_001)
    other = co.CommitAuthority()
    assert other.observe(**{"term": 2, "holder": "b", "lease_expires_ms": 90_000})
    assert not other.observe(2, "a", 999_999)           # equal term, different holder: ignored
    assert not other.observe(1, "a", 999_999)
    assert other.to_manifest() == {"commitTerm": 2, "commitHolder": "b", "leaseExpiresMs": 90_000}


def test_mesh_election_promotes_standby_and_places():
    m = co.MeshElection()
    assert m.heartbeat("h1", 0) == "elected" and m.term == 1
    assert m.heartbeat("h2", 10) == "standby" and m.heartbeat("h3", 20) == "standby"
    assert m.heartbeat("h1", 5_000) == "active"
    assert m.heartbeat("h3", 20_000) == "standby"       # lease ran out: first standby (h2) is promoted, not the caller
    assert m.active_host == "h2" and m.term == 2 and "h3" in m.standby
    p = m.placement("pipeline_sharded", 4, n_layers=30)
    assert [s["layerStart"] for s in p["stages"]] == [0, 8, 16, 24] and p["stages"][-1]["layerEnd"] == 30
    assert m.placement("sparse_expert", 8, n_experts=32)["expertRanges"][3] == [12, 16]
    with pytest.raises(ValueError):
        m.placement("sparse_expert", 3, n_experts=32)
    with pytest.raises(ValueError):
        m.placement("ring", 2)


def test_reactor_lane():
    assert co.reactor_model_profile("gpt-oss-20b", "psionic")["servingLane"] == "psionic"
    with pytest.raises(ValueError):
        co.reactor_model_profile("m", "vllm")
