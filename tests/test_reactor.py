"""Private-deployment contracts: policy resolution, install before pull, per-request routing, exact local metering and
evaluation receipts, run against a model served by this package's CPU backend."""
import pytest

from openagents_b200.control import reactor as rx
from openagents_b200.models.config import TINY_LLAMA
from openagents_b200.models.weights import PLAN_Q8_0, random_weights, save_gguf
from openagents_b200.serve.backend import CpuBackend
from openagents_b200.serve.server import ServedModel, ServerState

T0 = "2026-07-04T14:10:00.000Z"


def _catalog():
    return rx.model_catalog("catalog.reactor.v1", [
        rx.model_provenance("model.us.open", "Acme Labs", "US", "apache-2.0", "permissive"),
        rx.model_provenance("model.cn.open", "Dragon AI", "CN", "apache-2.0", "permissive"),
        rx.model_provenance("model.us.distilled", "Acme Labs", "US", "mit", "permissive",
                            distillation_lineage=[{"developer": "Dragon AI", "originJurisdiction": "CN", "disclosure": "reported"}]),
        rx.model_provenance("model.eu.research", "Uni", "EU", "cc-by-nc-4.0", "research_only", training_data_disclosure="full"),
    ], T0)


def test_policy_resolution_reasons_and_empty_set():
    cat = _catalog()
    pol = rx.model_policy("policy.us_only", "v3", "owner.acme", {"allowOriginJurisdictions": ["US"], "allowLicenseClasses": ["permissive"],
                                                                 "blockDevelopers": [" dragon ai "], "enforceDistillationLineageJurisdiction": True})
    d = rx.resolve_model_policy(cat, pol, T0, "decision.1")
    by = {m["modelRef"]: m for m in d["modelDecisions"]}
    assert d["status"] == "conforming_models" and d["conformingModelRefs"] == ["model.us.open"] and d["refusal"] is None
    assert by["model.cn.open"]["reasonRefs"] == ["reactor.policy.origin_not_allowed", "reactor.policy.developer_blocked"]
    assert by["model.us.distilled"]["reasonRefs"] == ["reactor.policy.lineage_origin_not_allowed"]      # the ancestor decides
    assert set(by["model.eu.research"]["reasonRefs"]) == {"reactor.policy.origin_not_allowed", "reactor.policy.license_class_not_allowed"}
    # without lineage enforcement the distilled model conforms
    lax = rx.model_policy("policy.us_only", "v4", "owner.acme", {"allowOriginJurisdictions": ["US"]})
    assert rx.resolve_model_policy(cat, lax, T0, "d2")["conformingModelRefs"] == ["model.us.open", "model.us.distilled"]
    none = rx.model_policy("policy.none", "v1", "owner.acme", {"allowOriginJurisdictions": ["JP"]})
    d3 = rx.resolve_model_policy(cat, none, T0, "d3")
    assert d3["status"] == "refused_empty_set" and d3["refusal"]["reason"] == "no_conforming_models"


def test_install_then_route_and_policy_tightening_takes_effect_per_request():
    cat = _catalog()
    pol = rx.model_policy("policy.us_only", "v3", "owner.acme", {"allowOriginJurisdictions": ["US"]})
    prof = rx.node_model_profile("node.rx3.1", "model.us.open", "US Open 8B", pol, model_artifact_refs=["artifact.gguf.sha256:abc"])
    assert prof["servingLane"] == "psionic" and prof["gateway"]["phoneHomeAllowedInServingPath"] is False and prof["exactLocalMeteringRequired"]
    inst = rx.provision_model(cat, pol, prof, "install", ["artifact.gguf.sha256:abc"], T0, "d.install", "receipt.install.1")
    assert inst["status"] == "installed" and inst["weightsPullAuthorization"] == "authorized" and inst["refusal"] is None
    r = rx.route_request(cat, pol, prof, inst, "model.us.open", "req.1", T0, "d.route.1")
    assert r["status"] == "routed" and r["routedModelRef"] == "model.us.open" and r["servingPathNetwork"] == "offline_once_provisioned"
    # a request for another model than the profile's; a refused install; a policy changed after install
    assert rx.route_request(cat, pol, prof, inst, "model.cn.open", "req.2", T0, "d.route.2")["status"] == "refused_profile_mismatch"
    bad_prof = rx.node_model_profile("node.rx3.2", "model.cn.open", "CN Open", pol)
    bad = rx.provision_model(cat, pol, bad_prof, "install", [], T0, "d.install2", "receipt.install.2")
    assert bad["status"] == "refused_policy" and bad["weightsPullAuthorization"] == "refused_before_pull"
    assert bad["refusal"]["reason"] == "policy_nonconforming_model" and "reactor.policy.origin_not_allowed" in bad["refusal"]["blockerRefs"]
    assert rx.route_request(cat, pol, bad_prof, bad, "model.cn.open", "req.3", T0, "d.route.3")["status"] == "refused_not_installed"
    ghost = rx.node_model_profile("node.rx3.3", "model.unknown", "Ghost", pol)
    assert rx.provision_model(cat, pol, ghost, "install", [], T0, "d", "r")["refusal"]["reason"] == "model_not_in_catalog"
    v4 = rx.model_policy("policy.us_only", "v4", "owner.acme", {"allowOriginJurisdictions": ["US"], "blockDevelopers": ["Acme Labs"]})
    late = rx.route_request(cat, v4, prof, inst, "model.us.open", "req.4", T0, "d.route.4")
    assert late["status"] == "refused_profile_mismatch" and "blocker.reactor.router.policy_binding_mismatch" in late["blockerRefs"]
    assert "reactor.policy.developer_blocked" in late["blockerRefs"]
    with pytest.raises(rx.ContractError):
        rx.node_model_profile("n", "m", "d", pol, serving_lane="other")


def test_metering_and_evaluation_against_a_served_model(tmp_path):
    cfg = TINY_LLAMA.with_(vocab=512, d_model=64, n_heads=2, n_kv_heads=1, head_dim=32, ffn=128)
    p = str(tmp_path / "tiny.gguf")
    save_gguf(p, cfg, random_weights(cfg, 0), PLAN_Q8_0)
    model = ServedModel("model.us.open", CpuBackend.from_gguf(p), None, max_num_seqs=2)
    state = ServerState([model])
    cat = _catalog()
    pol = rx.model_policy("policy.us_only", "v3", "owner.acme", {"allowOriginJurisdictions": ["US"]})
    prof = rx.node_model_profile("node.rx3.1", "model.us.open", "US Open", pol)
    r, usage = state.complete(model, [{"role": "user", "content": "hello"}], {"max_tokens": 4})
    m = rx.local_token_metering_receipt(prof, "model.us.open", "req.1", "receipt.meter.1", T0, usage)
    assert m["usageTruth"] == "exact" and m["totalTokens"] == usage["total_tokens"] == m["promptTokens"] + 4 and m["localOnly"] and m["blockerRefs"] == []
    nm = rx.local_token_metering_receipt(prof, "model.us.open", "req.2", "receipt.meter.2", T0, None)
    assert nm["usageTruth"] == "not_measured" and nm["totalTokens"] is None and nm["blockerRefs"][0] == "blocker.reactor.local_metering.not_measured"
    with pytest.raises(rx.ContractError):
        rx.local_token_metering_receipt(prof, "m", "r", "x", T0, {"prompt_tokens": 3, "completion_tokens": 4, "total_tokens": 8})
    # the harness this lane owns, run on the served model: what the model answers is what gets scored
    answer = model.tok.decode(state.complete(model, [{"role": "user", "content": "q1"}], {"max_tokens": 3})[0].output)
    complete = lambda prompt: model.tok.decode(state.complete(model, [{"role": "user", "content": prompt}], {"max_tokens": 3})[0].output)
    meas = rx.run_task_class_eval(complete, [{"prompt": "q1", "expected": answer}, {"prompt": "q1", "expected": "\x00never\x00"}])
    assert meas == {"state": "measured", "score": 0.5, "sampleCount": 2, "scoreUnit": "exact_match", "executionTarget": "rx3_served_model"}
    e1 = rx.model_eval_receipt(cat, "model.us.open", "extraction", "receipt.eval.1", T0, meas)
    e2 = rx.model_eval_receipt(cat, "model.us.open", "drafting", "receipt.eval.2", T0, {"state": "not_measured", "reasonRef": "reason.no_dataset"})
    assert e1["capabilityCopyAllowed"] and e1["runnerOwner"] == "psionic" and e1["score"] == 0.5
    assert not e2["capabilityCopyAllowed"] and e2["executionTarget"] == "not_measured" and e2["score"] is None
    mat = rx.eval_coverage_matrix(cat, [e1, e2], "matrix.1", T0)
    assert len(mat["cells"]) == 4 * 4 and sum(c["measurementState"] == "measured" for c in mat["cells"]) == 1
    sel = rx.select_capability_copy_eval_refs("model.us.open", ["extraction", "drafting"], [e1, e2], T0, "d.copy")
    assert sel["status"] == "blocked_not_measured" and sel["allowedEvalRefs"] == ["receipt.eval.1"] and "task_class:drafting" in sel["blockerRefs"]
    assert rx.select_capability_copy_eval_refs("model.us.open", ["extraction"], [e1], T0, "d")["status"] == "allowed"
    for bad in ({"state": "measured", "score": 1.5, "sampleCount": 2, "scoreUnit": "f1", "executionTarget": "rx3_served_model"},
                {"state": "measured", "score": 0.5, "sampleCount": 0, "scoreUnit": "f1", "executionTarget": "rx3_served_model"}):
        with pytest.raises(rx.ContractError):
            rx.model_eval_receipt(cat, "model.us.open", "extraction", "r", T0, bad)
    with pytest.raises(rx.ContractError):
        rx.model_eval_receipt(cat, "model.nope", "extraction", "r", T0, meas)
    with pytest.raises(rx.ContractError):
        rx.eval_coverage_matrix(cat, [e1, dict(e1, receiptRef="dup")], "m", T0)
    model.close()


def test_airgap_bundle_is_verified_offline_and_install_ops_revalidates_policy():
    import hashlib
    from cryptography.hazmat.primitives import serialization
    from cryptography.hazmat.primitives.asymmetric.ed25519 import Ed25519PrivateKey
    cat = _catalog()
    pol = rx.model_policy("policy.us_only", "v3", "owner.acme", {"allowOriginJurisdictions": ["US"]})
    prof = rx.node_model_profile("node.rx3.1", "model.us.open", "US Open 8B", pol)
    artifact = b"weights and runtime" * 100
    digest = hashlib.sha256(artifact).hexdigest()
    key = Ed25519PrivateKey.generate()
    pub = key.public_key().public_bytes(serialization.Encoding.Raw, serialization.PublicFormat.Raw)
    sig = key.sign(bytes.fromhex(digest))
    b = rx.airgap_update_bundle_manifest(prof, "bundle.rx3.2026_07", "2026.07.1", digest, "policy.us_only", "v3", "kid.release.1", "sig.bundle.2026_07", T0)
    assert b["callbackRequired"] is False and b["signatureAlg"] == "ed25519" and b["modelRef"] == "model.us.open"
    assert rx.verify_airgap_bundle(b, artifact, sig, pub) == []
    assert rx.verify_airgap_bundle(b, artifact + b"x", sig, pub) == ["blocker.reactor.airgap_update.artifact_digest_mismatch"]
    assert rx.verify_airgap_bundle(b, artifact, sig[:-1] + bytes([sig[-1] ^ 1]), pub) == ["blocker.reactor.airgap_update.signature_invalid"]
    ok = rx.install_ops_receipt("fresh_install", b, cat, pol, prof, T0, "receipt.ops.1", verification_blockers=rx.verify_airgap_bundle(b, artifact, sig, pub))
    assert ok["status"] == "succeeded" and ok["blockerRefs"] == [] and ok["rollbackToBundleRef"] is None and "sig.bundle.2026_07" in ok["verificationRefs"]
    rb = rx.install_ops_receipt("rollback", b, cat, pol, prof, T0, "receipt.ops.2", rollback_from_bundle_ref="bundle.rx3.2026_08")
    assert rb["status"] == "succeeded" and rb["rollbackFromBundleRef"] == "bundle.rx3.2026_08" and rb["rollbackToBundleRef"] == "bundle.rx3.2026_07"
    # the policy moved on since the bundle was cut; a bundle for another node; a tampered artifact; a model the policy refuses
    v4 = rx.model_policy("policy.us_only", "v4", "owner.acme", {"allowOriginJurisdictions": ["US"]})
    prof4 = rx.node_model_profile("node.rx3.1", "model.us.open", "US Open 8B", v4)
    stale = rx.install_ops_receipt("upgrade", b, cat, v4, prof4, T0, "receipt.ops.3")
    assert stale["status"] == "refused" and stale["blockerRefs"] == ["blocker.reactor.airgap_update.policy_binding_mismatch"]
    other = rx.node_model_profile("node.rx3.9", "model.us.open", "US Open 8B", pol)
    assert "blocker.reactor.airgap_update.profile_binding_mismatch" in rx.install_ops_receipt("upgrade", b, cat, pol, other, T0, "receipt.ops.4")["blockerRefs"]
    tampered = rx.install_ops_receipt("upgrade", b, cat, pol, prof, T0, "receipt.ops.5", verification_blockers=rx.verify_airgap_bundle(b, b"other", sig, pub))
    assert tampered["status"] == "refused" and tampered["blockerRefs"] == ["blocker.reactor.airgap_update.artifact_digest_mismatch"]
    cn = rx.node_model_profile("node.rx3.2", "model.cn.open", "CN Open", pol)
    bcn = rx.airgap_update_bundle_manifest(cn, "bundle.cn", "1", digest, "policy.us_only", "v3", "kid", "sig.cn", T0)
    refused = rx.install_ops_receipt("fresh_install", bcn, cat, pol, cn, T0, "receipt.ops.6")
    assert refused["status"] == "refused" and "blocker.reactor.install_ops.policy_revalidation_failed" in refused["blockerRefs"]
    assert "reactor.policy.origin_not_allowed" in refused["blockerRefs"]
    with pytest.raises(rx.ContractError):
        rx.airgap_update_bundle_manifest(prof, "b", "1", "nothex", "p", "v", "k", "s", T0)


def _dogfood_parts():
    cat = _catalog()
    pol = rx.model_policy("policy.us_only", "v3", "owner.acme", {"allowOriginJurisdictions": ["US"], "enforceDistillationLineageJurisdiction": True})
    prof = rx.node_model_profile("node.dogfood.1", "model.us.open", "US Open 8B", pol, placement="dogfood")
    b = rx.airgap_update_bundle_manifest(prof, "bundle.1", "1", "ab" * 32, "policy.us_only", "v3", "kid", "sig.1", T0)
    ops = rx.install_ops_receipt("fresh_install", b, cat, pol, prof, T0, "receipt.ops.ok")
    cn = rx.node_model_profile("node.dogfood.1", "model.cn.open", "CN Open", pol, placement="dogfood")
    bcn = rx.airgap_update_bundle_manifest(cn, "bundle.cn", "1", "cd" * 32, "policy.us_only", "v3", "kid", "sig.cn", T0)
    refused = rx.install_ops_receipt("fresh_install", bcn, cat, pol, cn, T0, "receipt.ops.refused")
    inst = rx.provision_model(cat, pol, prof, "install", ["bundle.1"], T0, "d.i", "receipt.install")
    routes = [rx.route_request(cat, pol, prof, inst, "model.us.open", f"req.{i}", T0, f"d.route.{i}") for i in range(2)]
    meters = [rx.local_token_metering_receipt(prof, "model.us.open", f"req.{i}", f"receipt.meter.{i}", T0,
                                              {"prompt_tokens": 10 + i, "completion_tokens": 5, "total_tokens": 15 + i}) for i in range(2)]
    return cat, pol, prof, ops, refused, routes, meters


def test_dogfood_run_receipt_needs_every_receipt_to_line_up():
    cat, pol, prof, ops, refused, routes, meters = _dogfood_parts()
    kw = dict(workload_ref="workload.leadgen", case_study_ref="doc.case_study", window_started_at=T0, window_ended_at=T0, generated_at=T0, receipt_ref="receipt.dogfood.1")
    r = rx.dogfood_run_receipt(prof, pol, ops, refused, routes, meters, **kw)
    assert r["status"] == "completed" and r["blockerRefs"] == [] and r["totalMeasuredTokens"] == 31 and r["refusedNonconformingModelRef"] == "model.cn.open"
    assert r["externalClaimFlipAllowed"] is False and "constraint.distillation_lineage_jurisdiction:enforced" in r["policyConstraintRefs"]
    r2 = rx.dogfood_run_receipt(prof, pol, ops, refused, routes, meters[:1], **kw)
    assert r2["status"] == "refused" and r2["blockerRefs"] == ["blocker.reactor.dogfood.missing_metering:req.1"]
    lax = rx.model_policy("policy.us_only", "v3", "owner.acme", {"allowOriginJurisdictions": ["US", "EU"]})
    r3 = rx.dogfood_run_receipt(prof, lax, ops, ops, routes, meters, **kw)          # no strict policy; the "refused" pull actually succeeded
    assert {"blocker.reactor.dogfood.strict_single_origin_policy_missing", "blocker.reactor.dogfood.nonconforming_pull_not_refused",
            "blocker.reactor.dogfood.refused_model_matches_served_model"} <= set(r3["blockerRefs"])
    prem = rx.node_model_profile("node.dogfood.1", "model.us.open", "US Open 8B", pol)
    assert "blocker.reactor.dogfood.node_not_dogfood_placement" in rx.dogfood_run_receipt(prem, pol, ops, refused, routes, meters, **kw)["blockerRefs"]


def test_improvement_ladder_receipts():
    cat, pol, *_ = _dogfood_parts()
    plan = rx.improvement_ladder_plan("plan.ladder.1", "doc.design", T0)
    assert plan["stages"] == list(rx.IMPROVEMENT_STAGES) and plan["consentRequired"] and not plan["capabilityClaimsAuthorized"]
    h = rx.harness_evolution_receipt("model.us.open", pol, "tool_call_repair", "harness.v1", "harness.v2", 6100, 6450, 300, "dataset.snap.1", "eval.delta.1", "receipt.h.1", T0)
    assert h["accepted"] and h["deltaBps"] == 350 and h["weightChangesAllowed"] is False and h["oneMechanismOnly"] is True
    assert not rx.harness_evolution_receipt("model.us.open", pol, "loop_robustness", "a", "b", 6100, 6200, 300, "d", "e", "r", T0)["accepted"]
    d = rx.distill_to_fit_receipt(cat, pol, "model.us.open", "artifact.student.gguf", "run.distill.1", 8000, 7850, 900, 300, 200, "dataset.snap.1", "capture.prompts.1",
                                  "eval.delta.2", "receipt.d.1", T0)
    assert d["acceptedForDogfood"] and d["costReductionBps"] == 6667 and d["qualityDeltaBps"] == -150 and d["routerSwapGateStatus"] == "passed" and not d["routeSwapAuthorized"]
    worse = rx.distill_to_fit_receipt(cat, pol, "model.us.open", "a", "r", 8000, 7000, 900, 300, 200, "d", "c", "e", "receipt.d.2", T0)
    assert not worse["acceptedForDogfood"] and worse["routerSwapGateStatus"] == "blocked"
    from_cn = rx.distill_to_fit_receipt(cat, pol, "model.cn.open", "a", "r", 8000, 8000, 900, 300, 200, "d", "c", "e", "receipt.d.3", T0)
    assert not from_cn["acceptedForDogfood"] and from_cn["sourceModelConformsToPolicy"] is False       # a teacher the policy refuses taints the student
    done = rx.improvement_ladder_dogfood_receipt(plan, h, d, "receipt.ladder.1", T0)
    assert done["status"] == "completed_internal" and done["blockerRefs"] == [] and done["externalClaimFlipAllowed"] is False
    blocked = rx.improvement_ladder_dogfood_receipt(plan, h, worse, "receipt.ladder.2", T0)
    assert blocked["status"] == "blocked_for_public_claims" and blocked["blockerRefs"] == ["blocker.reactor.improvement_ladder.distill_to_fit_not_accepted"]
    with pytest.raises(rx.ContractError):
        rx.harness_evolution_receipt("m", pol, "magic", "a", "b", 1, 2, 1, "d", "e", "r", T0)
