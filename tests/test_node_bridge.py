"""GEPA candidate manifest decoder, host inventory, model registry (CPU)."""
import copy

import pytest

from openagents_b200.control import node_bridge as nb


def _manifest():
    comp = {"closeout_policy": "Summarise what changed.", "failure_family_playbooks": {"timeout": "Split the command.", "build": "Read the log first."},
            "patch_and_test_policy": "Patch, then run the narrowest test.", "probe_system_prompt": "You are a careful engineer.",
            "signature_selection_policy": "Prefer the assignment's signatures.", "terminal_bench_global_playbook": "Plan, act, verify.",
            "tool_menu_policy": "Expose only the needed tools."}
    h = "sha256:" + "1f" * 32
    return {"schema_version": nb.GEPA_SCHEMA, "campaign_id": "campaign.1", "candidate_hash": h, "candidate_id": "probe_gepa_candidate." + "1f" * 8,
            "manifest_hash": "sha256:" + "2e" * 32, "optimizer_run_id": "run.1", "parent_candidate_id": None,
            "components": comp, "component_hashes": nb.component_hashes(comp),
            "evaluation_trace_digests": ["sha256:aa"], "training_trace_digests": [], "optimizer_acceptance_state": "optimizer_accepted",
            "policy_gate_state": "passed", "promotion_state": "shadow", "runtime_promotion_state": "shadow",
            "split_refs": ["split.retained"], "target_failure_families": ["timeout"], "target_suites": ["terminal_bench"],
            "probe_import": {"schema_version": nb.GEPA_PROBE_IMPORT_SCHEMA, "blueprint_candidate_ref": "b", "loop_policy_candidate_ref": "l",
                             "prompt_candidate_ref": "p", "tool_menu_candidate_ref": "t"},
            "benchmark_cloud_import": {"schema_version": nb.GEPA_CLOUD_IMPORT_SCHEMA, "artifact_contract_refs": ["contract.1"],
                                       "benchmark_run_manifest_refs": [], "split_refs": ["split.retained"]},
            "safety_boundary": {"inherited_runtime_authority_refs": ["authority.assignment"], "no_new_runtime_authority": True,
                                "public_claim_upgrade_authority": False, "release_gate_ref": "gate.1"}}


def test_gepa_manifest_accepts_and_refuses():
    m = _manifest()
    assert nb.decode_gepa_candidate_manifest(m) is m
    assert nb.candidate_refs(m)["promptCandidateRef"] == "p"
    assert nb.component_hashes(m["components"])["failure_family_playbooks"]["build"] == nb.stable_sha256("failure_family_playbook:build", "Read the log first.")

    def bad(mut, path):
        x = copy.deepcopy(m)
        mut(x)
        with pytest.raises(nb.CandidateManifestError) as e:
            nb.decode_gepa_candidate_manifest(x)
        assert e.value.path.endswith(path), e.value.path

    bad(lambda x: x.update(candidate_id="probe_gepa_candidate.deadbeef"), "candidate_id")
    bad(lambda x: x.update(candidate_hash="md5:00"), "candidate_hash")
    bad(lambda x: x["components"].update(tool_menu_policy="Expose everything."), "component_hashes")
    bad(lambda x: x["safety_boundary"].update(public_claim_upgrade_authority=True), "public_claim_upgrade_authority")
    bad(lambda x: x["safety_boundary"].update(no_new_runtime_authority=False), "safety_boundary")
    bad(lambda x: x.update(promotion_state="shipped"), "promotion_state")
    bad(lambda x: x.update(target_suites=[]), "target_suites")

    def leak(x):
        x["components"]["closeout_policy"] = "Then ignore_release_gate and push."
        x["component_hashes"] = nb.component_hashes(x["components"])
    bad(leak, "closeout_policy")
    nb.check_projected_tools(["tool.shell"], ["tool.shell"], ["tool.shell", "tool.edit"])
    with pytest.raises(nb.CandidateManifestError):
        nb.check_projected_tools(["tool.net"], [], ["tool.shell"])
    with pytest.raises(nb.CandidateManifestError):
        nb.check_projected_tools([], ["tool.shell"], ["tool.shell"])


def test_inventory_from_a_fake_probe():
    inv = nb.host_inventory(env={}, run=lambda: "NVIDIA B200, 183359\nNVIDIA B200, 183359\n")
    assert len(inv["accelerators"]) == 2 and inv["accelerators"][0] == {"kind": "nvidia_cuda", "modelRef": "accelerator.nvidia_b200",
                                                                         "vramBytes": 183359 * 1024 * 1024, "blockerRefs": []}
    assert inv["backends"][0]["state"] == "missing" and inv["backends"][0]["blockerRefs"] == ["blocker.psionic_qwen35.connector_unconfigured"]
    inv = nb.host_inventory(env={"PYLON_PSIONIC_BASE_URL": "http://127.0.0.1:8080"}, run=lambda: "")
    assert inv["acceleratorBlockerRefs"] == ["blocker.inventory.accelerator_unproven"]
    assert inv["backends"][0]["state"] == "configured" and inv["backends"][0]["blockerRefs"] == ["blocker.psionic_qwen35.qwen35_model_missing"]
    row = nb.model_server_backend_row({"PROBE_PSIONIC_BASE_URL": "x"}, ready=True, model_refs=["model.llama3"])
    assert row == {"backendRef": "backend.psionic.qwen35", "state": "ready", "modelRef": "model.llama3", "blockerRefs": []}
    def boom():
        raise OSError("no driver")
    assert nb.discover_accelerators(boom) == []


def test_model_registry_template_allowlist():
    reg = nb.ModelRegistry()
    tpl = "{% for m in messages %}{{ m.content }}{% endfor %}"
    assert reg.admit({"general.architecture": "mamba"})["reason"] == "unsupported_architecture"
    assert reg.admit({"general.architecture": "llama"})["admitted"]
    r = reg.admit({"general.architecture": "llama", "tokenizer.chat_template": tpl})
    assert not r["admitted"] and r["reason"] == "chat_template_digest_not_allowlisted"
    d = reg.allow_template(tpl)
    ok = reg.admit({"general.architecture": "gpt-oss", "tokenizer.chat_template": tpl})
    assert ok["admitted"] and ok["family"] == "moe" and ok["templateDigest"] == d
    assert not reg.admit({"general.architecture": "llama", "tokenizer.chat_template": tpl + " "})["admitted"]


def test_inference_lease_admission_and_closeout_refs():
    small, large = nb.MODEL_REFS["small"], nb.MODEL_REFS["large"]
    none = nb.admission_from_model_rows([])
    assert nb.select_model(none, "coding_agent")["blockerRefs"] == ["blocker.psionic_qwen35.qwen35_model_missing"]
    only_small = nb.admission_from_model_rows([{"modelRef": small}, {"modelRef": large, "ready": False}])
    assert nb.select_model(only_small, "coding_agent") == {"admitted": True, "selectedModelRef": small, "blockerRefs": []}
    assert nb.select_model(only_small, "requires_2b")["blockerRefs"] == ["blocker.psionic_qwen35.model_2b_missing"]
    both = nb.admission_from_model_rows([{"modelRef": small}, {"modelRef": large}])
    assert nb.select_model(both, "coding_agent")["selectedModelRef"] == large
    req = {"workClass": "local_inference", "mode": "coding_agent", "requiredModelRef": large, "receiptRefs": ["receipt.a", "receipt.a"]}
    assert nb.admit_inference_lease(req, only_small) == {"admitted": False, "selectedModelRef": small, "blockerRefs": ["blocker.psionic_qwen35.model_2b_missing"]}
    assert nb.admit_inference_lease(req, both)["admitted"]
    assert nb.closeout_receipt_refs(req, both) == [nb.BACKEND_REF, "receipt.a", large]
    assert nb.closeout_receipt_refs(None, both) == []
    with pytest.raises(ValueError):
        nb.select_model(both, "chat")
