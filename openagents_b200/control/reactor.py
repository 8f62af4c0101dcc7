"""Private-deployment ("reactor") contracts for a node that serves open models with this engine.

A deployment declares, per model, a node profile (which model, which serving lane: ``psionic`` for this engine or
``hydralisk`` for owner-run vLLM hosts, the OpenAI-compatible gateway endpoint, exact local metering required, no phone-home
in the serving path); an owner policy decides which catalogued models may be installed and served (jurisdiction, developer,
licence, weights openness, training-data disclosure, optionally the same for every distillation ancestor); every step
leaves a receipt: policy decision, install (weights are pulled only after the policy check), route decision per request,
local token metering per request (exact counts that reconcile, or an explicit ``not_measured``), evaluation per
(model, task class), a coverage matrix over the catalogue, and the rule that a capability claim may only be copied from
MEASURED evaluations.  The evaluation harness is owned by this engine's lane.

Restates packages/reactor-contracts/src/index.ts: lanes and profiles :61-156, policy :194-255, install / route / metering
receipts :258-333, evaluation :336-390, policy resolution :1106-1225, provisioning :1242-1305, routing :1317-1391, metering
:1396-1444, harness profile :1454-1468, evaluation receipts and coverage :1476-1680, air-gapped update bundles and
install operations :1675-1811, the dog-food run :1813-1949, the improvement ladder :789-910.  Records are plain dicts with the
reference's field names; ``ContractError`` replaces schema-decoding failures.  The need-to-know corpus rules and the
data-liberation pipeline of that package are in ``control.reactor_data``.
"""
from __future__ import annotations

SERVING_LANES = ("hydralisk", "psionic")
ENGINE_KINDS = ("vllm", "sglang", "tensorrt-llm", "llama.cpp", "fixture-openai-compatible", "openagents_b200")
PLACEMENTS = ("customer_premises", "customer_controlled_cloud", "dogfood", "fixture")
EVAL_TASK_CLASSES = ("drafting", "extraction", "rag_over_corpus", "agent_tool_use")
EVAL_TARGETS = ("rx3_served_model", "hosted_equivalent_large_model", "not_measured")
EVAL_SCORE_UNITS = ("score_0_to_1", "pass_rate", "exact_match", "f1")
ROUTING_PREFERENCES = ("capability_first", "sovereignty_first", "balanced")

PSIONIC_EVAL_HARNESS_PROFILE = {
    "schemaVersion": "openagents.reactor.eval_harness_profile.v1",
    "harnessRef": "reactor.eval_harness.psionic.task_class.v1",
    "runnerOwner": "psionic",
    "sourceRefs": ["openagents_b200.control.reactor.run_task_class_eval"],
    "supportedExecutionTargets": list(EVAL_TARGETS),
    "taskClassRefs": list(EVAL_TASK_CLASSES),
    "unrunMeasurementState": "not_measured",
}


class ContractError(ValueError):
    pass


def _need(cond: bool, code: str):
    if not cond:
        raise ContractError(code)


def _unique(xs):
    return list(dict.fromkeys(xs))


# ------------------------------------------------------------------------------------------------ records
def model_provenance(model_ref: str, developer: str, origin_jurisdiction: str, license: str, license_class: str,
                     weights_openness: str = "open_weights", training_data_disclosure: str = "undisclosed",
                     distillation_lineage: list[dict] | None = None, **extra) -> dict:
    """One catalogue row.  ``distillation_lineage``: ancestors as ``{developer, originJurisdiction, disclosure}``."""
    _need(bool(model_ref and developer and origin_jurisdiction), "reactor.catalog.incomplete_provenance")
    return {"modelRef": model_ref, "developer": developer, "originJurisdiction": origin_jurisdiction, "license": license,
            "licenseClass": license_class, "weightsOpenness": weights_openness, "trainingDataDisclosure": training_data_disclosure,
            "distillationLineage": list(distillation_lineage or []), **extra}


def model_catalog(catalog_ref: str, models: list[dict], generated_at: str, source_refs=()) -> dict:
    refs = [m["modelRef"] for m in models]
    _need(len(refs) == len(set(refs)), "reactor.catalog.duplicate_model_ref")
    return {"schemaVersion": "openagents.reactor_model_catalog.v1", "catalogRef": catalog_ref, "generatedAt": generated_at,
            "models": list(models), "sourceRefs": list(source_refs)}


def model_policy(policy_ref: str, version: str, owner_ref: str, constraints: dict, default_preference: str = "balanced",
                 task_preferences: list[dict] | None = None, source_refs=()) -> dict:
    _need(default_preference in ROUTING_PREFERENCES, "reactor.policy.unknown_routing_preference")
    c = {"enforceDistillationLineageJurisdiction": False, **constraints}
    return {"schemaVersion": "openagents.reactor.model_policy.v1", "constraints": c, "ownerRef": owner_ref, "policyRef": policy_ref,
            "routingPreferences": {"defaultPreference": default_preference, "taskPreferences": list(task_preferences or [])},
            "sourceRefs": list(source_refs), "version": version}


def node_model_profile(node_profile_ref: str, model_ref: str, display_name: str, policy: dict, serving_lane: str = "psionic",
                       engine_kind: str = "openagents_b200", engine_ref: str = "engine.openagents_b200", image_digest_ref: str = "",
                       model_artifact_refs=(), version_ref: str = "", endpoint_ref: str = "http://127.0.0.1:8080/v1",
                       placement: str = "customer_premises", source_refs=()) -> dict:
    _need(serving_lane in SERVING_LANES, "reactor.profile.unknown_serving_lane")
    _need(engine_kind in ENGINE_KINDS, "reactor.profile.unknown_engine_kind")
    _need(placement in PLACEMENTS, "reactor.profile.unknown_placement")
    return {"schemaVersion": "openagents.reactor.node_model_profile.v1", "displayName": display_name, "exactLocalMeteringRequired": True,
            "gateway": {"endpointRef": endpoint_ref, "phoneHomeAllowedInServingPath": False, "protocol": "openai.chat_completions.v1",
                        "servingPathNetwork": "offline_once_provisioned"},
            "modelRef": model_ref, "nodeProfileRef": node_profile_ref, "placement": placement, "policyRef": policy["policyRef"],
            "policyVersion": policy["version"], "servingLane": serving_lane,
            "servingStack": {"engineRef": engine_ref, "imageDigestRef": image_digest_ref, "kind": engine_kind,
                             "modelArtifactRefs": list(model_artifact_refs), "versionRef": version_ref},
            "sourceRefs": list(source_refs)}


# ------------------------------------------------------------------------------------------------ policy
def _norm(s: str) -> str:
    return s.strip().lower()


def _allowed(values, v, text=False) -> bool:          # an absent allow-list allows everything
    if values is None:
        return True
    return _norm(v) in [_norm(x) for x in values] if text else v in values


def _blocked(values, v, text=False) -> bool:
    if values is None:
        return False
    return _norm(v) in [_norm(x) for x in values] if text else v in values


def refusal_reasons(policy: dict, model: dict) -> list[str]:
    c, r = policy["constraints"], []
    if not _allowed(c.get("allowOriginJurisdictions"), model["originJurisdiction"]):
        r.append("reactor.policy.origin_not_allowed")
    if _blocked(c.get("blockOriginJurisdictions"), model["originJurisdiction"]):
        r.append("reactor.policy.origin_blocked")
    if not _allowed(c.get("allowDevelopers"), model["developer"], text=True):
        r.append("reactor.policy.developer_not_allowed")
    if _blocked(c.get("blockDevelopers"), model["developer"], text=True):
        r.append("reactor.policy.developer_blocked")
    if not _allowed(c.get("allowLicenses"), model["license"]):
        r.append("reactor.policy.license_not_allowed")
    if not _allowed(c.get("allowLicenseClasses"), model["licenseClass"]):
        r.append("reactor.policy.license_class_not_allowed")
    if not _allowed(c.get("allowWeightsOpenness"), model["weightsOpenness"]):
        r.append("reactor.policy.weights_openness_not_allowed")
    if not _allowed(c.get("requireTrainingDataDisclosure"), model["trainingDataDisclosure"]):
        r.append("reactor.policy.training_data_disclosure_not_allowed")
    if c.get("enforceDistillationLineageJurisdiction"):
        for anc in model.get("distillationLineage", []):
            if not _allowed(c.get("allowOriginJurisdictions"), anc["originJurisdiction"]):
                r.append("reactor.policy.lineage_origin_not_allowed")
            if _blocked(c.get("blockOriginJurisdictions"), anc["originJurisdiction"]):
                r.append("reactor.policy.lineage_origin_blocked")
    return _unique(r)


def resolve_model_policy(catalog: dict, policy: dict, decided_at: str, decision_ref: str, source_refs=()) -> dict:
    decisions = []
    for m in catalog["models"]:
        why = refusal_reasons(policy, m)
        decisions.append({"modelRef": m["modelRef"], "reasonRefs": why, "status": "refused" if why else "conforming"})
    ok = [d["modelRef"] for d in decisions if d["status"] == "conforming"]
    return {"schemaVersion": "openagents.reactor.model_policy_decision.v1", "catalogRef": catalog["catalogRef"],
            "conformingModelRefs": ok, "decidedAt": decided_at, "decisionRef": decision_ref, "modelDecisions": decisions,
            "policyRef": policy["policyRef"], "policyVersion": policy["version"],
            "refusal": None if ok else {"blockerRefs": _unique(x for d in decisions for x in d["reasonRefs"]), "reason": "no_conforming_models"},
            "sourceRefs": _unique([catalog["catalogRef"], policy["policyRef"], *source_refs]),
            "status": "conforming_models" if ok else "refused_empty_set"}


def _decision_for(decision: dict, model_ref: str):
    return next((d for d in decision["modelDecisions"] if d["modelRef"] == model_ref), None)


def provision_model(catalog: dict, policy: dict, profile: dict, action: str, artifact_refs, decided_at: str, decision_ref: str,
                    receipt_ref: str, source_refs=()) -> dict:
    """Install or upgrade: the weights pull is authorised only after the policy, the profile's policy binding and the
    catalogue all agree."""
    _need(action in ("install", "upgrade"), "reactor.provision.unknown_action")
    pd = resolve_model_policy(catalog, policy, decided_at, decision_ref, [profile["nodeProfileRef"], *source_refs])
    md = _decision_for(pd, profile["modelRef"])
    blockers = []
    if profile["policyRef"] != policy["policyRef"] or profile["policyVersion"] != policy["version"]:
        blockers.append("blocker.reactor.provision.policy_binding_mismatch")
    if md is None:
        blockers.append("blocker.reactor.provision.model_not_in_catalog")
    elif md["status"] != "conforming":
        blockers += ["blocker.reactor.provision.policy_nonconforming_model", *md["reasonRefs"]]
    blockers = _unique(blockers)
    ok = not blockers
    reason = ("model_not_in_catalog" if "blocker.reactor.provision.model_not_in_catalog" in blockers else
              "policy_binding_mismatch" if "blocker.reactor.provision.policy_binding_mismatch" in blockers else "policy_nonconforming_model")
    return {"schemaVersion": "openagents.reactor.model_install_receipt.v1", "action": action, "artifactRefs": list(artifact_refs),
            "catalogRef": catalog["catalogRef"], "decidedAt": decided_at, "decisionRef": decision_ref, "modelRef": profile["modelRef"],
            "nodeProfileRef": profile["nodeProfileRef"], "policyDecisionRef": pd["decisionRef"], "policyRef": policy["policyRef"],
            "policyVersion": policy["version"], "receiptRef": receipt_ref,
            "refusal": None if ok else {"blockerRefs": blockers, "reason": reason}, "servingLane": profile["servingLane"],
            "sourceRefs": _unique([profile["nodeProfileRef"], policy["policyRef"], pd["decisionRef"], *artifact_refs, *source_refs]),
            "status": "installed" if ok else "refused_policy", "weightsPullAuthorization": "authorized" if ok else "refused_before_pull"}


def route_request(catalog: dict, policy: dict, profile: dict, install_receipt: dict, requested_model_ref: str, request_ref: str,
                  decided_at: str, decision_ref: str, source_refs=()) -> dict:
    """Per-request route decision of the local OpenAI-compatible gateway: the policy is re-evaluated on every request, so
    tightening it takes effect without reinstalling."""
    pd = resolve_model_policy(catalog, policy, decided_at, decision_ref, [profile["nodeProfileRef"], request_ref])
    md = _decision_for(pd, requested_model_ref)
    b = []
    if profile["modelRef"] != requested_model_ref:
        b.append("blocker.reactor.router.profile_model_mismatch")
    if (install_receipt["nodeProfileRef"] != profile["nodeProfileRef"] or install_receipt["modelRef"] != profile["modelRef"] or
            install_receipt["policyRef"] != policy["policyRef"] or install_receipt["policyVersion"] != policy["version"]):
        b.append("blocker.reactor.router.install_receipt_binding_mismatch")
    if profile["policyRef"] != policy["policyRef"] or profile["policyVersion"] != policy["version"]:
        b.append("blocker.reactor.router.policy_binding_mismatch")
    if install_receipt["status"] != "installed" or install_receipt["weightsPullAuthorization"] != "authorized":
        b.append("blocker.reactor.router.model_not_installed")
    if md is None:
        b.append("blocker.reactor.router.model_not_in_catalog")
    elif md["status"] != "conforming":
        b += ["blocker.reactor.router.policy_nonconforming_model", *md["reasonRefs"]]
    b = _unique(b)
    if not b:
        status = "routed"
    elif "blocker.reactor.router.profile_model_mismatch" in b or "blocker.reactor.router.policy_binding_mismatch" in b:
        status = "refused_profile_mismatch"
    elif "blocker.reactor.router.model_not_installed" in b:
        status = "refused_not_installed"
    else:
        status = "refused_policy"
    return {"schemaVersion": "openagents.reactor.route_decision.v1", "blockerRefs": b, "catalogRef": catalog["catalogRef"],
            "decidedAt": decided_at, "decisionRef": decision_ref, "gatewayProtocol": profile["gateway"]["protocol"],
            "nodeProfileRef": profile["nodeProfileRef"], "policyDecisionRef": pd["decisionRef"], "policyRef": policy["policyRef"],
            "policyVersion": policy["version"], "requestRef": request_ref, "requestedModelRef": requested_model_ref,
            "routedModelRef": requested_model_ref if not b else None, "servingLane": profile["servingLane"],
            "servingPathNetwork": profile["gateway"]["servingPathNetwork"],
            "sourceRefs": _unique([profile["nodeProfileRef"], install_receipt["receiptRef"], policy["policyRef"], pd["decisionRef"], *source_refs]),
            "status": status}


# ------------------------------------------------------------------------------------------------ metering
def local_token_metering_receipt(profile: dict, model_ref: str, request_ref: str, receipt_ref: str, generated_at: str,
                                 usage: dict | None, reason_ref: str = "reason.reactor.local_metering.engine_reported_no_usage",
                                 source_refs=()) -> dict:
    """``usage``: this server's OpenAI usage object (``prompt_tokens`` / ``completion_tokens`` / ``total_tokens``) or None.
    Exact counts must be non-negative integers that add up; anything else is an error, never an estimate."""
    exact = usage is not None
    if exact:
        p, c, t = usage.get("prompt_tokens"), usage.get("completion_tokens"), usage.get("total_tokens")
        ok = all(isinstance(v, int) and not isinstance(v, bool) and v >= 0 for v in (p, c, t))
        _need(ok and p + c == t, "reactor.local_metering.exact_counts_do_not_reconcile")
    return {"schemaVersion": "openagents.reactor.local_token_metering_receipt.v1",
            "blockerRefs": [] if exact else ["blocker.reactor.local_metering.not_measured", reason_ref],
            "completionTokens": usage["completion_tokens"] if exact else None, "generatedAt": generated_at, "localOnly": True,
            "measurementState": "measured" if exact else "not_measured", "modelRef": model_ref, "nodeProfileRef": profile["nodeProfileRef"],
            "policyRef": profile["policyRef"], "policyVersion": profile["policyVersion"],
            "promptTokens": usage["prompt_tokens"] if exact else None, "receiptRef": receipt_ref, "requestRef": request_ref,
            "servingLane": profile["servingLane"], "sourceRefs": _unique([profile["nodeProfileRef"], request_ref, *source_refs]),
            "totalTokens": usage["total_tokens"] if exact else None, "usageTruth": "exact" if exact else "not_measured"}


# ------------------------------------------------------------------------------------------------ evaluation
def run_task_class_eval(complete, samples: list[dict], score_unit: str = "exact_match") -> dict:
    """The harness this lane owns: ``complete(prompt) -> text`` is the served model (greedy); each sample is
    ``{prompt, expected}``; a sample passes when the expected string occurs in the answer.  Returns the measurement part of
    an evaluation receipt."""
    _need(len(samples) > 0, "reactor.eval.no_samples")
    hits = sum(1 for s in samples if str(s["expected"]) in complete(s["prompt"]))
    return {"state": "measured", "score": hits / len(samples), "sampleCount": len(samples), "scoreUnit": score_unit,
            "executionTarget": "rx3_served_model"}


def model_eval_receipt(catalog: dict, model_ref: str, task_class_ref: str, receipt_ref: str, generated_at: str, measurement: dict,
                       eval_dataset_ref: str | None = None, harness: dict | None = None, source_refs=()) -> dict:
    h = harness or PSIONIC_EVAL_HARNESS_PROFILE
    _need(any(m["modelRef"] == model_ref for m in catalog["models"]), "reactor.eval.model_not_in_catalog")
    _need(task_class_ref in EVAL_TASK_CLASSES and task_class_ref in h["taskClassRefs"], "reactor.eval.task_class_not_supported_by_harness")
    measured = measurement.get("state") == "measured"
    if measured:
        sc, n = measurement.get("score"), measurement.get("sampleCount")
        _need(isinstance(sc, (int, float)) and 0 <= sc <= 1 and isinstance(n, int) and n > 0,
              "reactor.eval.measured_receipt_invalid_score_or_samples")
        _need(measurement.get("executionTarget") in h["supportedExecutionTargets"], "reactor.eval.execution_target_not_supported_by_harness")
        _need(measurement.get("scoreUnit") in EVAL_SCORE_UNITS, "reactor.eval.unknown_score_unit")
    return {"schemaVersion": "openagents.reactor.model_eval_receipt.v1",
            "blockerRefs": [] if measured else ["blocker.reactor.eval.not_measured", measurement.get("reasonRef", "reason.reactor.eval.not_run")],
            "capabilityCopyAllowed": measured,
            "evalDatasetRef": eval_dataset_ref or ("dataset.reactor.task_class_eval.inline" if measured else "dataset.reactor.task_class_eval.not_measured"),
            "executionTarget": measurement["executionTarget"] if measured else "not_measured", "generatedAt": generated_at,
            "harnessRef": h["harnessRef"], "measurementState": "measured" if measured else "not_measured", "modelRef": model_ref,
            "receiptRef": receipt_ref, "runnerOwner": h["runnerOwner"], "sampleCount": measurement["sampleCount"] if measured else None,
            "score": float(measurement["score"]) if measured else None, "scoreUnit": measurement["scoreUnit"] if measured else None,
            "sourceRefs": _unique([catalog["catalogRef"], h["harnessRef"], *source_refs]), "taskClassRef": task_class_ref}


def _measured_by_key(receipts: list[dict]) -> dict:
    out = {}
    for r in receipts:
        if r["measurementState"] != "measured" or not r["capabilityCopyAllowed"]:
            continue
        k = (r["modelRef"], r["taskClassRef"])
        _need(k not in out, "reactor.eval.duplicate_measured_receipt_for_model_task")
        out[k] = r
    return out


def eval_coverage_matrix(catalog: dict, receipts: list[dict], matrix_ref: str, generated_at: str, task_class_refs=None, source_refs=()) -> dict:
    tasks = _unique(task_class_refs or EVAL_TASK_CLASSES)
    _need(all(t in EVAL_TASK_CLASSES for t in tasks), "reactor.eval.unknown_task_class")
    by = _measured_by_key(receipts)
    cells = []
    for m in catalog["models"]:
        for t in tasks:
            r = by.get((m["modelRef"], t))
            cells.append({"blockerRefs": [], "capabilityCopyAllowed": True, "measurementState": "measured", "modelRef": m["modelRef"],
                          "receiptRef": r["receiptRef"], "score": r["score"], "taskClassRef": t} if r else
                         {"blockerRefs": ["blocker.reactor.eval.not_measured", f"model:{m['modelRef']}", f"task_class:{t}"],
                          "capabilityCopyAllowed": False, "measurementState": "not_measured", "modelRef": m["modelRef"], "receiptRef": None,
                          "score": None, "taskClassRef": t})
    return {"schemaVersion": "openagents.reactor.eval_coverage_matrix.v1", "catalogRef": catalog["catalogRef"], "cells": cells,
            "generatedAt": generated_at, "matrixRef": matrix_ref,
            "sourceRefs": _unique([catalog["catalogRef"], *[r["receiptRef"] for r in receipts], *source_refs])}


def select_capability_copy_eval_refs(model_ref: str, task_class_refs, receipts: list[dict], decided_at: str, decision_ref: str,
                                     source_refs=()) -> dict:
    """Marketing or catalogue copy may cite a capability only from measured evaluations of exactly that model and task."""
    tasks = _unique(task_class_refs)
    _need(all(t in EVAL_TASK_CLASSES for t in tasks), "reactor.eval.unknown_task_class")
    by = _measured_by_key(receipts)
    allowed = [by[(model_ref, t)]["receiptRef"] for t in tasks if (model_ref, t) in by]
    blockers = [x for t in tasks if (model_ref, t) not in by
                for x in ("blocker.reactor.capability_copy.eval_not_measured", f"model:{model_ref}", f"task_class:{t}")]
    return {"schemaVersion": "openagents.reactor.capability_copy_eval_decision.v1", "allowedEvalRefs": allowed, "blockerRefs": blockers,
            "decidedAt": decided_at, "decisionRef": decision_ref, "modelRef": model_ref, "sourceRefs": _unique([*allowed, *source_refs]),
            "status": "allowed" if not blockers else "blocked_not_measured", "taskClassRefs": tasks}


# ---------------------------------------------------------------- air-gapped updates (index.ts:405-447 types, :1675-1811 builders)
AIRGAP_VERIFIER_REF = "openagents_b200.control.reactor.verify_airgap_bundle"
AIRGAP_PUBLIC_KEY_REF = "keys/release-pubkey.json"


def airgap_update_bundle_manifest(profile: dict, bundle_ref: str, bundle_version: str, artifact_sha256: str, policy_ref: str, policy_version: str,
                                  signature_kid: str, signature_ref: str, created_at: str, public_key_ref: str = AIRGAP_PUBLIC_KEY_REF,
                                  verifier_ref: str = AIRGAP_VERIFIER_REF, source_refs=()) -> dict:
    """What travels on the medium beside the artifact: which model for which node profile under which policy version, the
    artifact's SHA-256, and where the detached ed25519 signature and its public key are.  Never needs a callback."""
    _need(len(artifact_sha256) == 64 and all(c in "0123456789abcdef" for c in artifact_sha256), "reactor.airgap.artifact_sha256")
    return {"schemaVersion": "openagents.reactor.airgap_update_bundle_manifest.v1", "artifactSha256": artifact_sha256, "bundleRef": bundle_ref,
            "bundleVersion": bundle_version, "callbackRequired": False, "createdAt": created_at, "modelRef": profile["modelRef"],
            "nodeProfileRef": profile["nodeProfileRef"], "policyRef": policy_ref, "policyVersion": policy_version, "publicKeyRef": public_key_ref,
            "signatureAlg": "ed25519", "signatureKid": signature_kid, "signatureRef": signature_ref,
            "sourceRefs": _unique([profile["nodeProfileRef"], signature_ref, public_key_ref, verifier_ref, *source_refs]), "verifierRef": verifier_ref}


def verify_airgap_bundle(bundle: dict, artifact: bytes, signature: bytes, public_key: bytes) -> list[str]:
    """Offline check of a bundle on the node: the artifact hashes to what the manifest says and the detached signature over
    that digest verifies under the given ed25519 public key (32 raw bytes).  Returns blocker refs (empty = verified)."""
    import hashlib
    out = []
    if hashlib.sha256(artifact).hexdigest() != bundle["artifactSha256"]:
        out.append("blocker.reactor.airgap_update.artifact_digest_mismatch")
    try:
        from cryptography.exceptions import InvalidSignature
        from cryptography.hazmat.primitives.asymmetric.ed25519 import Ed25519PublicKey
        try:
            Ed25519PublicKey.from_public_bytes(public_key).verify(signature, bytes.fromhex(bundle["artifactSha256"]))
        except (InvalidSignature, ValueError):
            out.append("blocker.reactor.airgap_update.signature_invalid")
    except ImportError:                                      # no ed25519 implementation on this node: fail closed
        out.append("blocker.reactor.airgap_update.signature_unverifiable")
    return out


def install_ops_receipt(action: str, bundle: dict, catalog: dict, policy: dict, profile: dict, decided_at: str, receipt_ref: str,
                        rollback_from_bundle_ref: str | None = None, rollback_to_bundle_ref: str | None = None, verification_blockers=(),
                        source_refs=()) -> dict:
    """Fresh install, upgrade or rollback from a bundle: the bundle must be bound to this profile and this policy version, the
    policy is re-validated against the catalogue at install time (a model the policy no longer admits is refused before any
    weights move), and the offline verification (``verify_airgap_bundle``) must have found nothing."""
    _need(action in ("fresh_install", "upgrade", "rollback"), "reactor.install_ops.unknown_action")
    inst = provision_model(catalog, policy, profile, "install" if action == "fresh_install" else "upgrade",
                           [bundle["bundleRef"], f"sha256:{bundle['artifactSha256']}"], decided_at, f"{receipt_ref}.policy_decision",
                           f"{receipt_ref}.model_install", [bundle["bundleRef"], *source_refs])
    blockers = list(verification_blockers)
    if bundle.get("callbackRequired") is not False:
        blockers.append("blocker.reactor.airgap_update.callback_required")
    if not (bundle["nodeProfileRef"] == profile["nodeProfileRef"] and bundle["modelRef"] == profile["modelRef"]):
        blockers.append("blocker.reactor.airgap_update.profile_binding_mismatch")
    if not (bundle["policyRef"] == policy["policyRef"] and bundle["policyVersion"] == policy["version"]):
        blockers.append("blocker.reactor.airgap_update.policy_binding_mismatch")
    if inst["status"] != "installed":
        blockers += ["blocker.reactor.install_ops.policy_revalidation_failed", *(inst["refusal"] or {}).get("blockerRefs", [])]
    blockers = _unique(blockers)
    rb = action == "rollback"
    return {"schemaVersion": "openagents.reactor.install_ops_receipt.v1", "action": action, "blockerRefs": blockers, "bundleRef": bundle["bundleRef"],
            "decidedAt": decided_at, "modelInstallReceiptRef": inst["receiptRef"], "modelRef": profile["modelRef"], "nodeProfileRef": profile["nodeProfileRef"],
            "policyDecisionRef": inst["policyDecisionRef"], "policyRef": policy["policyRef"], "policyVersion": policy["version"], "receiptRef": receipt_ref,
            "rollbackFromBundleRef": rollback_from_bundle_ref if rb else None, "rollbackToBundleRef": (rollback_to_bundle_ref or bundle["bundleRef"]) if rb else None,
            "sourceRefs": _unique([bundle["bundleRef"], bundle["signatureRef"], inst["receiptRef"], inst["policyDecisionRef"], *source_refs]),
            "status": "refused" if blockers else "succeeded",
            "verificationRefs": _unique([bundle["verifierRef"], bundle["publicKeyRef"], bundle["signatureRef"], inst["policyDecisionRef"]])}


# ---------------------------------------------------------------- dog-food run and the improvement ladder (index.ts:449-481, :789-910, :1813-1949)
IMPROVEMENT_STAGES = ("distill_to_fit", "flywheel_training", "harness_evolution")
HARNESS_MECHANISMS = ("context_fidelity", "deliverable_landing", "loop_robustness", "tool_call_repair")


def _policy_is_single_origin_with_lineage(policy: dict) -> bool:
    c = policy["constraints"]
    return bool(c.get("enforceDistillationLineageJurisdiction")) and len(c.get("allowOriginJurisdictions") or []) == 1


def dogfood_run_receipt(profile: dict, policy: dict, install_ops: dict, refused_install_ops: dict, route_receipts: list[dict], metering_receipts: list[dict],
                        workload_ref: str, case_study_ref: str, window_started_at: str, window_ended_at: str, generated_at: str, receipt_ref: str,
                        source_refs=()) -> dict:
    """One measured internal run of a private deployment, from its receipts: the node is a dog-food placement bound to a
    strict policy (one allowed origin jurisdiction, lineage enforced), the served model was installed through install-ops, a
    non-conforming model was REFUSED by the same policy before any pull, every request was routed under that policy and has
    an exact local metering receipt.  Anything else blocks; the receipt never authorises an external claim."""
    b = []
    if profile.get("placement") != "dogfood":
        b.append("blocker.reactor.dogfood.node_not_dogfood_placement")
    if not (profile["policyRef"] == policy["policyRef"] and profile["policyVersion"] == policy["version"]):
        b.append("blocker.reactor.dogfood.profile_policy_binding_mismatch")
    if not _policy_is_single_origin_with_lineage(policy):
        b.append("blocker.reactor.dogfood.strict_single_origin_policy_missing")
    if install_ops["status"] != "succeeded":
        b.append("blocker.reactor.dogfood.install_ops_not_succeeded")
    if not (install_ops["nodeProfileRef"] == profile["nodeProfileRef"] and install_ops["modelRef"] == profile["modelRef"]
            and install_ops["policyRef"] == policy["policyRef"] and install_ops["policyVersion"] == policy["version"]):
        b.append("blocker.reactor.dogfood.install_ops_binding_mismatch")
    if refused_install_ops["status"] != "refused":
        b.append("blocker.reactor.dogfood.nonconforming_pull_not_refused")
    if "blocker.reactor.install_ops.policy_revalidation_failed" not in refused_install_ops["blockerRefs"]:
        b.append("blocker.reactor.dogfood.nonconforming_pull_not_policy_refused")
    if refused_install_ops["modelRef"] == profile["modelRef"]:
        b.append("blocker.reactor.dogfood.refused_model_matches_served_model")
    for r in route_receipts:
        if r["status"] != "routed":
            b += ["blocker.reactor.dogfood.route_not_routed", *r["blockerRefs"]]
        if not (r["nodeProfileRef"] == profile["nodeProfileRef"] and r["policyRef"] == policy["policyRef"] and r["policyVersion"] == policy["version"]):
            b.append("blocker.reactor.dogfood.route_binding_mismatch")
    for m in metering_receipts:
        if not (m["nodeProfileRef"] == profile["nodeProfileRef"] and m["policyRef"] == policy["policyRef"] and m["policyVersion"] == policy["version"]):
            b.append("blocker.reactor.dogfood.metering_binding_mismatch")
        if not (m["measurementState"] == "measured" and m["usageTruth"] == "exact" and m["totalTokens"] is not None):
            b.append("blocker.reactor.dogfood.local_metering_not_exact")
    requests = _unique([r["requestRef"] for r in route_receipts])
    metered = {m["requestRef"] for m in metering_receipts}
    b += [f"blocker.reactor.dogfood.missing_metering:{q}" for q in requests if q not in metered]
    b = _unique(b)
    c = policy["constraints"]
    return {"schemaVersion": "openagents.reactor.dogfood_run_receipt.v1", "blockerRefs": b, "caseStudyWriteupRef": case_study_ref, "externalClaimFlipAllowed": False,
            "externalPilotAuthorized": False, "generatedAt": generated_at, "installOpsReceiptRef": install_ops["receiptRef"],
            "localMeteringReceiptRefs": [m["receiptRef"] for m in metering_receipts], "measuredWindowStartedAt": window_started_at,
            "measuredWindowEndedAt": window_ended_at, "nodeProfileRef": profile["nodeProfileRef"], "placement": profile.get("placement"),
            "policyConstraintRefs": _unique([*[f"constraint.origin_jurisdiction:{j}" for j in c.get("allowOriginJurisdictions") or []],
                                             "constraint.distillation_lineage_jurisdiction:" + ("enforced" if c.get("enforceDistillationLineageJurisdiction") else "not_enforced")]),
            "policyDecisionReceiptRefs": _unique([install_ops["policyDecisionRef"], refused_install_ops["policyDecisionRef"], *[r["policyDecisionRef"] for r in route_receipts]]),
            "policyRef": policy["policyRef"], "policyVersion": policy["version"], "publicSafe": True, "receiptRef": receipt_ref,
            "refusedNonconformingInstallOpsReceiptRef": refused_install_ops["receiptRef"], "refusedNonconformingModelRef": refused_install_ops["modelRef"],
            "requestRefs": requests, "routeDecisionRefs": [r["decisionRef"] for r in route_receipts],
            "sourceRefs": _unique([profile["nodeProfileRef"], policy["policyRef"], install_ops["receiptRef"], refused_install_ops["receiptRef"], case_study_ref,
                                   *[r["decisionRef"] for r in route_receipts], *[m["receiptRef"] for m in metering_receipts], *source_refs]),
            "status": "refused" if b else "completed", "totalMeasuredTokens": sum(m["totalTokens"] or 0 for m in metering_receipts),
            "workloadRef": workload_ref, "workloadTruth": "internal_openagents"}


def improvement_ladder_plan(plan_ref: str, design_doc_ref: str, generated_at: str, stages=IMPROVEMENT_STAGES, source_refs=()) -> dict:
    _need(all(s in IMPROVEMENT_STAGES for s in stages) and len(stages) > 0, "reactor.improvement_ladder.unknown_stage")
    return {"schemaVersion": "openagents.reactor.improvement_ladder_plan_receipt.v1", "boundaryRequirement": "customer_premises_or_regulated_private",
            "capabilityClaimsAuthorized": False, "consentRequired": True, "customerDataUsed": False, "customerWeightsOwnerRequired": True,
            "designDocRef": design_doc_ref, "generatedAt": generated_at, "planRef": plan_ref, "sourceRefs": _unique([design_doc_ref, *source_refs]),
            "stages": list(stages)}


def harness_evolution_receipt(model_ref: str, policy: dict, mechanism_class: str, baseline_harness_ref: str, candidate_harness_ref: str,
                              baseline_score_bps: int, candidate_score_bps: int, acceptance_threshold_bps: int, dataset_snapshot_ref: str,
                              eval_delta_ref: str, receipt_ref: str, generated_at: str, transfer_labels=(), source_refs=()) -> dict:
    """A change of ONE harness mechanism (no weight changes), accepted only when the evaluated gain reaches the threshold."""
    _need(mechanism_class in HARNESS_MECHANISMS, "reactor.harness_evolution.unknown_mechanism")
    delta = int(candidate_score_bps) - int(baseline_score_bps)
    return {"schemaVersion": "openagents.reactor.harness_evolution_dogfood_receipt.v1", "acceptanceThresholdBps": acceptance_threshold_bps,
            "accepted": delta >= acceptance_threshold_bps, "baselineHarnessRef": baseline_harness_ref, "baselineScoreBps": baseline_score_bps,
            "candidateHarnessRef": candidate_harness_ref, "candidateScoreBps": candidate_score_bps, "costObjectiveIncluded": True, "customerDataUsed": False,
            "datasetSnapshotRef": dataset_snapshot_ref, "deltaBps": delta, "evalDeltaRef": eval_delta_ref, "generatedAt": generated_at,
            "mechanismClass": mechanism_class, "modelRef": model_ref, "oneMechanismOnly": True, "optimizerRef": "mutalisk", "policyRef": policy["policyRef"],
            "policyVersion": policy["version"], "receiptRef": receipt_ref, "runnerRef": "psionic",
            "sourceRefs": _unique([baseline_harness_ref, candidate_harness_ref, dataset_snapshot_ref, eval_delta_ref, *source_refs]),
            "stage": "harness_evolution", "transferLabels": list(transfer_labels), "weightChangesAllowed": False, "workloadTruth": "internal_openagents_dogfood"}


def distill_to_fit_receipt(catalog: dict, policy: dict, source_model_ref: str, candidate_artifact_ref: str, distillation_run_ref: str,
                           baseline_quality_bps: int, candidate_quality_bps: int, baseline_cost_micro_usd_per_1k: int, candidate_cost_micro_usd_per_1k: int,
                           max_quality_loss_bps: int, dataset_snapshot_ref: str, input_distribution_capture_ref: str, eval_delta_ref: str,
                           receipt_ref: str, generated_at: str, source_refs=()) -> dict:
    """A smaller model distilled from a served one (``train.distill``): accepted for internal use when the SOURCE model still conforms to
    the policy at this moment, the candidate is cheaper, and the evaluated quality loss stays within the bound.  The router swap stays a
    separate, evaluation-gated step; this receipt never authorises it."""
    pd = resolve_model_policy(catalog, policy, generated_at, f"{receipt_ref}.policy_decision", [source_model_ref, *source_refs])
    md = _decision_for(pd, source_model_ref)
    conforms = md is not None and md["status"] == "conforming"
    _need(baseline_cost_micro_usd_per_1k > 0, "reactor.distill_to_fit.baseline_cost")
    dq = int(candidate_quality_bps) - int(baseline_quality_bps)
    cost_red = round((baseline_cost_micro_usd_per_1k - candidate_cost_micro_usd_per_1k) / baseline_cost_micro_usd_per_1k * 10_000)
    gate = conforms and cost_red > 0 and dq >= -abs(max_quality_loss_bps)
    return {"schemaVersion": "openagents.reactor.distill_to_fit_dogfood_receipt.v1", "acceptedForDogfood": gate,
            "baselineCostPer1kTokensMicrousd": baseline_cost_micro_usd_per_1k, "baselineQualityScoreBps": baseline_quality_bps,
            "candidateArtifactRef": candidate_artifact_ref, "candidateCostPer1kTokensMicrousd": candidate_cost_micro_usd_per_1k,
            "candidateModelClass": "smaller_distilled_model", "candidateQualityScoreBps": candidate_quality_bps, "costReductionBps": cost_red,
            "customerDataUsed": False, "datasetSnapshotRef": dataset_snapshot_ref, "distillationRunRef": distillation_run_ref, "evalDeltaRef": eval_delta_ref,
            "generatedAt": generated_at, "inputDistributionCaptureRef": input_distribution_capture_ref, "policyRef": policy["policyRef"],
            "policyRevalidated": True, "policyVersion": policy["version"], "qualityDeltaBps": dq, "receiptRef": receipt_ref, "routeSwapAuthorized": False,
            "routerSwapGate": "eval_gated_rx3_router", "routerSwapGateStatus": "passed" if gate else "blocked", "runnerRef": "psionic",
            "sourceModelConformsToPolicy": conforms, "sourceModelRef": source_model_ref,
            "sourceRefs": _unique([source_model_ref, candidate_artifact_ref, distillation_run_ref, dataset_snapshot_ref, eval_delta_ref, pd["decisionRef"], *source_refs]),
            "stage": "distill_to_fit", "workloadTruth": "internal_openagents_dogfood"}


def improvement_ladder_dogfood_receipt(plan: dict, harness: dict, distill: dict, receipt_ref: str, generated_at: str, source_refs=()) -> dict:
    b = []
    if "harness_evolution" in plan["stages"] and not harness["accepted"]:
        b.append("blocker.reactor.improvement_ladder.harness_evolution_not_accepted")
    if "distill_to_fit" in plan["stages"] and not distill["acceptedForDogfood"]:
        b.append("blocker.reactor.improvement_ladder.distill_to_fit_not_accepted")
    return {"schemaVersion": "openagents.reactor.improvement_ladder_dogfood_receipt.v1", "blockerRefs": b, "capabilityClaimsAuthorized": False,
            "customerDataUsed": False, "distillToFitReceiptRef": distill["receiptRef"], "externalClaimFlipAllowed": False, "generatedAt": generated_at,
            "harnessEvolutionReceiptRef": harness["receiptRef"], "planRef": plan["planRef"], "receiptRef": receipt_ref,
            "sourceRefs": _unique([plan["planRef"], harness["receiptRef"], distill["receiptRef"], *source_refs]),
            "status": "blocked_for_public_claims" if b else "completed_internal", "workloadTruth": "internal_openagents_dogfood"}
