"""What a contributor node consumes from, and reports about, the ML stack.

* GEPA candidate manifest (``psionic.probe_gepa_candidate_manifest.v1``): a text-bundle optimisation
  candidate (prompts, playbooks, tool-menu policy) with per-component hashes, optimizer and promotion
  states and trace digests.  It is not neural-network training; the node only decodes and checks it.
  Reference: apps/pylon/packages/runtime/src/benchmark/candidate-execution.ts:20 (schema version),
  :71-93 (fields), :127-145 (decoder), :216-257 (rules), :449-477 (component hashes), :479-498 (unsafe text).
* Host inventory: accelerators found by running ``nvidia-smi --query-gpu=name,memory.total``, and the
  model-server backend row with its blocker refs (ready / configured / missing).
  Reference: packages/pylon-core/src/shared/inventory.ts:143-150 (backend row), :240-258 (probe), :287-289 (env flag).
* Model registry: which GGUF architectures the engine admits for GPU serving, and the exact chat-template
  digests it will render (docs/muse/muse-glimmer.md:118-126).
"""
from __future__ import annotations

import hashlib
import os
import re
import shutil
import subprocess

GEPA_SCHEMA = "psionic.probe_gepa_candidate_manifest.v1"
GEPA_PROBE_IMPORT_SCHEMA = "probe.prompt_candidate_import.v1"
GEPA_CLOUD_IMPORT_SCHEMA = "benchmark_cloud.probe_candidate_import.v1"
_TEXT_FIELDS = ("probe_system_prompt", "terminal_bench_global_playbook", "signature_selection_policy", "tool_menu_policy",
                "patch_and_test_policy", "closeout_policy")
_UNSAFE = ("access_token", "refresh_token", "bearer ", "mdk_mnemonic", "wallet_mnemonic", "private-repo://", "bypass_release_gate",
           "ignore_release_gate", "disable_release_gate", "public_claim_upgrade_authority", "request_new_runtime_authority",
           "new_runtime_authority", "grant_runtime_authority")
_STATES = {"optimizer_acceptance_state": ("draft", "optimizer_accepted", "rejected"), "policy_gate_state": ("pending", "passed", "failed", "blocked"),
           "promotion_state": ("draft", "optimizer_accepted", "shadow", "release_candidate", "active", "rejected", "reverted"),
           "runtime_promotion_state": ("not_promoted", "shadow", "release_candidate", "active", "reverted")}


class CandidateManifestError(ValueError):
    def __init__(self, path: str, reason: str):
        super().__init__(f"{path}: {reason}")
        self.path, self.reason = path, reason


def stable_sha256(label: str, value: str) -> str:
    return "sha256:" + hashlib.sha256(label.encode() + b"\0" + value.encode()).hexdigest()


def short_hash(h: str) -> str:
    return h[7:23] if h.startswith("sha256:") else h[:16]


def component_hashes(components: dict) -> dict:
    out = {k: stable_sha256(k, components[k]) for k in _TEXT_FIELDS}
    out["failure_family_playbooks"] = {f: stable_sha256(f"failure_family_playbook:{f}", t)
                                       for f, t in sorted(components["failure_family_playbooks"].items())}
    return out


def unsafe_candidate_text(text: str) -> bool:
    t = text.lower()
    return any(n in t for n in _UNSAFE) or t.startswith("sk-") or " sk-" in t


def decode_gepa_candidate_manifest(m) -> dict:
    """Checks shape, states, hash-derived id, the safety boundary, component text and component hashes; returns the manifest."""
    P = "gepaCandidateManifest"
    if not isinstance(m, dict):
        raise CandidateManifestError(P, "must be an object")
    if m.get("schema_version") != GEPA_SCHEMA:
        raise CandidateManifestError(f"{P}.schema_version", f"must be {GEPA_SCHEMA}")
    for k in ("campaign_id", "candidate_hash", "candidate_id", "manifest_hash", "optimizer_run_id"):
        if not isinstance(m.get(k), str):
            raise CandidateManifestError(f"{P}.{k}", "must be a string")
    for k in ("candidate_id", "candidate_hash", "manifest_hash"):
        if not m[k].strip():
            raise CandidateManifestError(f"{P}.{k}", "must be non-empty")
    for k, allowed in _STATES.items():
        if m.get(k) not in allowed:
            raise CandidateManifestError(f"{P}.{k}", f"must be one of {allowed}")
    for k in ("split_refs", "target_suites", "target_failure_families", "evaluation_trace_digests", "training_trace_digests"):
        if not isinstance(m.get(k), list) or not all(isinstance(x, str) for x in m[k]):
            raise CandidateManifestError(f"{P}.{k}", "must be an array of strings")
    for k in ("split_refs", "target_suites", "target_failure_families"):
        if not m[k]:
            raise CandidateManifestError(f"{P}.{k}", "must be non-empty")
    for k in ("probe_import", "benchmark_cloud_import", "safety_boundary", "components"):
        if not isinstance(m.get(k), dict):
            raise CandidateManifestError(f"{P}.{k}", "must be an object")
    pi, ci, sb = m["probe_import"], m["benchmark_cloud_import"], m["safety_boundary"]
    for k in ("blueprint_candidate_ref", "loop_policy_candidate_ref", "prompt_candidate_ref", "tool_menu_candidate_ref"):
        if not isinstance(pi.get(k), str) or not pi[k].strip():
            raise CandidateManifestError(f"{P}.probe_import.{k}", "must be a non-empty string")
    if pi.get("schema_version") != GEPA_PROBE_IMPORT_SCHEMA or ci.get("schema_version") != GEPA_CLOUD_IMPORT_SCHEMA:
        raise CandidateManifestError(f"{P}.probe_import", "import blocks carry their own schema versions")
    if not ci.get("artifact_contract_refs"):
        raise CandidateManifestError(f"{P}.benchmark_cloud_import.artifact_contract_refs", "must be non-empty")
    if not m["candidate_hash"].startswith("sha256:"):
        raise CandidateManifestError(f"{P}.candidate_hash", "must be a sha256 content hash ref")
    if m["candidate_id"] != f"probe_gepa_candidate.{short_hash(m['candidate_hash'])}":
        raise CandidateManifestError(f"{P}.candidate_id", "must match candidate hash prefix")
    if not sb.get("no_new_runtime_authority") or not sb.get("inherited_runtime_authority_refs"):
        raise CandidateManifestError(f"{P}.safety_boundary", "must inherit runtime authority from the Probe assignment")
    if sb.get("public_claim_upgrade_authority"):
        raise CandidateManifestError(f"{P}.safety_boundary.public_claim_upgrade_authority", "candidate text cannot carry public-claim upgrade authority")
    comp = m["components"]
    fam = comp.get("failure_family_playbooks")
    if not isinstance(fam, dict) or not fam:
        raise CandidateManifestError(f"{P}.components.failure_family_playbooks", "must be non-empty")
    for field, text in [(k, comp.get(k)) for k in _TEXT_FIELDS] + [(f"failure_family_playbooks.{f}", t) for f, t in fam.items()]:
        if not isinstance(text, str) or not text.strip():
            raise CandidateManifestError(f"{P}.components.{field}", "must be non-empty")
        if unsafe_candidate_text(text):
            raise CandidateManifestError(f"{P}.components.{field}", "contains authority-bypass, credential, private-repo, or release-gate bypass text")
    if component_hashes(comp) != m.get("component_hashes"):
        raise CandidateManifestError(f"{P}.component_hashes", "must match component text hashes")
    return m


def candidate_refs(m: dict) -> dict:
    pi = m["probe_import"]
    return {"blueprintCandidateRef": pi["blueprint_candidate_ref"], "loopPolicyCandidateRef": pi["loop_policy_candidate_ref"],
            "promptCandidateRef": pi["prompt_candidate_ref"], "toolMenuCandidateRef": pi["tool_menu_candidate_ref"]}


def check_projected_tools(projected, required, allowed, denied=()):
    """A candidate's tool menu must contain the required refs and stay inside allowed minus denied."""
    for r in required:
        if r not in projected:
            raise CandidateManifestError("projectedToolRefs", "projected tool menu must include required tool refs")
    for r in projected:
        if r not in allowed:
            raise CandidateManifestError("projectedToolRefs", "projected tool menu can only include allowed tool refs")
        if r in denied:
            raise CandidateManifestError("projectedToolRefs", "projected tool menu cannot include denied tool refs")


# ---------------------------------------------------------------- inventory
def _ref_segment(s: str) -> str:
    return re.sub(r"[^a-z0-9]+", "_", s.lower()).strip("_") or "unknown"


def parse_nvidia_smi(csv_text: str) -> list[dict]:
    """Rows of ``name, memory.total`` (MiB, no units) -> accelerator records."""
    out = []
    for line in csv_text.splitlines():
        if not line.strip():
            continue
        name, _, mem = line.rpartition(",")
        try:
            vram = int(float(mem.strip())) * 1024 * 1024
        except ValueError:
            vram = None
        out.append({"kind": "nvidia_cuda", "modelRef": f"accelerator.{_ref_segment(name.strip())}", "vramBytes": vram, "blockerRefs": []})
    return out


def discover_accelerators(run=None) -> list[dict]:
    """Reads only: never changes a GPU setting."""
    if run is None:
        if shutil.which("nvidia-smi") is None:
            return []
        def run():
            p = subprocess.run(["nvidia-smi", "--query-gpu=name,memory.total", "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=20)
            return p.stdout if p.returncode == 0 else ""
    try:
        return parse_nvidia_smi(run())
    except (OSError, subprocess.SubprocessError):
        return []


def model_server_backend_row(env=None, ready: bool = False, model_refs=()) -> dict:
    env = os.environ if env is None else env
    configured = bool(env.get("PYLON_PSIONIC_BASE_URL") or env.get("PROBE_PSIONIC_BASE_URL") or env.get("B200_SERVE_BASE_URL"))
    blockers = [] if ready else (["blocker.psionic_qwen35.qwen35_model_missing"] if configured else ["blocker.psionic_qwen35.connector_unconfigured"])
    return {"backendRef": "backend.psionic.qwen35", "state": "ready" if ready else "configured" if configured else "missing",
            "modelRef": (model_refs[0] if model_refs else None), "blockerRefs": blockers}


def host_inventory(env=None, run=None, ready: bool = False, model_refs=()) -> dict:
    accs = discover_accelerators(run)
    return {"cpuCores": os.cpu_count(), "accelerators": accs,
            "acceleratorBlockerRefs": [] if accs else ["blocker.inventory.accelerator_unproven"],
            "backends": [model_server_backend_row(env, ready, model_refs)]}


# ---------------------------------------------------------------- model registry and chat-template allowlist
ADMITTED_ARCHITECTURES = {"llama": "dense", "qwen2": "dense", "qwen3": "dense", "qwen35": "dense", "gemma3": "dense", "gemma4": "dense",
                          "gpt-oss": "moe", "gpt2": "dense"}


def template_digest(template: str) -> str:
    return hashlib.sha256(template.encode()).hexdigest()


def template_admitted(template: str, extra_digests=()) -> bool:
    """Whether a GGUF chat template may be rendered by the server: its digest must be on the allowlist: the digests
    given, plus those in ``B200_CHAT_TEMPLATE_ALLOW`` (comma-separated sha256 hex).  A template is code that runs on
    every request, so an unknown one is never rendered; the server then uses its built-in template."""
    import os
    allowed = set(extra_digests) | {d.strip() for d in os.environ.get("B200_CHAT_TEMPLATE_ALLOW", "").split(",") if d.strip()}
    return template_digest(template) in allowed


class ModelRegistry:
    """Admission of a GGUF for GPU serving: a known ``general.architecture`` and, when the file carries a
    chat template, a digest on the allowlist (an unknown template is refused rather than rendered approximately)."""

    def __init__(self, allowed_template_digests=()):
        self.allowed = set(allowed_template_digests)

    def allow_template(self, template: str) -> str:
        d = template_digest(template)
        self.allowed.add(d)
        return d

    def admit(self, metadata: dict) -> dict:
        arch = metadata.get("general.architecture")
        if arch not in ADMITTED_ARCHITECTURES:
            return {"admitted": False, "reason": "unsupported_architecture", "architecture": arch}
        tpl = metadata.get("tokenizer.chat_template")
        if tpl is not None and template_digest(tpl) not in self.allowed:
            return {"admitted": False, "reason": "chat_template_digest_not_allowlisted", "architecture": arch, "templateDigest": template_digest(tpl)}
        return {"admitted": True, "architecture": arch, "family": ADMITTED_ARCHITECTURES[arch], "templateDigest": template_digest(tpl) if tpl else None}


# ---------------------------------------------------------------- assignment leases that ask for local inference
# A lease may carry local-inference requirements {workClass, mode, requiredModelRef?, receiptRefs?}.  The runner admits
# the lease only if a served model row satisfies the mode, and attaches the backend ref, the selected model ref and the
# lease's receipt refs to the closeout.  In the reference the selector is an archived stub that always refuses with
# ``blocker.psionic_qwen35.archived_to_backroom``; here it is live against the rows the model server reports.
# Reference: apps/pylon/src/assignment.ts:112-119 (requirements), :1334-1347 (admission), :2437-2461 (closeout refs);
# apps/pylon/packages/runtime/src/backends/psionic-qwen/model-admission.ts:1-24, contract.ts:1-6.
BACKEND_REF = "backend.psionic.qwen35"
MODEL_REFS = {"small": "model.psionic.qwen35.0_8b.q8_0", "large": "model.psionic.qwen35.2b.q8_0"}
TASK_MODES = ("coding_agent", "requires_2b")


def admission_from_model_rows(rows) -> dict:
    """rows: [{modelRef, ready}] as listed by the model server (``/v1/models``).  The listing comes over HTTP: anything that is
    not a row with a string ``modelRef`` is dropped rather than trusted."""
    rows = [r for r in rows if isinstance(r, dict) and isinstance(r.get("modelRef"), str) and r["modelRef"]] if isinstance(rows, (list, tuple)) else []
    observed = [r["modelRef"] for r in rows]
    admitted = [r["modelRef"] for r in rows if r.get("ready", True) is True]
    return {"rows": list(rows), "observedModelRefs": observed, "admittedModelRefs": admitted,
            "blockerRefs": [] if admitted else ["blocker.psionic_qwen35.qwen35_model_missing"]}


def select_model(admission: dict, mode: str) -> dict:
    if mode not in TASK_MODES:
        raise ValueError(f"mode must be one of {TASK_MODES}")
    if admission["blockerRefs"]:
        return {"admitted": False, "selectedModelRef": None, "blockerRefs": list(admission["blockerRefs"])}
    adm = admission["admittedModelRefs"]
    if mode == "requires_2b":
        if MODEL_REFS["large"] not in adm:
            return {"admitted": False, "selectedModelRef": None, "blockerRefs": ["blocker.psionic_qwen35.model_2b_missing"]}
        return {"admitted": True, "selectedModelRef": MODEL_REFS["large"], "blockerRefs": []}
    pick = MODEL_REFS["large"] if MODEL_REFS["large"] in adm else adm[0]       # the stronger row when it is there
    return {"admitted": True, "selectedModelRef": pick, "blockerRefs": []}


def admit_inference_lease(requirements: dict, admission: dict) -> dict:
    sel = select_model(admission, requirements["mode"])
    blockers = list(sel["blockerRefs"])
    need = requirements.get("requiredModelRef")
    if need and sel["selectedModelRef"] != need:
        blockers.append("blocker.psionic_qwen35.model_2b_missing" if need == MODEL_REFS["large"] else "blocker.psionic_qwen35.required_model_missing")
    return {"admitted": not blockers, "selectedModelRef": sel["selectedModelRef"], "blockerRefs": sorted(set(blockers))}


def closeout_receipt_refs(requirements: dict | None, admission: dict) -> list[str]:
    if not requirements:
        return []
    refs = [BACKEND_REF] + list(requirements.get("receiptRefs") or [])
    sel = select_model(admission, requirements["mode"])["selectedModelRef"]
    return list(dict.fromkeys(refs + ([sel] if sel else [])))
