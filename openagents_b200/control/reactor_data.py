"""The two data-facing contracts of a private deployment: need-to-know retrieval and the data-liberation pipeline.

* ``evaluate_need_to_know_access``: which requested corpus documents a retrieval step (the ``rag_over_corpus`` task class)
  may hand to the model.  Hard rules first: the document must exist, sit in the request's workspace and matter, both of
  which the subject must hold, and the subject needs an allowed role or to be named on the document.  Only documents that
  pass go to the soft check: a logged oracle verdict that the need to know is plausible; a missing verdict denies.  The
  default is deny, the oracle never rescues a hard denial, and the receipt logs refs, never content
  (packages/reactor-contracts/src/index.ts:483-630 types, :1951-1989 hard and soft blockers, :1991-2112 evaluation).
* ``run_data_liberation_pipeline``: move a vendor export (rows of string fields) into the customer's own store through a
  declared mapping: per record class, rows are transformed field by field (``identity`` / ``trim`` / ``lowercase``), a row
  missing a required field fails, one missing an optional field loads as partial; each class gets a verification receipt
  with counts, FNV-1a checksums of source and loaded sets and up to three spot-diff samples; the report is passed /
  partial / failed and never authorises customer engagement (:633-786 types, :2114-2152 checksum and transforms, :2154-2371).
"""
from __future__ import annotations

import json

from .reactor import ContractError, _need, _unique

ROLE_REFS = ("client_admin", "client_member", "external_reviewer", "matter_attorney", "matter_analyst", "operator")
OUTPUT_MODES = ("citation", "source", "summary")
ORACLE_VERDICTS = ("need_to_know_plausible", "not_need_to_know", "not_evaluated")
TRANSFORMS = ("identity", "lowercase", "trim")
ADAPTER_KINDS = ("generic_csv_api_saas_export", "salesforce_contact_export")

NEED_TO_KNOW_RULESET_V1 = {
    "schemaVersion": "openagents.reactor.need_to_know_ruleset.v1", "defaultAction": "deny",
    "hardRuleRefs": ["rule.reactor.need_to_know.workspace_scope", "rule.reactor.need_to_know.matter_scope", "rule.reactor.need_to_know.role_or_user_scope"],
    "oraclePolicyRef": "policy.reactor.need_to_know.oracle.logged_after_hard_rules.v1", "ruleSetRef": "ruleset.reactor.need_to_know.v1",
    "sourceRefs": [], "version": "1",
}


def _check_request(req: dict):
    _need(req.get("outputMode") in OUTPUT_MODES, "request.outputMode")
    for k in ("matterRef", "queryIntentRef", "requestRef", "workspaceRef"):
        _need(isinstance(req.get(k), str) and req[k], f"request.{k}")
    s = req.get("subject") or {}
    _need(isinstance(s.get("subjectUserRef"), str) and s["subjectUserRef"], "request.subject.subjectUserRef")
    _need(all(r in ROLE_REFS for r in s.get("roleRefs", [])), "request.subject.roleRefs")


def _hard_blockers(req: dict, doc: dict) -> list[str]:
    s = req["subject"]
    out = []
    if not (doc["workspaceRef"] in s.get("workspaceRefs", []) and req["workspaceRef"] == doc["workspaceRef"]):
        out.append("blocker.reactor.need_to_know.workspace_scope_mismatch")
    if not (doc["matterRef"] in s.get("matterRefs", []) and req["matterRef"] == doc["matterRef"]):
        out.append("blocker.reactor.need_to_know.matter_scope_mismatch")
    if not (set(s.get("roleRefs", [])) & set(doc.get("allowedRoleRefs", [])) or s["subjectUserRef"] in doc.get("allowedUserRefs", [])):
        out.append("blocker.reactor.need_to_know.role_or_user_scope_missing")
    return out


def evaluate_need_to_know_access(rule_set: dict, request: dict, documents: list[dict], decided_at: str, receipt_ref: str,
                                 oracle_verdicts=(), source_refs=()) -> dict:
    _need(rule_set.get("schemaVersion") == "openagents.reactor.need_to_know_ruleset.v1" and rule_set.get("defaultAction") == "deny", "ruleSet")
    _check_request(request)
    verdicts = {}
    for v in oracle_verdicts:
        _need(v.get("verdict") in ORACLE_VERDICTS, "oracleVerdict.verdict")
        verdicts[v["documentRef"]] = v
    by_ref = {d["documentRef"]: d for d in documents}
    decisions = []
    for ref in request.get("requestedDocumentRefs", []):
        doc = by_ref.get(ref)
        base = {"decisionRef": f"{receipt_ref}.decision.{ref}", "documentRef": ref, "hardRuleRefs": list(rule_set["hardRuleRefs"])}
        if doc is None:
            decisions.append({**base, "blockerRefs": ["blocker.reactor.need_to_know.document_not_found"], "citationRefs": [], "hardDecisionStatus": "failed",
                              "oracleDecisionStatus": "skipped_hard_denied", "oracleVerdictRef": None,
                              "reasonRefs": ["reason.reactor.need_to_know.document_not_found"], "status": "denied_hard_rule"})
            continue
        hard = _hard_blockers(request, doc)
        v = verdicts.get(ref)
        if hard:
            decisions.append({**base, "blockerRefs": hard, "citationRefs": [], "hardDecisionStatus": "failed", "oracleDecisionStatus": "skipped_hard_denied",
                              "oracleVerdictRef": v["verdictRef"] if v else None, "reasonRefs": hard, "status": "denied_hard_rule"})
            continue
        if v is None:
            soft = ["blocker.reactor.need_to_know.oracle_verdict_missing"]
        elif v["verdict"] == "need_to_know_plausible":
            soft = []
        else:
            soft = ["blocker.reactor.need_to_know.oracle_not_plausible", *v.get("reasonRefs", [])]
        decisions.append({**base, "blockerRefs": soft, "citationRefs": [] if soft else list(doc.get("citationRefs", [])), "hardDecisionStatus": "passed",
                          "oracleDecisionStatus": "failed" if soft else "passed", "oracleVerdictRef": v["verdictRef"] if v else None,
                          "reasonRefs": soft or ["reason.reactor.need_to_know.allowed"], "status": "denied_soft_oracle" if soft else "allowed"})
    allowed = [d["documentRef"] for d in decisions if d["status"] == "allowed"]
    denied = [d["documentRef"] for d in decisions if d["status"] != "allowed"]
    return {"schemaVersion": "openagents.reactor.corpus_access_decision_receipt.v1", "decidedAt": decided_at,
            "deniedCitationRefs": _unique([c for r in denied if r in by_ref for c in by_ref[r].get("citationRefs", [])]), "deniedDocumentRefs": denied,
            "documentDecisions": decisions, "generatedSummaryContentLogged": False, "matterRef": request["matterRef"], "oracleAppliedAfterHardRules": True,
            "oracleVerdictRefs": _unique([v["verdictRef"] for v in verdicts.values()]), "outputMode": request["outputMode"],
            "queryIntentRef": request["queryIntentRef"], "rawDocumentContentLogged": False, "receiptRef": receipt_ref,
            "requestedDocumentRefs": list(request.get("requestedDocumentRefs", [])), "ruleSetRef": rule_set["ruleSetRef"], "ruleSetVersion": rule_set["version"],
            "selectedCitationRefs": _unique([c for d in decisions for c in d["citationRefs"]]), "selectedDocumentRefs": allowed,
            "sourceRefs": _unique([rule_set["ruleSetRef"], request["requestRef"], *[d["decisionRef"] for d in decisions], *source_refs]),
            "subjectUserRef": request["subject"]["subjectUserRef"], "workspaceRef": request["workspaceRef"]}


# ---------------------------------------------------------------- data liberation
def stable_checksum(value) -> str:
    """FNV-1a (32 bit) over the canonical JSON (sorted keys, no spaces) of ``value``, by UTF-16 code unit like the reference."""
    s = json.dumps(value, sort_keys=True, separators=(",", ":"), ensure_ascii=False)
    h = 0x811C9DC5
    data = s.encode("utf-16-le")
    for i in range(0, len(data), 2):
        h ^= data[i] | (data[i + 1] << 8)
        h = (h * 0x01000193) & 0xFFFFFFFF
    return f"fnv1a32:{h:08x}"


def apply_transforms(value: str, transform_refs) -> str:
    for t in transform_refs:
        if t not in TRANSFORMS:
            raise ContractError(f"fieldMapping.transformRefs: {t!r}")
        value = value.lower() if t == "lowercase" else value.strip() if t == "trim" else value
    return value


def run_data_liberation_pipeline(adapter: dict, export_rows: list[dict], customer_store_ref: str, generated_at: str, report_ref: str, source_refs=()) -> dict:
    _need(adapter.get("schemaVersion") == "openagents.reactor.data_liberation_adapter_config.v1", "adapter.schemaVersion")
    _need(adapter.get("adapterKind") in ADAPTER_KINDS and adapter.get("exportTransport") in ("api_json", "csv_file"), "adapter.kind")
    _need(adapter.get("customerDataAllowed") is False and adapter.get("fixtureTruth") == "synthetic_public_fixture", "adapter.fixtureTruth")
    for r in export_rows:
        _need(isinstance(r.get("fields"), dict) and all(isinstance(v, str) for v in r["fields"].values()), "exportRow.fields")
    receipts = []
    for m in adapter["recordClassMappings"]:
        rows = [r for r in export_rows if r["sourceRecordTypeRef"] == m["sourceRecordTypeRef"]]
        loaded, failed, partial, reasons = [], [], [], []
        for r in rows:
            values, miss_req, miss_opt = {}, [], []
            for fm in m["fieldMappings"]:
                raw = r["fields"].get(fm["sourceField"])
                if raw is None or not raw.strip():
                    (miss_req if fm["required"] else miss_opt).append(fm["sourceField"])
                    continue
                values[fm["targetField"]] = apply_transforms(raw, fm["transformRefs"])
            if miss_req:
                failed.append(r["rowRef"])
                reasons += [f"reason.reactor.data_liberation.missing_required_field:{f}" for f in miss_req]
                continue
            if miss_opt:
                partial.append(r["rowRef"])
                reasons += [f"reason.reactor.data_liberation.missing_optional_field:{f}" for f in miss_opt]
            loaded.append({"recordClassRef": m["recordClassRef"], "sourceRowRef": r["rowRef"],
                           "targetRecordRef": f"{customer_store_ref}.{m['recordClassRef']}.{r['rowRef']}", "values": values})
        status = "passed" if not failed and not partial else ("failed" if not loaded else "partial")
        blockers = [] if status == "passed" else _unique([f"blocker.reactor.data_liberation.record_class_{status}", *reasons])
        src = {r["rowRef"]: r for r in rows}
        samples = []
        for rec in loaded[:3]:
            checks = []
            for fm in m["fieldMappings"]:
                if fm["targetField"] not in rec["values"]:
                    continue
                a = stable_checksum(apply_transforms(src[rec["sourceRowRef"]]["fields"].get(fm["sourceField"], ""), fm["transformRefs"]))
                b = stable_checksum(rec["values"][fm["targetField"]])
                checks.append({"loadedValueChecksum": b, "matched": a == b, "sourceValueChecksum": a, "targetField": fm["targetField"]})
            samples.append({"fieldChecks": checks, "sampleRef": f"{report_ref}.sample.{rec['sourceRowRef']}", "sourceRowRef": rec["sourceRowRef"],
                            "targetRecordRef": rec["targetRecordRef"]})
        receipts.append({"schemaVersion": "openagents.reactor.data_liberation_record_class_verification_receipt.v1", "adapterRef": adapter["adapterRef"],
                         "blockerRefs": blockers, "customerControlledStoreRef": customer_store_ref, "customerDataLogged": False, "failedRowCount": len(failed),
                         "failedRowRefs": failed, "generatedAt": generated_at, "loadedChecksum": stable_checksum(loaded), "loadedRowCount": len(loaded),
                         "partialRowCount": len(partial), "partialRowRefs": partial, "receiptRef": f"{report_ref}.receipt.{m['recordClassRef']}",
                         "recordClassRef": m["recordClassRef"], "schemaMappingRef": m["schemaMappingRef"],
                         "sourceChecksum": stable_checksum([{"fields": r["fields"], "rowRef": r["rowRef"], "sourceRecordTypeRef": r["sourceRecordTypeRef"]} for r in rows]),
                         "sourceRefs": _unique([adapter["adapterRef"], m["schemaMappingRef"], *source_refs]), "sourceRowCount": len(rows),
                         "spotDiffSamples": samples, "status": status, "targetSchemaRef": m["targetSchemaRef"], "transformedRowCount": len(loaded)})
    status = "passed" if all(r["status"] == "passed" for r in receipts) else ("partial" if any(r["status"] != "failed" for r in receipts) else "failed")
    blockers = [] if status == "passed" else _unique([f"blocker.reactor.data_liberation.pipeline_{status}", *[b for r in receipts for b in r["blockerRefs"]]])
    return {"schemaVersion": "openagents.reactor.data_liberation_pipeline_report.v1", "adapterRefs": [adapter["adapterRef"]], "blockerRefs": blockers,
            "customerControlledStoreRef": customer_store_ref, "customerDataLogged": False, "customerEngagementAuthorized": False,
            "failedRowCount": sum(r["failedRowCount"] for r in receipts), "fixtureTruth": adapter["fixtureTruth"], "generatedAt": generated_at,
            "loadedRowCount": sum(r["loadedRowCount"] for r in receipts), "packageCopyAuthorized": False,
            "partialRowCount": sum(r["partialRowCount"] for r in receipts), "recordClassRefs": [r["recordClassRef"] for r in receipts], "reportRef": report_ref,
            "sourceRefs": _unique([adapter["adapterRef"], *[r["receiptRef"] for r in receipts], *source_refs]),
            "sourceRowCount": sum(r["sourceRowCount"] for r in receipts), "status": status,
            "verificationReceiptRefs": [r["receiptRef"] for r in receipts], "verificationReceipts": receipts}
