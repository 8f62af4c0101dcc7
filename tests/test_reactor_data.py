"""Need-to-know retrieval decisions and the data-liberation pipeline."""
import pytest

from openagents_b200.control import reactor_data as rd
from openagents_b200.control.reactor import ContractError

DOCS = [{"documentRef": "doc.a", "workspaceRef": "ws.1", "matterRef": "m.1", "allowedRoleRefs": ["matter_attorney"], "allowedUserRefs": [], "citationRefs": ["cite.a1", "cite.a2"]},
        {"documentRef": "doc.b", "workspaceRef": "ws.1", "matterRef": "m.2", "allowedRoleRefs": ["matter_attorney"], "allowedUserRefs": [], "citationRefs": ["cite.b"]},
        {"documentRef": "doc.c", "workspaceRef": "ws.1", "matterRef": "m.1", "allowedRoleRefs": ["client_admin"], "allowedUserRefs": ["user.7"], "citationRefs": ["cite.c"]},
        {"documentRef": "doc.d", "workspaceRef": "ws.1", "matterRef": "m.1", "allowedRoleRefs": ["matter_attorney"], "allowedUserRefs": [], "citationRefs": ["cite.d"]}]


def req(**kw):
    base = {"matterRef": "m.1", "outputMode": "citation", "queryIntentRef": "intent.q1", "requestRef": "req.1", "workspaceRef": "ws.1",
            "requestedDocumentRefs": ["doc.a", "doc.b", "doc.c", "doc.d", "doc.zz"],
            "subject": {"matterRefs": ["m.1"], "roleRefs": ["matter_attorney"], "subjectUserRef": "user.7", "workspaceRefs": ["ws.1"]}}
    return {**base, **kw}


def verdict(doc, kind, reasons=()):
    return {"documentRef": doc, "loggedAt": "t", "modelRef": "model.oracle", "reasonRefs": list(reasons), "requestRef": "req.1", "verdict": kind, "verdictRef": "verdict." + doc}


def test_hard_rules_then_oracle_default_deny():
    vs = [verdict("doc.a", "need_to_know_plausible"), verdict("doc.b", "need_to_know_plausible"), verdict("doc.c", "not_need_to_know", ["reason.unrelated"])]
    r = rd.evaluate_need_to_know_access(rd.NEED_TO_KNOW_RULESET_V1, req(), DOCS, "2026-01-01T00:00:00Z", "receipt.n2k.1", vs)
    by = {d["documentRef"]: d for d in r["documentDecisions"]}
    assert by["doc.a"]["status"] == "allowed" and by["doc.a"]["citationRefs"] == ["cite.a1", "cite.a2"]
    assert by["doc.b"]["status"] == "denied_hard_rule" and by["doc.b"]["oracleDecisionStatus"] == "skipped_hard_denied"        # a plausible verdict rescues nothing
    assert by["doc.b"]["blockerRefs"] == ["blocker.reactor.need_to_know.matter_scope_mismatch"]
    assert by["doc.c"]["status"] == "denied_soft_oracle" and by["doc.c"]["hardDecisionStatus"] == "passed"                      # named user passes the hard rule
    assert by["doc.c"]["blockerRefs"] == ["blocker.reactor.need_to_know.oracle_not_plausible", "reason.unrelated"]
    assert by["doc.d"]["status"] == "denied_soft_oracle" and by["doc.d"]["blockerRefs"] == ["blocker.reactor.need_to_know.oracle_verdict_missing"]
    assert by["doc.zz"]["status"] == "denied_hard_rule" and by["doc.zz"]["blockerRefs"] == ["blocker.reactor.need_to_know.document_not_found"]
    assert r["selectedDocumentRefs"] == ["doc.a"] and r["selectedCitationRefs"] == ["cite.a1", "cite.a2"]
    assert r["deniedCitationRefs"] == ["cite.b", "cite.c", "cite.d"] and r["rawDocumentContentLogged"] is False and r["oracleAppliedAfterHardRules"] is True
    outsider = req(subject={"matterRefs": ["m.1"], "roleRefs": ["external_reviewer"], "subjectUserRef": "user.9", "workspaceRefs": ["ws.2"]})
    r2 = rd.evaluate_need_to_know_access(rd.NEED_TO_KNOW_RULESET_V1, outsider, DOCS, "t", "receipt.n2k.2", vs)
    assert r2["selectedDocumentRefs"] == [] and set(r2["documentDecisions"][0]["blockerRefs"]) == {
        "blocker.reactor.need_to_know.workspace_scope_mismatch", "blocker.reactor.need_to_know.role_or_user_scope_missing"}
    with pytest.raises(ContractError):
        rd.evaluate_need_to_know_access({**rd.NEED_TO_KNOW_RULESET_V1, "defaultAction": "allow"}, req(), DOCS, "t", "r")
    with pytest.raises(ContractError):
        rd.evaluate_need_to_know_access(rd.NEED_TO_KNOW_RULESET_V1, req(outputMode="raw"), DOCS, "t", "r")


ADAPTER = {"schemaVersion": "openagents.reactor.data_liberation_adapter_config.v1", "adapterKind": "generic_csv_api_saas_export", "adapterRef": "adapter.crm.csv",
           "customerDataAllowed": False, "exportTransport": "csv_file", "fixtureTruth": "synthetic_public_fixture", "sourceRefs": [], "vendorRef": "vendor.crm", "version": "1",
           "recordClassMappings": [
               {"recordClassRef": "contact", "schemaMappingRef": "mapping.contact.v1", "sourceRecordTypeRef": "Contact", "targetSchemaRef": "schema.contact.v1",
                "fieldMappings": [{"mappingRef": "m.email", "required": True, "sourceField": "Email", "targetField": "email", "transformRefs": ["trim", "lowercase"]},
                                  {"mappingRef": "m.name", "required": True, "sourceField": "Name", "targetField": "name", "transformRefs": ["trim"]},
                                  {"mappingRef": "m.phone", "required": False, "sourceField": "Phone", "targetField": "phone", "transformRefs": ["identity"]}]},
               {"recordClassRef": "account", "schemaMappingRef": "mapping.account.v1", "sourceRecordTypeRef": "Account", "targetSchemaRef": "schema.account.v1",
                "fieldMappings": [{"mappingRef": "m.acct", "required": True, "sourceField": "AccountName", "targetField": "name", "transformRefs": ["trim"]}]}]}
ROWS = [{"rowRef": "row.1", "sourceRecordTypeRef": "Contact", "fields": {"Email": " Ada@Example.ORG ", "Name": " Ada ", "Phone": "555"}},
        {"rowRef": "row.2", "sourceRecordTypeRef": "Contact", "fields": {"Email": "bob@example.org", "Name": "Bob", "Phone": "  "}},
        {"rowRef": "row.3", "sourceRecordTypeRef": "Contact", "fields": {"Name": "No Mail"}},
        {"rowRef": "row.4", "sourceRecordTypeRef": "Account", "fields": {"AccountName": "Acme"}}]


def test_pipeline_loads_marks_partial_and_failed_rows():
    rep = rd.run_data_liberation_pipeline(ADAPTER, ROWS, "store.customer", "2026-01-01T00:00:00Z", "report.dl.1")
    contact, account = rep["verificationReceipts"]
    assert contact["status"] == "partial" and contact["loadedRowCount"] == 2 and contact["failedRowRefs"] == ["row.3"] and contact["partialRowRefs"] == ["row.2"]
    assert contact["blockerRefs"] == ["blocker.reactor.data_liberation.record_class_partial", "reason.reactor.data_liberation.missing_optional_field:Phone",
                                      "reason.reactor.data_liberation.missing_required_field:Email"]
    s = contact["spotDiffSamples"][0]
    assert s["targetRecordRef"] == "store.customer.contact.row.1" and all(c["matched"] for c in s["fieldChecks"]) and [c["targetField"] for c in s["fieldChecks"]] == ["email", "name", "phone"]
    assert s["fieldChecks"][0]["loadedValueChecksum"] == rd.stable_checksum("ada@example.org")
    assert account["status"] == "passed" and account["blockerRefs"] == []
    assert rep["status"] == "partial" and rep["loadedRowCount"] == 3 and rep["failedRowCount"] == 1 and rep["sourceRowCount"] == 4
    assert rep["customerEngagementAuthorized"] is False and rep["blockerRefs"][0] == "blocker.reactor.data_liberation.pipeline_partial"
    ok = rd.run_data_liberation_pipeline(ADAPTER, [ROWS[0], ROWS[3]], "store.customer", "t", "report.dl.2")
    assert ok["status"] == "passed" and ok["blockerRefs"] == []
    bad = rd.run_data_liberation_pipeline({**ADAPTER, "recordClassMappings": ADAPTER["recordClassMappings"][:1]}, [ROWS[2]], "store.customer", "t", "report.dl.3")
    assert bad["status"] == "failed" and bad["blockerRefs"][0] == "blocker.reactor.data_liberation.pipeline_failed"
    with pytest.raises(ContractError):
        rd.run_data_liberation_pipeline({**ADAPTER, "customerDataAllowed": True}, ROWS, "s", "t", "r")


def test_checksum_is_fnv1a_over_canonical_json():
    assert rd.stable_checksum("") == "fnv1a32:" + format(((((0x811C9DC5 ^ 0x22) * 0x01000193) & 0xFFFFFFFF) ^ 0x22) * 0x01000193 & 0xFFFFFFFF, "08x")
    assert rd.stable_checksum({"b": 1, "a": [2, {"d": 3, "c": 4}]}) == rd.stable_checksum({"a": [2, {"c": 4, "d": 3}], "b": 1})
    assert rd.stable_checksum("a") != rd.stable_checksum("b") and rd.apply_transforms("  MiXed ", ["trim", "lowercase"]) == "mixed"
