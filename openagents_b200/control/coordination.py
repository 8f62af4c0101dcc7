"""Coordination records around a training network and a serving mesh.

* NIP-TRN events: the Nostr-side records of a training network.  They carry identifiers, counts,
  digests and pointers, never tensors.  Kinds: 39500 network contract, 39501 node record, 39510
  window, 39511 receipt, 39512 validator verdict, 39520 artifact locator, 39530 contribution
  closeout.  Builders return unsigned events (kind, content, tags); ``check_event`` applies the
  required-tag rules; ``aggregate_window`` applies a window's weighted-average rule to its receipts
  (weights only: the tensors are averaged by the trainer's reduce-scatter).
  Reference: docs/nips/TRN.md:25-31 (scope), :171-177 (non-goals), :182-198 (kinds), :205-262 (tags),
  :324-350, :446-470, :562-575, :756-795 (examples).
* Commit authority: which node may commit a merged update, as a (term, holder) record with a lease;
  a higher term always wins, an equal term only for the same holder
  (docs/2026-06-10-cs336-assignment-training-audit.md:143-147 names the coordinator/term records).
* Mesh host election: term, active host, standby set and lease for a serving mesh, and the typed
  topologies it can place (docs/teardowns/2026-07-21-buzz-teardown.md:660-688).
* Reactor serving lane: a node declares per model profile which engine family serves it
  (packages/reactor-contracts/src/index.ts:61,152).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field

KIND_NETWORK, KIND_NODE, KIND_WINDOW, KIND_RECEIPT, KIND_VERDICT, KIND_ARTIFACT, KIND_CLOSEOUT = 39500, 39501, 39510, 39511, 39512, 39520, 39530
ADDRESSABLE = {KIND_NETWORK, KIND_NODE, KIND_WINDOW, KIND_ARTIFACT}
_REQUIRED = {KIND_NETWORK: ("d", "status"), KIND_NODE: ("d", "network", "role"), KIND_WINDOW: ("d", "network", "status", "sync_profile", "base_checkpoint"),
             KIND_RECEIPT: ("window", "network", "base_checkpoint", "p"), KIND_VERDICT: ("window", "network", "status", "p"),
             KIND_ARTIFACT: ("d", "network", "class", "x"), KIND_CLOSEOUT: ("window", "network", "p", "status")}
_FORBIDDEN_CONTENT_KEYS = ("tensor", "weights", "gradient", "gradients", "optimizer_state", "samples")


class TrnError(ValueError):
    pass


def _event(kind: int, content: dict, tags: list) -> dict:
    for k in content:
        if k in _FORBIDDEN_CONTENT_KEYS:
            raise TrnError(f"TRN events carry records and pointers, not {k}")
    return {"kind": kind, "content": json.dumps({"schema": 1, **content}, separators=(",", ":")), "tags": [list(map(str, t)) for t in tags]}


def tag_values(event: dict, name: str) -> list:
    """The values of every ``name`` tag.  Events come from relays: anything that is not a list of string lists counts as no tag."""
    tags = event.get("tags") if isinstance(event, dict) else None
    if not isinstance(tags, list):
        return []
    return [t[1:] for t in tags if isinstance(t, list) and t and t[0] == name and all(isinstance(x, str) for x in t)]


def first_tag(event: dict, name: str):
    v = tag_values(event, name)
    return v[0][0] if v and v[0] else None


def check_event(event: dict) -> list[str]:
    """Missing required tags (unknown tags are never an error)."""
    if not isinstance(event, dict):
        return ["not_an_event"]
    kind = event.get("kind")
    need = _REQUIRED.get(kind) if isinstance(kind, int) and not isinstance(kind, bool) else None
    if need is None:
        return [f"unknown_kind:{kind!r}"[:80]]
    errs = [f"missing_tag:{n}" for n in need if first_tag(event, n) is None]
    try:
        body = json.loads(event.get("content")) if isinstance(event.get("content"), str) else None
    except ValueError:
        body = None
    if not isinstance(body, dict):
        errs.append("content_not_json")
    elif body.get("schema") != 1:
        errs.append("content_schema")
    return errs


def network_contract(network_id: str, name: str, governance_revision: str, roles=("validator", "checkpoint_authority", "miner"),
                     window_cadence_s: int = 3600, status: str = "active") -> dict:
    return _event(KIND_NETWORK, {"name": name, "governance_revision": governance_revision},
                  [["d", network_id], ["status", status], ["window_cadence", window_cadence_s]] + [["role", r] for r in roles])


def node_record(network_id: str, node_id: str, roles, backend: str = "cuda", accelerator: str = "8xb200", storage: str = "remote_authoritative") -> dict:
    return _event(KIND_NODE, {"node": node_id},
                  [["d", f"{network_id}:{node_id}"], ["network", network_id]] + [["role", r] for r in roles]
                  + [["cap", "backend", backend], ["cap", "accelerator", accelerator], ["cap", "storage", storage]])


def training_window(network_id: str, window_id: str, round_index: int, base_checkpoint: str, planned_local_steps: int, policy: str,
                    min_participants: int = 1, min_weight_fraction: float = 0.8, aggregation_deadline_unix: int | None = None,
                    sync_profile: str = "diloco", status: str = "active") -> dict:
    return _event(KIND_WINDOW, {"round": round_index, "aggregation_deadline_unix": aggregation_deadline_unix},
                  [["d", window_id], ["network", network_id], ["status", status], ["sync_profile", sync_profile], ["round", round_index], ["policy", policy],
                   ["base_checkpoint", base_checkpoint], ["planned_local_steps", planned_local_steps], ["aggregation_rule", "weighted_avg"],
                   ["aggregation_weight", "tokens"], ["min_participants", min_participants], ["min_weight_fraction", min_weight_fraction]])


def training_receipt(window: dict, trainer_pubkey: str, local_steps: int, tokens: int, artifact_id: str, manifest_digest: str) -> dict:
    base = first_tag(window, "base_checkpoint")
    return _event(KIND_RECEIPT, {"subject_pubkey": trainer_pubkey, "base_checkpoint_id": base, "local_step_count": local_steps,
                                 "consumed_token_count": tokens, "aggregation_weight_value": str(tokens)},
                  [["window", first_tag(window, "d")], ["network", first_tag(window, "network")], ["round", first_tag(window, "round")],
                   ["base_checkpoint", base], ["local_steps", local_steps], ["tokens", tokens], ["weight", tokens], ["artifact", artifact_id],
                   ["manifest", manifest_digest], ["p", trainer_pubkey, "", "subject"]])


def validator_verdict(window: dict, receipt_event_id: str, trainer_pubkey: str, status: str, reason: str | None = None) -> dict:
    if status not in ("accepted", "rejected", "quarantined"):
        raise TrnError("verdict status must be accepted, rejected or quarantined")
    tags = [["window", first_tag(window, "d")], ["network", first_tag(window, "network")], ["status", status], ["e", receipt_event_id, "", "receipt"],
            ["p", trainer_pubkey, "", "subject"]]
    return _event(KIND_VERDICT, {"receipt": receipt_event_id}, tags + ([["reason", reason]] if reason else []))


def artifact_locator(window: dict, artifact_id: str, role: str, sha256: str, url: str, **content) -> dict:
    if role not in ("local_update", "aggregate", "checkpoint"):
        raise TrnError("artifact role must be local_update, aggregate or checkpoint")
    return _event(KIND_ARTIFACT, {"artifact_role": role, "base_checkpoint_id": first_tag(window, "base_checkpoint"), **content},
                  [["d", artifact_id], ["network", first_tag(window, "network")], ["window", first_tag(window, "d")], ["class", role],
                   ["base_checkpoint", first_tag(window, "base_checkpoint")], ["x", sha256], ["url", url]])


def aggregate_window(window: dict, receipts: list[dict], verdicts: list[dict]) -> dict:
    """Which contributions an aggregate of this window may include and with what weights: same window and
    base checkpoint, an ``accepted`` verdict (by receipt index), and the window's participation floors."""
    def number(event, name, default, cast):
        """A numeric tag; one that does not parse counts as ``default`` (a receipt with a garbled weight contributes nothing)."""
        try:
            v = cast(first_tag(event, name) or default)
            return v if v == v and abs(v) != float("inf") else default
        except (TypeError, ValueError, OverflowError):
            return default

    if check_event(window) or first_tag(window, "d") is None:
        raise TrnError("the window record is malformed")
    wid, base = first_tag(window, "d"), first_tag(window, "base_checkpoint")
    accepted = {first_tag(v, "e") for v in verdicts if first_tag(v, "window") == wid and first_tag(v, "status") == "accepted"} - {None}
    admitted, offered = [], 0
    for i, r in enumerate(receipts):
        if not isinstance(r, dict) or first_tag(r, "window") != wid:
            continue
        w = max(0, number(r, "weight", 0, int))
        offered += w
        rid = r.get("id", f"receipt-{i}")
        if first_tag(r, "base_checkpoint") == base and isinstance(rid, str) and rid in accepted and w > 0 and first_tag(r, "p") is not None:
            admitted.append({"trainer": first_tag(r, "p"), "weight": w, "artifact": first_tag(r, "artifact")})
    total = sum(a["weight"] for a in admitted)
    ok = (len(admitted) >= max(1, number(window, "min_participants", 1, int))
          and (offered == 0 or total / offered >= number(window, "min_weight_fraction", 0.0, float)) and total > 0)
    return {"window": wid, "base_checkpoint": base, "aggregation_rule": first_tag(window, "aggregation_rule"), "admitted": admitted,
            "admitted_update_count": len(admitted), "admitted_weight_total": str(total),
            "normalized_weights": [a["weight"] / total for a in admitted] if total else [], "promotion_state": "candidate" if ok else "superseded",
            "quorum_met": ok}


# ---------------------------------------------------------------- commit authority and mesh election
@dataclass
class CommitAuthority:
    """(term, holder, lease): who may commit merged updates.  Stored in the checkpoint manifest."""
    term: int = 0
    holder: str | None = None
    lease_expires_ms: int = 0

    def claim(self, node: str, now_ms: int, lease_ms: int = 30_000) -> bool:
        """A node takes (or renews) the authority: always when it is free or expired, otherwise only the holder."""
        if self.holder is None or now_ms >= self.lease_expires_ms:
            self.term += 1 if self.holder != node or now_ms >= self.lease_expires_ms else 0
            self.holder, self.lease_expires_ms = node, now_ms + lease_ms
            return True
        if self.holder == node:
            self.lease_expires_ms = now_ms + lease_ms
            return True
        return False

    def may_commit(self, node: str, term: int, now_ms: int) -> bool:
        return self.holder == node and term == self.term and now_ms < self.lease_expires_ms

    def observe(self, term: int, holder: str, lease_expires_ms: int) -> bool:
        """Merge a record seen elsewhere: a higher term wins; an equal term only extends the same holder's lease."""
        if term > self.term or (term == self.term and holder == self.holder and lease_expires_ms > self.lease_expires_ms):
            self.term, self.holder, self.lease_expires_ms = term, holder, lease_expires_ms
            return True
        return False

    def to_manifest(self) -> dict:
        return {"commitTerm": self.term, "commitHolder": self.holder, "leaseExpiresMs": self.lease_expires_ms}


TOPOLOGIES = ("replicated", "pipeline_sharded", "layer_sharded", "tensor_sharded", "sparse_expert")


@dataclass
class MeshElection:
    """Host election of a serving mesh: one active host per term, an ordered standby set, a lease."""
    term: int = 0
    active_host: str | None = None
    standby: list = field(default_factory=list)
    lease_expires_ms: int = 0

    def heartbeat(self, host: str, now_ms: int, lease_ms: int = 10_000) -> str:
        if self.active_host is None or (now_ms >= self.lease_expires_ms and host != self.active_host):
            # the lease ran out: the longest-waiting standby takes over (the caller joins the queue first)
            if host not in self.standby:
                self.standby.append(host)
            promoted = self.standby.pop(0)
            self.term, self.active_host, self.lease_expires_ms = self.term + 1, promoted, now_ms + lease_ms
            return "elected" if promoted == host else "standby"
        if host == self.active_host:
            self.lease_expires_ms = now_ms + lease_ms
            return "active"
        if host not in self.standby:
            self.standby.append(host)
        return "standby"

    def placement(self, topology: str, n_gpus: int, n_layers: int = 0, n_experts: int = 0) -> dict:
        """Typed placement for a single box of ``n_gpus``: stages for layer splits, ranges for experts."""
        if topology not in TOPOLOGIES:
            raise ValueError(f"unknown topology {topology!r}")
        if topology in ("pipeline_sharded", "layer_sharded"):
            per = -(-n_layers // n_gpus)
            stages = [{"nodeRef": f"gpu{g}", "layerStart": g * per, "layerEnd": min(n_layers, (g + 1) * per), "role": "stage"} for g in range(n_gpus)
                      if g * per < n_layers]
            return {"topology": topology, "stages": stages}
        if topology == "sparse_expert":
            if n_experts % n_gpus:
                raise ValueError("experts must divide evenly over the GPUs")
            per = n_experts // n_gpus
            return {"topology": topology, "expertRanges": [[g * per, (g + 1) * per] for g in range(n_gpus)]}
        return {"topology": topology, "ranks": n_gpus, "stages": [{"nodeRef": "box", "layerStart": 0, "layerEnd": n_layers, "role": "stage"}]}


SERVING_LANES = ("hydralisk", "psionic")


def reactor_model_profile(model_ref: str, serving_lane: str, eval_harness_owner: str = "psionic") -> dict:
    if serving_lane not in SERVING_LANES:
        raise ValueError(f"serving lane must be one of {SERVING_LANES}")
    return {"modelRef": model_ref, "servingLane": serving_lane, "evalHarnessProfileOwner": eval_harness_owner}
