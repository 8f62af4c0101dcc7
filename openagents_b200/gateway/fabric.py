"""Serving-fabric client side: provider-adapter seam, the serve dispatch with its parity gate, the
HTTP transport, the node admission gate and the network adapter.

This is the compatibility surface between a gateway and ``b200-serve`` (``POST /v1/serve``).
Reference: inference/provider-adapter.ts:52-88 (request, usage), :246-285 (typed error with a
retryable flag), :288-338 (adapter and registry); inference/psionic-fabric-serve.ts:116-173
(wire types), :267-315 (normalisation), :358-408 (five-step dispatch: transport fault passes
through, malformed fails closed, more than one stage is refused, no verified parity means no
success, then result + receipt); inference/pylon-fabric-http-transport.ts:71-78 (status classes),
:98-130 (bearer POST); inference/khala-pylon-admission.ts:39-70, 100-217 (admission);
inference/openagents-network-adapter.ts:215-297 (paid-traffic gate, inert-by-default adapter).
"""
from __future__ import annotations

import json
import urllib.error
import urllib.request
from dataclasses import dataclass, field
from datetime import datetime

from ..receipts.manifests import clears_paid_traffic, serving_receipt

FABRIC_PARITY_UNVERIFIED_KIND = "fabric_parity_unverified"
FABRIC_SHARDED_UNSUPPORTED_KIND = "fabric_sharded_unsupported"
FABRIC_MALFORMED_RESPONSE_KIND = "malformed_response"
FABRIC_TRANSPORT_ERROR_KIND = "transport_error"
NETWORK_NOT_LIVE_KIND = "network_lane_not_live"
ADMISSION_REFUSED_KIND = "pylon_admission_refused"


class InferenceAdapterError(Exception):
    def __init__(self, adapter_id: str, kind: str, reason: str, retryable: bool = False, http_status: int | None = None):
        super().__init__(f"{adapter_id}: {kind}: {reason}")
        self.adapter_id, self.kind, self.reason, self.retryable, self.http_status = adapter_id, kind, reason, retryable, http_status


@dataclass(frozen=True)
class InferenceRequest:
    model: str
    messages: tuple
    stream: bool = False
    passthrough_params: dict = field(default_factory=dict)
    priority: str = "external"          # batch | external | internal_stress | keep_warm


@dataclass(frozen=True)
class InferenceUsage:
    prompt_tokens: int
    completion_tokens: int
    total_tokens: int
    cached_prompt_tokens: int | None = None
    reasoning_tokens: int | None = None


@dataclass(frozen=True)
class InferenceResult:
    content: str
    finish_reason: str
    served_model: str
    usage: InferenceUsage


class ProviderRegistry:
    """adapter id -> adapter (an object with ``id`` and ``complete(request)``)."""

    def __init__(self):
        self._adapters = {}

    def register(self, adapter):
        self._adapters[adapter.id] = adapter

    def get(self, adapter_id: str):
        return self._adapters.get(adapter_id)

    def ids(self):
        return list(self._adapters)


# ---------------------------------------------------------------- serve dispatch
def _usage(u) -> InferenceUsage | None:
    if not isinstance(u, dict):
        return None
    try:
        p, c, t = u["promptTokens"], u["completionTokens"], u["totalTokens"]
    except KeyError:
        return None
    if not all(isinstance(v, int) and v >= 0 for v in (p, c, t)):
        return None
    return InferenceUsage(p, c, t, u.get("cachedPromptTokens"), u.get("reasoningTokens"))


def _stages(s) -> list | None:
    if not isinstance(s, list):
        return None
    for st in s:
        if not (isinstance(st, dict) and isinstance(st.get("nodeRef"), str) and isinstance(st.get("layerStart"), int)
                and isinstance(st.get("layerEnd"), int) and st.get("role") in ("stage", "coordinator", "draft")):
            return None
    return s


def normalize_serve_response(raw):
    """dict (or JSON string) -> validated serve response dict, or None if malformed."""
    if isinstance(raw, str):
        try:
            raw = json.loads(raw)
        except json.JSONDecodeError:
            return None
    if not isinstance(raw, dict):
        return None
    usage, stages = _usage(raw.get("usage")), _stages(raw.get("stages"))
    ok = (isinstance(raw.get("content"), str) and isinstance(raw.get("finishReason"), str) and raw["finishReason"].strip()
          and isinstance(raw.get("servedModel"), str) and raw["servedModel"].strip()
          and isinstance(raw.get("servingRunRef"), str) and raw["servingRunRef"].strip()
          and raw.get("parityMode") in ("exact_greedy_parity", "none") and isinstance(raw.get("parityVerified"), bool)
          and usage is not None and stages is not None)
    if not ok:
        return None
    out = {k: raw[k] for k in ("content", "finishReason", "servedModel", "servingRunRef", "parityMode", "parityVerified")}
    out["usage"], out["stages"] = usage, stages
    if isinstance(raw.get("paidTrafficVerification"), dict):
        out["paidTrafficVerification"] = raw["paidTrafficVerification"]
    return out


def dispatch_psionic_serve(transport, adapter_id: str = "openagents-network"):
    """Returns ``dispatch(request) -> (InferenceResult, receipt)``; ``transport(serve_request)``
    returns a response dict / JSON string or raises ``InferenceAdapterError``."""

    def dispatch(request: InferenceRequest):
        raw = transport({"model": request.model, "messages": [dict(m) for m in request.messages],
                         "passthroughParams": dict(request.passthrough_params), "requireExactGreedyParity": True})
        serve = normalize_serve_response(raw)
        if serve is None:
            raise InferenceAdapterError(adapter_id, FABRIC_MALFORMED_RESPONSE_KIND, "fabric serve returned a malformed serve response")
        if len(serve["stages"]) > 1:
            raise InferenceAdapterError(adapter_id, FABRIC_SHARDED_UNSUPPORTED_KIND,
                                        "shard-WAN multi-stage serving is deferred; whole-small-model only this wave")
        if not (serve["parityMode"] == "exact_greedy_parity" and serve["parityVerified"]):
            raise InferenceAdapterError(adapter_id, FABRIC_PARITY_UNVERIFIED_KIND,
                                        "fabric serve did not return a verified exact-greedy parity receipt")
        result = InferenceResult(serve["content"], serve["finishReason"], serve["servedModel"], serve["usage"])
        wire = dict(serve)
        wire["usage"] = {}
        receipt = serving_receipt(wire)
        if "paidTrafficVerification" in serve:
            receipt["paidTrafficVerification"] = serve["paidTrafficVerification"]
        return result, receipt

    return dispatch


def classify_status(status: int) -> tuple[str, bool]:
    if status == 429:
        return "rate_limited", True
    if status == 503:
        return "service_overloaded", True
    if status >= 500:
        return "upstream_error", True
    return "request_rejected", False


def make_http_transport(endpoint: str, bearer_token: str, opener=urllib.request.urlopen, timeout_s: float = 120.0,
                        adapter_id: str = "openagents-network"):
    """POST the serve request as JSON with bearer auth.  ``opener`` is injectable for tests."""

    def transport(serve_request: dict):
        req = urllib.request.Request(endpoint, data=json.dumps(serve_request).encode(),
                                     headers={"Content-Type": "application/json", "Authorization": f"Bearer {bearer_token}"})
        try:
            with opener(req, timeout=timeout_s) as r:
                return r.read().decode()
        except urllib.error.HTTPError as e:
            kind, retryable = classify_status(e.code)
            raise InferenceAdapterError(adapter_id, kind, f"fabric serve answered HTTP {e.code}", retryable, e.code)
        except (urllib.error.URLError, OSError) as e:
            raise InferenceAdapterError(adapter_id, FABRIC_TRANSPORT_ERROR_KIND, str(e), True)

    return transport


# ---------------------------------------------------------------- admission
DEFAULT_HEARTBEAT_TTL_MS = 90_000
HEALTHY_HEARTBEAT_STATUSES = frozenset(("ok", "healthy", "active", "ready"))
ADMISSION_POLICY_REF = "policy.khala_pylon_admission.v1"
_B = "blocker.pylon_admission."


@dataclass(frozen=True)
class ServingSnapshot:
    pylon_ref: str
    status: str
    capability_refs: tuple
    serving_lane_refs: tuple
    latest_heartbeat_at: str | None
    latest_heartbeat_status: str | None
    wallet_ready: bool
    spark_payout_target_ref: str | None


def decide_admission(s: ServingSnapshot, required_capability_ref: str, now_ms: int, heartbeat_ttl_ms: int | None = None) -> dict:
    ttl = heartbeat_ttl_ms if isinstance(heartbeat_ttl_ms, (int, float)) and heartbeat_ttl_ms > 0 else DEFAULT_HEARTBEAT_TTL_MS
    blockers = []
    if s.status != "active":
        blockers.append(_B + "registration_not_active")
    if required_capability_ref not in s.capability_refs:
        blockers.append(_B + "capability_not_advertised")
    if not s.serving_lane_refs:
        blockers.append(_B + "no_serving_lane_advert")
    hb = None
    if s.latest_heartbeat_at is not None:
        try:
            hb = datetime.fromisoformat(s.latest_heartbeat_at.replace("Z", "+00:00")).timestamp() * 1000
        except ValueError:
            hb = None
    if hb is None:
        blockers.append(_B + "no_heartbeat")
    else:
        if s.latest_heartbeat_status not in HEALTHY_HEARTBEAT_STATUSES:
            blockers.append(_B + "heartbeat_not_healthy")
        if now_ms - hb > ttl:
            blockers.append(_B + "heartbeat_stale")
    if not s.wallet_ready:
        blockers.append(_B + "wallet_not_ready")
    if not (s.spark_payout_target_ref or "").strip():
        blockers.append(_B + "no_spark_payout_target")
    return {"schema": "openagents.khala_pylon_admission.v1", "pylonRef": s.pylon_ref, "admitted": not blockers,
            "blockerRefs": blockers, "policyRefs": [ADMISSION_POLICY_REF]}


# ---------------------------------------------------------------- network adapter
class OpenAgentsNetworkAdapter:
    """The ``openagents-network`` lane: inert unless a dispatch is injected; with an admission
    snapshot provider it refuses before dispatch when the node is not admitted."""
    id = "openagents-network"

    def __init__(self, dispatch=None, admission=None):
        self._dispatch, self._admission = dispatch, admission

    def complete(self, request: InferenceRequest):
        if self._dispatch is None:
            raise InferenceAdapterError(self.id, NETWORK_NOT_LIVE_KIND, "the network lane has no live dispatch", False)
        if self._admission is not None:
            decision = self._admission()
            if not decision["admitted"]:
                raise InferenceAdapterError(self.id, ADMISSION_REFUSED_KIND, ",".join(decision["blockerRefs"]), False)
        result, receipt = self._dispatch(request)
        return result, receipt, clears_paid_traffic(receipt)
