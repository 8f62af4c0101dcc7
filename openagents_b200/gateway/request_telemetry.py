"""Per-request telemetry record: every number is measured or the ``not_measured`` sentinel.

Reference: inference/khala-telemetry.ts:1-50 (contract), :86-94 ``measured``, :108 request classes,
:185 block, :223 record.  Derived fields: inter-token latency = generation wall clock / (completion
tokens - 1); perceived tokens/s = completion tokens / generation seconds; unaccounted tokens = total
- (prompt + completion); margin bucket from (price - cost) / price at 0.1 and 0.4; missing timing
splits, region, health score, fallback reason and economics each add a blocker ref.
"""
from __future__ import annotations

import math

from .metadata import NOT_MEASURED, UNKNOWN_QUANTIZATION, UNKNOWN_SPECULATION, quantization_metadata, speculation_metadata
from .prompt_cache import hash_cache_affinity_key

SCHEMA = "openagents.khala.telemetry.v1"
REQUEST_CLASSES = ("interactive_stream", "async_job", "verifier_run", "batch")
VERIFICATION_CLASSES = ("none", "seeded", "test_passed", "exact_trace_replay", "unverified", "failed")
EXECUTED_VERDICTS = ("not_executed", "passed", "failed")
SETTLEMENT_STATES = ("not_applicable", "pending", "settled")
ECONOMICS_STATES = ("measured", "simulated", "pending", NOT_MEASURED)


def measured(v):
    if v is None or isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v) or v < 0:
        return NOT_MEASURED
    return v


def is_measured(v) -> bool:
    return v != NOT_MEASURED


def margin_bucket(cost, price) -> str:
    if not (is_measured(cost) and is_measured(price)):
        return NOT_MEASURED
    margin = price - cost
    if margin < 0:
        return "negative"
    if margin == 0:
        return "zero"
    ratio = 0 if price == 0 else margin / price
    return "thin" if ratio < 0.1 else "standard" if ratio < 0.4 else "rich"


def build_record(*, request_id, requested_model, served_model, route, provider, request_class, verification_class="none",
                 executed_verdict="not_executed", settlement_state="not_applicable", quantization: dict | None = None,
                 speculation: dict | None = None, prompt_tokens=None, completion_tokens=None, total_tokens=None,
                 cached_input_tokens=None, ttft_ms=None, total_wall_clock_ms=None, generation_wall_clock_ms=None,
                 provider_time_ms=None, gateway_overhead_ms=None, verifier_time_ms=None, settlement_time_ms=None,
                 queue_wait_ms=None, batch_wait_ms=None, region=None, provider_health_score=None,
                 cache_affinity_key_raw=None, fallback_reason=..., scalar_reward=None, verifier_receipt_ref=None,
                 cost_basis_msat=None, price_msat=None, economics_state=None, settlement_receipt_refs=(), blocker_refs=()) -> dict:
    for v, allowed in ((request_class, REQUEST_CLASSES), (verification_class, VERIFICATION_CLASSES),
                       (executed_verdict, EXECUTED_VERDICTS), (settlement_state, SETTLEMENT_STATES)):
        if v not in allowed:
            raise ValueError(f"{v!r} is not one of {allowed}")
    cost, price = measured(cost_basis_msat), measured(price_msat)
    if economics_state is None:
        economics_state = "measured" if is_measured(cost) and is_measured(price) else "pending" if settlement_state == "pending" else NOT_MEASURED
    gen = generation_wall_clock_ms
    gen_ok = isinstance(gen, (int, float)) and math.isfinite(gen)
    itl = gen / (completion_tokens - 1) if gen_ok and gen >= 0 and isinstance(completion_tokens, int) and completion_tokens > 1 else NOT_MEASURED
    tps = completion_tokens / (gen / 1000) if gen_ok and gen > 0 and isinstance(completion_tokens, int) and completion_tokens >= 0 else NOT_MEASURED
    p, c, t = measured(prompt_tokens), measured(completion_tokens), measured(total_tokens)
    unaccounted = max(0, t - (p + c)) if all(is_measured(x) for x in (p, c, t)) else NOT_MEASURED
    region_ok = isinstance(region, str) and region.strip() != ""
    auto = []
    for val, ref in ((provider_time_ms, "provider_time_not_measured"), (gateway_overhead_ms, "gateway_overhead_not_measured"),
                     (verifier_time_ms, "verifier_time_not_measured"), (settlement_time_ms, "settlement_time_not_measured")):
        if not is_measured(measured(val)):
            auto.append(ref)
    if not region_ok:
        auto.append("region_not_measured")
    if not is_measured(measured(provider_health_score)):
        auto.append("provider_health_score_not_measured")
    if fallback_reason is ...:
        auto.append("fallback_reason_not_reported")
    if economics_state in (NOT_MEASURED, "pending", "simulated"):
        auto.append("economics_" + economics_state)
    refs = list(dict.fromkeys(list(blocker_refs) + auto))
    fb = fallback_reason if isinstance(fallback_reason, str) and fallback_reason.strip() else None
    return {
        "schemaVersion": SCHEMA, "requestId": request_id, "requestedModel": requested_model, "servedModel": served_model,
        "quantization": dict(UNKNOWN_QUANTIZATION) if quantization is None else quantization_metadata(**quantization),
        "speculation": dict(UNKNOWN_SPECULATION) if speculation is None else speculation_metadata(**speculation),
        "route": route, "provider": provider, "region": region if region_ok else NOT_MEASURED,
        "providerHealthScore": measured(provider_health_score),
        "cacheAffinityKeyHash": hash_cache_affinity_key(cache_affinity_key_raw) if isinstance(cache_affinity_key_raw, str) and cache_affinity_key_raw.strip() else None,
        "fallbackReason": fb, "requestClass": request_class, "promptTokens": p, "completionTokens": c, "totalTokens": t,
        "cachedInputTokens": measured(cached_input_tokens), "unaccountedTokens": unaccounted, "ttftMs": measured(ttft_ms),
        "interTokenLatencyMs": itl, "perceivedTps": tps, "totalWallClockMs": measured(total_wall_clock_ms),
        "providerTimeMs": measured(provider_time_ms), "gatewayOverheadMs": measured(gateway_overhead_ms),
        "verifierTimeMs": measured(verifier_time_ms), "settlementTimeMs": measured(settlement_time_ms),
        "queueWaitMs": measured(queue_wait_ms), "batchWaitMs": measured(batch_wait_ms),
        "verificationClass": verification_class, "executedVerdict": executed_verdict, "scalarReward": measured(scalar_reward),
        "verifierReceiptRef": verifier_receipt_ref, "costBasisMsat": cost, "priceMsat": price, "economicsState": economics_state,
        "marginBucket": margin_bucket(cost, price), "settlementState": settlement_state,
        "settlementReceiptRefs": list(settlement_receipt_refs), "blockerRefs": refs,
    }


_BLOCK_FIELDS = ("requestClass", "promptTokens", "completionTokens", "totalTokens", "cachedInputTokens", "ttftMs",
                 "totalWallClockMs", "verificationClass", "executedVerdict", "scalarReward")


def block_from_record(record: dict, detail_ref: str | None) -> dict:
    """The compact public block that rides on a response; the full record stays server-side."""
    out = {"schemaVersion": SCHEMA}
    out.update({k: record[k] for k in _BLOCK_FIELDS})
    out["detailRef"] = detail_ref
    return out
