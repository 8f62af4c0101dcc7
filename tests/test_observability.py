"""Served-token ledger, serving-rate monitor, chat trace emitter and the byte-level BPE tokenizer (CPU)."""
import json

from openagents_b200.gateway.observability import (REASON_LANE_DOWN, REASON_RATE_LOW, ChatTraceEmitter, RateMonitorConfig,
                                                   ServedTokensLedger, ServingRateMonitor, classify_serving_rate, redact,
                                                   validate_trajectory)
from openagents_b200.serve.generation import BpeTokenizer, _byte_alphabet, tokenizer_from_metadata


def test_ledger_is_idempotent_and_public_safe(tmp_path):
    t = [1000.0]
    path = str(tmp_path / "ledger.jsonl")
    led = ServedTokensLedger(path, now=lambda: t[0])
    assert led.record("req-1", "tiny", 10, 5)["inserted"]
    assert led.record("req-1", "tiny", 10, 5) == {"inserted": False, "reason": "duplicate"}      # a replay never double-counts
    assert led.record("req-2", "tiny", 0, 0) == {"inserted": False, "reason": "zero_tokens"}
    t[0] = 5000.0
    led.record("req-3", "tiny", 7, 3, demand_kind="not-a-kind")
    assert led.total() == 25 and led.tokens_since(4000.0) == 10
    row = json.loads(open(path).readline())
    assert set(row) == {"idempotencyKey", "requestId", "accountRef", "modelId", "servedModel", "adapterId", "inputTokens",
                        "outputTokens", "demandKind", "recordedAt"}      # refs and counts only: no prompt, no completion
    assert ServedTokensLedger(path).total() == 25                        # reloads from disk
    assert led.rows["served:req-3"]["demandKind"] == "unlabeled"


def test_rate_monitor_classifies_and_dedupes_alerts():
    cfg = RateMonitorConfig(token_floor_per_hour=100, lane_down_minutes=15, cadence_minutes=5)
    assert classify_serving_rate(500, 990.0, 1000.0, cfg)["status"] == "healthy"
    low = classify_serving_rate(50, 990.0, 1000.0, cfg)
    assert low["status"] == "serving_rate_low" and low["reasonRefs"] == [REASON_RATE_LOW]
    down = classify_serving_rate(50, None, 1000.0, cfg)
    assert down["status"] == "glm_down" and down["alertKinds"] == ["glm_down", "serving_rate_low"] and REASON_LANE_DOWN in down["reasonRefs"]
    t = [10_000.0]
    led = ServedTokensLedger(now=lambda: t[0])
    mon = ServingRateMonitor(led, cfg, now=lambda: t[0])
    mon.lane_heartbeat()
    first = mon.tick()
    assert first["classification"]["status"] == "serving_rate_low" and len(first["alertRefs"]) == 1
    assert mon.tick()["alertRefs"] == []              # same window: no second alert of the same kind
    t[0] += 400
    assert len(mon.tick()["alertRefs"]) == 1          # next window
    led.record("r", "m", 200, 0)
    assert mon.tick()["classification"]["status"] == "healthy"
    t[0] += 16 * 60
    assert mon.tick()["classification"]["status"] == "glm_down"       # no heartbeat for 16 minutes
    assert RateMonitorConfig.from_env({"SERVING_RATE_MONITOR_ENABLED": "false"}).enabled is False
    assert mon.should_run_at(300.0) and not mon.should_run_at(360.0)


def test_trace_emitter_is_off_by_default_redacts_and_validates():
    msgs = [{"role": "system", "content": "be brief"}, {"role": "user", "content": "my key is sk-abcdefghijklmnopqrstuvwx ok?"}]
    assert ChatTraceEmitter().emit(msgs, "hi", opted_in=True) == {"emitted": False, "reason": "disabled"}
    em = ChatTraceEmitter(enabled=True)
    assert em.emit(msgs, "hi", opted_in=False)["reason"] == "disabled"          # the request must opt in too
    r = em.emit(msgs, "sure", opted_in=True, tool_calls=[{"id": "c1", "function": {"name": "f", "arguments": "{}"}}])
    assert r["emitted"] and r["redactions"] == 1
    traj = em.store[r["traceId"]]["trajectory"]
    assert validate_trajectory(traj) == [] and "sk-abc" not in json.dumps(traj)
    assert traj["agent"]["model_name"] == "openagents/khala" and traj["steps"][-1]["tool_calls"][0]["function_name"] == "f"
    assert em.store[r["traceId"]]["visibility"] == "unlisted"
    assert validate_trajectory({"schema_version": "x"}) != []
    assert redact({"a": ["Bearer abcdefghijklmnopqrstuvwxyz0123"]})[1] == 1


def test_byte_level_bpe_round_trip_and_merge_order():
    b2u = _byte_alphabet()
    base = [b2u[b] for b in range(256)]
    merges = ["h e", "l l", "he ll", "hell o", "Ġ w", "Ġw o"]
    toks = base + [m.replace(" ", "") for m in merges] + ["<|eot|>"]
    tk = BpeTokenizer(toks, merges, eos_id=len(toks) - 1, token_types=[1] * (len(toks) - 1) + [3])
    ids = tk.encode("hello world<|eot|>héllo ☃")
    assert tk.decode(ids) == "hello world<|eot|>héllo ☃"
    assert ids[0] == toks.index("hello") and ids[1] == toks.index("Ġwo") and toks.index("<|eot|>") in ids
    meta = {"tokenizer.ggml.tokens": toks, "tokenizer.ggml.merges": merges, "tokenizer.ggml.eos_token_id": len(toks) - 1,
            "tokenizer.ggml.token_type": [1] * (len(toks) - 1) + [3]}
    assert isinstance(tokenizer_from_metadata(meta, len(toks)), BpeTokenizer)
    assert tokenizer_from_metadata({}, 512).encode("a") == [97]


def test_ledger_memory_is_bounded_and_totals_stay_exact(tmp_path):
    from openagents_b200.gateway.observability import ServedTokensLedger
    t = [1_000_000.0]
    path = str(tmp_path / "big.jsonl")
    led = ServedTokensLedger(path, now=lambda: t[0], max_rows_in_memory=100)
    for i in range(1000):
        t[0] += 1.0                                     # one request a second, 3 tokens each
        assert led.record(f"r{i}", "m", 1, 2)["inserted"]
    assert len(led.rows) <= 100 and led.total() == 3000 and led.public_projection() == {"tokensServed": 3000, "rows": 1000}
    assert led.record("r999", "m", 1, 2) == {"inserted": False, "reason": "duplicate"}       # recent keys are still recognised
    assert led.tokens_since(t[0] - 9.5) == 30                                               # inside the kept rows: exact
    far = led.tokens_since(t[0] - 600)                                                      # beyond them: per-minute series
    assert 600 * 3 <= far <= 661 * 3
    assert led.tokens_since(0) == 3000
    with open(path, "a") as f:
        f.write('{"idempotencyKey": "served:torn", "inputTok')                              # the process died mid-write
    again = ServedTokensLedger(path, now=lambda: t[0], max_rows_in_memory=100)
    assert again.total() == 3000 and len(again.rows) <= 100 and again.public_projection()["rows"] == 1000
