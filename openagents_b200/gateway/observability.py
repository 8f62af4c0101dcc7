"""Serving observability: the served-token ledger, the serving-rate monitor and the chat trace emitter.

The three pieces follow the reference gateway's modules of the same purpose:

* ``ServedTokensLedger``: one row per COMPLETED request, keyed idempotently by the request id, counted whatever
  metering path handled it, zero-token completions skipped, rows public-safe (refs, model ids, integer counts,
  timestamps; never prompts or completions)
  (apps/openagents.com/workers/api/src/inference/served-tokens-recorder.ts:1-40).
* ``ServingRateMonitor``: every ``cadence_minutes`` classify the last hour's served tokens against a floor and the
  serving lane's last healthy heartbeat against a down window; raise at most one alert per kind per window
  (apps/openagents.com/workers/api/src/inference/serving-rate-monitor.ts:14-31,100-140).
* ``ChatTraceEmitter``: flag-gated and off by default; a completed chat session becomes a redacted trajectory whose
  model name is the public id, validated and checked by a tripwire before it is stored; a failure never touches the
  response (apps/openagents.com/workers/api/src/inference/khala-chat-trace-emitter.ts:1-40).
"""
from __future__ import annotations

import json
import os
import re
import threading
import time
import uuid
from dataclasses import dataclass, field

REASON_RATE_LOW = "blocker.public.serving_rate.tokens_per_hour_below_floor"
REASON_LANE_DOWN = "blocker.public.serving_rate.glm_lane_down"
DEMAND_KINDS = ("external", "internal", "internal_stress", "own_capacity", "unlabeled")

_UNSAFE = re.compile(r"(sk-[A-Za-z0-9]{16,}|AKIA[0-9A-Z]{16}|-----BEGIN [A-Z ]*PRIVATE KEY-----|Bearer\s+[A-Za-z0-9._\-]{20,}|"
                     r"xox[baprs]-[A-Za-z0-9\-]{10,}|ghp_[A-Za-z0-9]{30,}|nsec1[a-z0-9]{20,})")


class ServedTokensLedger:
    """Canonical record of served tokens.  ``record`` is safe to call from any thread and never raises into the
    serving path: a persistence error is counted and swallowed, because the ledger is a projection of the served
    answer, not its source."""

    def __init__(self, path: str | None = None, now=time.time, max_rows_in_memory: int = 100_000):
        """``max_rows_in_memory``: rows kept for idempotency and inspection.  Totals and the per-minute series behind
        ``tokens_since`` are running sums, so a server that has answered millions of requests holds a bounded ledger; the file
        (when there is one) keeps every row.  A duplicate of a row older than the kept window would be counted again."""
        self.path, self.now, self.max_rows = path, now, max(1, int(max_rows_in_memory))
        self.rows: dict[str, dict] = {}
        self.lock = threading.Lock()
        self.persist_errors = 0
        self._total, self._count = 0, 0
        self._minutes: dict[int, int] = {}             # minute index -> tokens recorded in that minute (last 48 h)
        self._dropped_until = float("-inf")            # recordedAt of the newest row no longer in ``rows``
        if path and os.path.exists(path):
            for line in open(path):
                if line.strip():
                    try:
                        row = json.loads(line)
                        key = row["idempotencyKey"]
                        int(row["inputTokens"]), int(row["outputTokens"]), float(row["recordedAt"])
                    except (ValueError, KeyError, TypeError):
                        continue                       # a torn last line of a ledger that was being written when the process died
                    if key not in self.rows:
                        self._admit(key, row)

    def _admit(self, key: str, row: dict):
        n = row["inputTokens"] + row["outputTokens"]
        self.rows[key] = row
        self._total += n
        self._count += 1
        minute = int(row["recordedAt"] // 60)
        self._minutes[minute] = self._minutes.get(minute, 0) + n
        if len(self.rows) > self.max_rows:
            for k in list(self.rows)[: max(1, self.max_rows // 10)]:
                self._dropped_until = max(self._dropped_until, self.rows.pop(k)["recordedAt"])
            horizon = minute - 48 * 60
            for m in [m for m in self._minutes if m < horizon]:
                del self._minutes[m]

    def record(self, request_id: str, model_id: str, input_tokens: int, output_tokens: int, account_ref: str = "account.anonymous",
               adapter_id: str = "psionic", demand_kind: str = "unlabeled", served_model: str | None = None) -> dict:
        inp, out = max(0, int(input_tokens)), max(0, int(output_tokens))
        if inp + out == 0:
            return {"inserted": False, "reason": "zero_tokens"}
        if demand_kind not in DEMAND_KINDS:
            demand_kind = "unlabeled"
        row = {"idempotencyKey": f"served:{request_id}", "requestId": request_id, "accountRef": account_ref, "modelId": model_id,
               "servedModel": served_model or model_id, "adapterId": adapter_id, "inputTokens": inp, "outputTokens": out,
               "demandKind": demand_kind, "recordedAt": self.now()}
        with self.lock:
            if row["idempotencyKey"] in self.rows:
                return {"inserted": False, "reason": "duplicate"}
            self._admit(row["idempotencyKey"], row)
            if self.path:
                try:
                    with open(self.path, "a") as f:
                        f.write(json.dumps(row, sort_keys=True) + "\n")
                except OSError:
                    self.persist_errors += 1
        return {"inserted": True, "row": row}

    def total(self) -> int:
        with self.lock:
            return self._total

    def tokens_since(self, t: float) -> int:
        """Tokens recorded at or after ``t``: exact from the kept rows while they reach back that far, else from the per-minute
        series (whole minutes, so up to one minute more than asked)."""
        with self.lock:
            if t > self._dropped_until:
                return sum(r["inputTokens"] + r["outputTokens"] for r in self.rows.values() if r["recordedAt"] >= t)
            first = int(t // 60)
            return sum(n for m, n in self._minutes.items() if m >= first)

    def public_projection(self) -> dict:
        with self.lock:
            return {"tokensServed": self._total, "rows": self._count}


@dataclass
class RateMonitorConfig:
    enabled: bool = True
    cadence_minutes: int = 5
    lane_down_minutes: int = 15
    token_floor_per_hour: int = 50_000_000

    @classmethod
    def from_env(cls, env: dict | None = None) -> "RateMonitorConfig":
        env = os.environ if env is None else env

        def pos_int(key, default):
            try:
                v = int(str(env.get(key, "")).strip())
                return v if v > 0 else default
            except ValueError:
                return default

        return cls(enabled=str(env.get("SERVING_RATE_MONITOR_ENABLED", "true")).strip().lower() == "true",
                   cadence_minutes=pos_int("SERVING_RATE_MONITOR_CADENCE_MINUTES", 5),
                   lane_down_minutes=pos_int("SERVING_RATE_MONITOR_GLM_DOWN_MINUTES", 15),
                   token_floor_per_hour=pos_int("SERVING_RATE_MONITOR_TOKEN_FLOOR_PER_HOUR", 50_000_000))


def classify_serving_rate(tokens_last_hour: int, latest_healthy_heartbeat: float | None, now: float,
                          cfg: RateMonitorConfig) -> dict:
    """Lane-down wins over rate-low in ``status``; both alert kinds are listed when both hold."""
    lane_ok = latest_healthy_heartbeat is not None and now - latest_healthy_heartbeat <= cfg.lane_down_minutes * 60
    low = max(0, int(tokens_last_hour)) < cfg.token_floor_per_hour
    kinds, reasons = [], []
    if not lane_ok:
        kinds.append("glm_down")
        reasons.append(REASON_LANE_DOWN)
    if low:
        kinds.append("serving_rate_low")
        reasons.append(REASON_RATE_LOW)
    status = "glm_down" if not lane_ok else "serving_rate_low" if low else "healthy"
    return {"status": status, "alertKinds": kinds, "reasonRefs": reasons, "glmHealthy": lane_ok,
            "tokensLastHour": max(0, int(tokens_last_hour)), "tokenFloorPerHour": cfg.token_floor_per_hour,
            "latestHealthyGlmHeartbeatAt": latest_healthy_heartbeat}


class ServingRateMonitor:
    def __init__(self, ledger: ServedTokensLedger, cfg: RateMonitorConfig | None = None, now=time.time):
        self.ledger, self.cfg, self.now = ledger, cfg or RateMonitorConfig(), now
        self.heartbeat: float | None = None
        self.alerts: list[dict] = []

    def lane_heartbeat(self, healthy: bool = True):
        if healthy:
            self.heartbeat = self.now()

    def should_run_at(self, t: float) -> bool:
        return int(t // 60) % max(1, self.cfg.cadence_minutes) == 0

    def tick(self) -> dict:
        now = self.now()
        if not self.cfg.enabled:
            return {"enabled": False, "ranAt": now, "alertRefs": [], "classification": {"status": "disabled"}}
        c = classify_serving_rate(self.ledger.tokens_since(now - 3600), self.heartbeat, now, self.cfg)
        refs = []
        window = self.cfg.cadence_minutes * 60
        for kind, reason in zip(c["alertKinds"], c["reasonRefs"]):
            if any(a["classification"] == kind and a["detectedAt"] > now - window for a in self.alerts):
                continue               # one alert per kind per window
            aid = uuid.uuid4().hex
            a = {"id": aid, "alertRef": f"serving_rate_alert.{kind}.{int(now)}.{aid[:8]}", "detectedAt": now,
                 "classification": kind, "reasonRef": reason, "burnTokensWindow": c["tokensLastHour"], "windowMinutes": 60,
                 "stallThresholdTokens": self.cfg.token_floor_per_hour,
                 "recoveryActions": ["check_lane_health", "check_replica_pool"] if kind == "glm_down" else ["check_demand", "check_admission"]}
            self.alerts.append(a)
            refs.append(a["alertRef"])
        return {"enabled": True, "ranAt": now, "alertRefs": refs, "classification": c}


def redact(value):
    """Replace credential-shaped substrings in every string of a JSON-like value; returns (value, hits)."""
    hits = 0

    def walk(v):
        nonlocal hits
        if isinstance(v, str):
            out, n = _UNSAFE.subn("[redacted]", v)
            hits += n
            return out
        if isinstance(v, list):
            return [walk(x) for x in v]
        if isinstance(v, dict):
            return {k: walk(x) for k, x in v.items()}
        return v

    return walk(value), hits


def validate_trajectory(t: dict) -> list[str]:
    errs = []
    if t.get("schema_version") != "ATIF-v1.7":
        errs.append("schema_version")
    if not isinstance(t.get("session_id"), str) or not t.get("session_id"):
        errs.append("session_id")
    if not isinstance(t.get("agent"), dict) or not t["agent"].get("name") or not t["agent"].get("model_name"):
        errs.append("agent")
    steps = t.get("steps")
    if not isinstance(steps, list) or not steps:
        errs.append("steps")
    else:
        for i, s in enumerate(steps):
            if s.get("step_id") != i + 1 or s.get("source") not in ("user", "agent", "system") or not isinstance(s.get("message"), str):
                errs.append(f"steps[{i}]")
    return errs


@dataclass
class ChatTraceEmitter:
    """``emit`` does nothing (``reason = "disabled"``) unless the emitter is enabled AND the request opted in."""
    enabled: bool = False
    public_model_name: str = "openagents/khala"
    store: dict = field(default_factory=dict)

    def emit(self, messages: list[dict], assistant_text: str, opted_in: bool, tool_calls: list[dict] | None = None,
             owner_ref: str | None = None, visibility: str = "unlisted") -> dict:
        if not self.enabled or not opted_in:
            return {"emitted": False, "reason": "disabled"}
        try:
            steps = []
            for m in messages:
                src = {"user": "user", "system": "system"}.get(m.get("role"), "agent")
                steps.append({"step_id": len(steps) + 1, "source": src, "message": str(m.get("content") or "")})
            last = {"step_id": len(steps) + 1, "source": "agent", "message": assistant_text, "model_name": self.public_model_name}
            if tool_calls:
                last["tool_calls"] = [{"tool_call_id": c.get("id", f"call_{i}"), "function_name": c.get("function", {}).get("name", ""),
                                       "arguments": c.get("function", {}).get("arguments", "")} for i, c in enumerate(tool_calls)]
            steps.append(last)
            traj = {"schema_version": "ATIF-v1.7", "session_id": uuid.uuid4().hex,
                    "agent": {"name": "khala-chat", "version": "1", "model_name": self.public_model_name}, "steps": steps,
                    "extra": {"reward_eligible": False, "consent": "withheld"}}
            traj, hits = redact(traj)
            errs = validate_trajectory(traj)
            if errs:
                return {"emitted": False, "reason": "invalid:" + ",".join(errs)}
            if _UNSAFE.search(json.dumps(traj)):          # tripwire: anything credential-shaped left means reject, not store
                return {"emitted": False, "reason": "tripwire"}
            tid = str(uuid.uuid4())
            self.store[tid] = {"trajectory": traj, "visibility": visibility, "ownerRef": owner_ref, "redactions": hits}
            return {"emitted": True, "traceId": tid, "path": f"/trace/{tid}", "redactions": hits}
        except Exception as e:      # noqa: BLE001 - fail soft: the completion has already been delivered
            return {"emitted": False, "reason": f"error:{type(e).__name__}"}
