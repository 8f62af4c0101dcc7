"""Measured-or-sentinel telemetry values and a small Prometheus histogram.

Every number in a report is either measured or the explicit ``not_measured`` sentinel, never a
silent zero (reference: apps/openagents.com/workers/api/src/inference/khala-telemetry.ts:14-24,
86-94).
"""
from __future__ import annotations

import bisect
import math

NOT_MEASURED = "not_measured"


def not_measured() -> dict:
    return {"state": NOT_MEASURED}


def measured(value: float, unit: str | None = None) -> dict:
    if value is None or not isinstance(value, (int, float)) or not math.isfinite(value):
        return not_measured()
    d = {"state": "measured", "value": value}
    if unit:
        d["unit"] = unit
    return d


def is_measured(v) -> bool:
    return isinstance(v, dict) and v.get("state") == "measured"


class Histogram:
    def __init__(self, bounds: list[float]):
        self.bounds = sorted(bounds)
        self.counts = [0] * (len(self.bounds) + 1)
        self.sum, self.n = 0.0, 0

    def observe(self, v: float):
        self.counts[bisect.bisect_left(self.bounds, v)] += 1
        self.sum += v
        self.n += 1

    def quantile(self, q: float):
        """Nearest-rank quantile over bucket upper bounds (None when empty)."""
        if not self.n:
            return None
        rank, acc = max(1, math.ceil(q * self.n)), 0
        for i, c in enumerate(self.counts):
            acc += c
            if acc >= rank:
                return self.bounds[i] if i < len(self.bounds) else math.inf
        return math.inf

    def prometheus(self, name: str) -> list[str]:
        out, acc = [], 0
        for b, c in zip(self.bounds, self.counts):
            acc += c
            out.append(f'{name}_bucket{{le="{b}"}} {acc}')
        out.append(f'{name}_bucket{{le="+Inf"}} {self.n}')
        out += [f"{name}_sum {self.sum}", f"{name}_count {self.n}"]
        return out
