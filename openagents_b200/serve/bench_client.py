"""HTTP benchmark client and serving preflight for an OpenAI-compatible endpoint (stdlib only).

Benchmark: six scenarios x N repetitions of a streamed ``/chat/completions`` call at temperature 0.
Per call: time to the first content-or-reasoning token (TTFT), time to first visible content, total time,
completion tokens per second from the first token and end to end, the server's own ``timings``, whether the
expected string appears.  A sampler thread records the resident memory of the server's process tree once a
second.  Reference: docs/muse/benchmarks/run_llama_cpp_benchmark.py:29-123 (scenarios), :135-184 (sampler),
:196-311 (streamed call), :392-406 (document).

Preflight: an owner-gated known-answer run against a live endpoint that emits self-benchmark, serve, replay
and capability evidence with digests only: never the endpoint URL, the key, the prompt or the raw output.
Reference: apps/pylon/scripts/real-serving-preflight.ts:1-60 (contract), :170-341 (flow).

    python -m openagents_b200.serve.bench_client bench --base-url http://127.0.0.1:8000/v1 --server-pid PID --output out.json
    B200_SERVING_BENCH=1 B200_SERVING_ENDPOINT=... B200_SERVING_OWNER_APPROVAL_REF=... python -m openagents_b200.serve.bench_client preflight
"""
from __future__ import annotations

import argparse
import base64
import hashlib
import json
import os
import platform
import sys
import threading
import time
import urllib.error
import urllib.request
from pathlib import Path

from ..utils.cli import cli_entry

BENCH_SCHEMA = "openagents.muse.chat_completions_benchmark.v2"
PREFLIGHT_SCHEMA = "openagents.pylon.live_serving_preflight_run.v0.1"


def long_context(n: int = 1200, needle_at: int = 731, needle: str = "LANTERN-4821") -> str:
    rows = []
    for i in range(n):
        value = needle if i == needle_at else f"FILLER-{(i * 7919) % 10000:04d}"
        rows.append(f"Entry {i:04d}: region {i % 17}, shelf {i % 29}, verification value {value}.")
    return "\n".join(rows)


def scenarios() -> list[dict]:
    u = lambda s: [{"role": "user", "content": s}]
    return [
        {"name": "exact_instruction", "messages": u("Reply with exactly: muse-ready"), "reasoning_effort": "low", "max_tokens": 128, "expected": "muse-ready"},
        {"name": "code_generation", "messages": u("Write a Python function named stable_unique that returns items in first-seen order without using set "
                                                  "on the items. Include type hints and three assert examples. Return code only."),
         "reasoning_effort": "medium", "max_tokens": 256, "expected": "stable_unique"},
        {"name": "reasoning", "messages": u("A farmer must move a wolf, a goat, and a cabbage across a river. The boat carries the farmer and one item. "
                                            "The wolf cannot stay with the goat, and the goat cannot stay with the cabbage. Give the shortest valid "
                                            "crossing sequence and state its number of trips."),
         "reasoning_effort": "high", "max_tokens": 384, "expected": "7"},
        {"name": "long_context_retrieval", "messages": u("Read the records below. Return only the verification value from Entry 0731.\n\n" + long_context()),
         "reasoning_effort": "low", "max_tokens": 128, "expected": "LANTERN-4821"},
        {"name": "multi_turn_memory", "messages": [{"role": "user", "content": "Remember that this project's codename is cobalt-orchid."},
                                                   {"role": "assistant", "content": "I will remember the project codename."},
                                                   {"role": "user", "content": "What is the codename? Return only the codename."}],
         "reasoning_effort": "low", "max_tokens": 128, "expected": "cobalt-orchid"},
        {"name": "structured_json", "messages": u("Return one compact JSON object with keys model, local, and capabilities. Set model to muse-glimmer, "
                                                  "local to true, and capabilities to an array containing chat and reasoning. No prose."),
         "reasoning_effort": "medium", "max_tokens": 192, "expected": "muse-glimmer"},
    ]


def process_tree_rss_kib(root_pid: int, proc: str = "/proc") -> int:
    """Resident memory of a process and all its descendants, from /proc/<pid>/stat (ppid) and statm (pages)."""
    table = {}
    for entry in os.listdir(proc):
        if not entry.isdigit():
            continue
        try:
            stat = Path(proc, entry, "stat").read_text()
            ppid = int(stat[stat.rindex(")") + 2:].split()[1])
            pages = int(Path(proc, entry, "statm").read_text().split()[1])
        except (OSError, ValueError, IndexError):
            continue
        table[int(entry)] = (ppid, pages)
    tree, grew = {root_pid}, True
    while grew:
        more = {p for p, (pp, _) in table.items() if pp in tree} - tree
        grew = bool(more)
        tree |= more
    page_kib = os.sysconf("SC_PAGE_SIZE") // 1024 if hasattr(os, "sysconf") else 4
    return sum(table[p][1] for p in tree if p in table) * page_kib


class MemorySampler:
    def __init__(self, pid: int, period_s: float = 1.0, probe=process_tree_rss_kib):
        self.pid, self.period, self.probe, self.samples_kib = pid, period_s, probe, []
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while True:                      # first sample at once, so that a run shorter than the period still has one
            kib = self.probe(self.pid)
            if kib:
                self.samples_kib.append(kib)
            if self._stop.wait(self.period):
                return

    def start(self):
        self._thread.start()

    def finish(self) -> dict:
        self._stop.set()
        self._thread.join()
        return {"samples": len(self.samples_kib), "peak_rss_kib": max(self.samples_kib) if self.samples_kib else None}


def consume_stream(lines, started: float, clock=time.perf_counter) -> dict:
    """Fold ``data:`` lines of a chat-completions stream into the timing record (separated out so it can be tested offline)."""
    first_token = first_content = None
    content, reasoning, finish, usage, timings, events = [], [], None, None, None, 0
    for raw in lines:
        line = (raw.decode("utf-8") if isinstance(raw, bytes) else raw).strip()
        if not line.startswith("data: "):
            continue
        data = line[6:]
        if data == "[DONE]":
            break
        ev = json.loads(data)
        events += 1
        choice = (ev.get("choices") or [{}])[0]
        delta = choice.get("delta") or {}
        c, r = delta.get("content") or "", delta.get("reasoning_content") or ""
        if first_token is None and (c or r):
            first_token = clock()
        if first_content is None and c:
            first_content = clock()
        content.append(c)
        reasoning.append(r)
        finish = choice.get("finish_reason") or finish
        usage = ev.get("usage") or usage
        timings = ev.get("timings") or timings
    finished = clock()
    n = (usage or {}).get("completion_tokens")
    decode_s = None if first_token is None else finished - first_token
    return {"finish_reason": finish, "event_count": events, "ttft_seconds": None if first_token is None else first_token - started,
            "first_content_seconds": None if first_content is None else first_content - started, "total_seconds": finished - started,
            "observed_decode_seconds": decode_s,
            "observed_completion_per_second": n / decode_s if n is not None and decode_s else None,
            "end_to_end_completion_per_second": n / (finished - started) if n is not None and finished > started else None,
            "visible_output": "".join(content), "reasoning_output": "".join(reasoning), "usage": usage, "timings": timings}


def streamed_chat(base_url: str, api_key: str, model: str, scenario: dict, repetition: int, max_tokens=None, reasoning_control: str = "api",
                  seed=None, opener=urllib.request.urlopen) -> dict:
    payload = {"model": model, "messages": scenario["messages"], "temperature": 0, "max_tokens": max_tokens or scenario["max_tokens"],
               "stream": True, "stream_options": {"include_usage": True}}
    if seed is not None:
        payload["seed"] = seed
    if reasoning_control == "api":
        payload["reasoning_effort"] = scenario["reasoning_effort"]
    else:
        payload["chat_template_kwargs"] = {"reasoning_strength": scenario["reasoning_effort"], "return_reasoning": True}
    req = urllib.request.Request(f"{base_url}/chat/completions", data=json.dumps(payload).encode(), method="POST",
                                 headers={"Authorization": f"Bearer {api_key}", "Content-Type": "application/json"})
    started = time.perf_counter()
    status, error, rec = None, None, None
    try:
        with opener(req, timeout=300) as resp:
            status = getattr(resp, "status", 200)
            rec = consume_stream(resp, started)
    except (urllib.error.URLError, TimeoutError, json.JSONDecodeError) as e:
        status, error = getattr(e, "code", None), f"{type(e).__name__}: {e}"
        rec = consume_stream([], started)
    rec.update({"scenario": scenario["name"], "repetition": repetition, "request": payload, "http_status": status, "error": error,
                "expected": scenario["expected"], "expected_observed": scenario["expected"].lower() in rec["visible_output"].lower()})
    return rec


def summarize(results: list[dict]) -> dict:
    """Per scenario: medians of TTFT and decode rate over the repetitions that returned 200."""
    def med(v):
        v = sorted(x for x in v if x is not None)
        return None if not v else v[len(v) // 2] if len(v) % 2 else (v[len(v) // 2 - 1] + v[len(v) // 2]) / 2
    out = {}
    for name in dict.fromkeys(r["scenario"] for r in results):
        rs = [r for r in results if r["scenario"] == name and r["http_status"] == 200]
        out[name] = {"ok": len(rs), "ttft_seconds_median": med([r["ttft_seconds"] for r in rs]),
                     "decode_tok_s_median": med([(r["timings"] or {}).get("predicted_per_second") or r["observed_completion_per_second"] for r in rs]),
                     "expected_observed": sum(1 for r in rs if r["expected_observed"])}
    return out


def run_benchmark(base_url, api_key, model, configuration, repetitions=3, seed=42, only=None, max_tokens=None, reasoning_control="api",
                  server_pid=None, opener=urllib.request.urlopen, log=None) -> dict:
    sampler = MemorySampler(server_pid) if server_pid else None
    if sampler:
        sampler.start()
    results = []
    for sc in scenarios():
        if only and sc["name"] not in only:
            continue
        for rep in range(1, repetitions + 1):
            r = streamed_chat(base_url, api_key, model, sc, rep, max_tokens, reasoning_control, seed, opener)
            results.append(r)
            if log:
                log(json.dumps({"scenario": r["scenario"], "repetition": rep, "status": r["http_status"], "ttft_seconds": r["ttft_seconds"],
                                "total_seconds": r["total_seconds"], "predicted_per_second": (r["timings"] or {}).get("predicted_per_second"),
                                "observed_completion_per_second": r["observed_completion_per_second"], "expected_observed": r["expected_observed"]}))
    return {"schema": BENCH_SCHEMA, "configuration": configuration, "captured_at": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()),
            "environment": {"platform": platform.platform(), "python": platform.python_version()}, "model": model,
            "memory": sampler.finish() if sampler else None, "summary": summarize(results), "results": results}


# ---------------------------------------------------------------- preflight
def digest_b64url(text: str) -> str:
    return base64.urlsafe_b64encode(hashlib.sha256(text.encode()).digest()).rstrip(b"=").decode()


def call_completion(endpoint, api_key, model_ref, prompt, max_new_tokens, opener=urllib.request.urlopen) -> dict:
    headers = {"content-type": "application/json"}
    if api_key:
        headers["authorization"] = f"Bearer {api_key}"
    body = {"model": model_ref, "messages": [{"role": "user", "content": prompt}], "max_tokens": max_new_tokens, "temperature": 0}
    t0 = time.perf_counter()
    with opener(urllib.request.Request(endpoint, data=json.dumps(body).encode(), headers=headers, method="POST"), timeout=300) as resp:
        obj = json.load(resp)
    ms = max(1, int((time.perf_counter() - t0) * 1000))
    ch = (obj.get("choices") or [{}])[0]
    text = (ch.get("message") or {}).get("content") or ch.get("text") or ""
    usage = obj.get("usage") or {}
    n = usage.get("completion_tokens", usage.get("total_tokens"))
    return {"outputDigest": digest_b64url(text.strip()), "wallClockMs": ms, "promptTokens": usage.get("prompt_tokens", 0),
            "completionTokens": n if isinstance(n, (int, float)) and n >= 0 else max(1, len(text.split())), "model": obj.get("model", model_ref)}


def run_preflight(env=None, opener=urllib.request.urlopen, now=None) -> dict:
    """Owner-gated: refuses to run unless the bench flag, the endpoint and an owner approval ref are present."""
    env = os.environ if env is None else env
    get = lambda k, d=None: (env.get(k) or "").strip() or d
    if get("B200_SERVING_BENCH") != "1":
        raise PermissionError("B200_SERVING_BENCH=1 is required")
    endpoint, approval = get("B200_SERVING_ENDPOINT"), get("B200_SERVING_OWNER_APPROVAL_REF")
    if not endpoint or not approval:
        raise PermissionError("B200_SERVING_ENDPOINT and B200_SERVING_OWNER_APPROVAL_REF are required")
    model_ref, engine = get("B200_SERVING_MODEL_REF", "model.default"), get("B200_SERVING_ENGINE", "openagents_b200")
    prompt, expected = get("B200_SERVING_SELF_BENCH_PROMPT", "Respond with exactly OK and nothing else."), get("B200_SERVING_EXPECTED_OUTPUT", "OK")
    max_new = int(get("B200_SERVING_MAX_NEW_TOKENS", "1"))
    observed = now or time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())
    want = digest_b64url(expected)
    bench = call_completion(endpoint, get("B200_SERVING_API_KEY"), model_ref, prompt, max_new, opener)
    serve = call_completion(endpoint, get("B200_SERVING_API_KEY"), model_ref, prompt, max_new, opener)
    replay = call_completion(endpoint, get("B200_SERVING_API_KEY"), model_ref, prompt, max_new, opener)
    parity, replay_ok = serve["outputDigest"] == want, replay["outputDigest"] == serve["outputDigest"]
    metrics = {"ttftMs": serve["wallClockMs"], "tokensPerSecond": round(serve["completionTokens"] / (serve["wallClockMs"] / 1000), 6),
               "promptTokens": serve["promptTokens"], "completionTokens": serve["completionTokens"], "wallClockMs": serve["wallClockMs"]}
    blockers = ([] if bench["outputDigest"] == want else ["blocker.serving.self_benchmark_known_answer_failed"]) \
        + ([] if parity else ["blocker.serving.canary_failed"]) + ([] if replay_ok else ["blocker.serving.replay_mismatch"])
    return {"schema": PREFLIGHT_SCHEMA, "observedAt": observed, "endpointRef": "endpoint.redacted.openai_compatible.local_or_owner_supplied",
            "ownerApprovalRef": approval, "modelRef": model_ref, "engine": engine, "quantization": get("B200_SERVING_QUANTIZATION", "q4_k"),
            "gpuClass": get("B200_SERVING_GPU_CLASS", "accelerator.nvidia_b200"),
            "selfBenchmark": {"workloadRef": "workload.pylon.serving.self_bench.known_answer.v1", "passed": bench["outputDigest"] == want,
                              "wallClockMs": bench["wallClockMs"], "receiptRef": "receipt.serving.self_bench." + hashlib.sha256(
                                  f"{model_ref}|{engine}|{bench['outputDigest']}".encode()).hexdigest()[:16]},
            "servingReceipt": {"promptDigest": digest_b64url(prompt), "outputDigest": serve["outputDigest"], "maxNewTokens": max_new, "temperature": 0,
                               "metrics": metrics, "verification": {"parityPassed": parity, "canaryRef": "canary.pylon.serving.known_answer.ok.v1",
                                                                    "canaryPassed": parity, "replayMatched": replay_ok}},
            "ready": not blockers, "blockerRefs": blockers}


@cli_entry("b200-serve-bench")
def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="b200-serve-bench")
    sub = ap.add_subparsers(dest="cmd", required=True)
    b = sub.add_parser("bench")
    b.add_argument("--base-url", default="http://127.0.0.1:8000/v1")
    b.add_argument("--api-key", default="local")
    b.add_argument("--model", default="default")
    b.add_argument("--configuration", default="openagents_b200")
    b.add_argument("--repetitions", type=int, default=3)
    b.add_argument("--seed", type=int, default=42)
    b.add_argument("--omit-seed", action="store_true")
    b.add_argument("--scenario", action="append")
    b.add_argument("--max-tokens", type=int)
    b.add_argument("--reasoning-control", choices=("api", "template"), default="api")
    b.add_argument("--server-pid", type=int)
    b.add_argument("--output", type=Path, required=True)
    sub.add_parser("preflight")
    a = ap.parse_args(argv)
    if a.cmd == "preflight":
        print(json.dumps(run_preflight(), indent=1))
        return 0
    doc = run_benchmark(a.base_url, a.api_key, a.model, a.configuration, a.repetitions, None if a.omit_seed else a.seed, a.scenario, a.max_tokens,
                        a.reasoning_control, a.server_pid, log=lambda s: print(s, flush=True))
    a.output.write_text(json.dumps(doc, indent=1))
    return 0


if __name__ == "__main__":
    sys.exit(main())
