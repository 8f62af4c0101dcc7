"""The gateway as a process: API keys, model gating, lane plans, overflow, metering and telemetry in front of one or more
model servers (``b200-serve``), over HTTP on both sides.

    b200-gateway --config gateway.json --port 8787

Routes: ``POST /v1/chat/completions`` (JSON or server-sent events), ``GET /v1/models``, ``GET /v1/quote``, ``GET /health``,
``GET /metrics`` (Prometheus text), ``GET /admin/telemetry`` (the last public telemetry blocks; needs the admin key).

The configuration file is JSON::

    {"keys":    [{"key": "sk-...", "account": "acct.1", "balance_msat": 100000, "allowed_models": null, "max_inflight": 4,
                  "premium": false, "no_meter": false}],
     "nodes":   [{"id": "openagents-network", "kind": "serve", "endpoint": "http://127.0.0.1:8080", "bearer": "node-key"},
                 {"id": "hydralisk", "kind": "openai", "endpoint": "http://10.0.0.2:8080/v1", "bearer": "...", "upstream_model": null},
                 {"id": "hydralisk-pool", "kind": "pool", "replicas": [{"replicaId": "r0", "endpoint": "...", "bearer": "...", "maxInflight": 8}]}],
     "plans":   {"tiny": ["hydralisk", "openagents-network"], "*": ["openagents-network"]},
     "pricing": [{"model": "tiny", "input_usd_per_mtok": 0.1, "output_usd_per_mtok": 0.4, "lane": "open"}],
     "gates":   [{"model": "fast", "alias_of": "tiny"}, {"model": "big", "premium": true}],
     "internal_accounts": [], "platform_funded": true, "ledger": "served_tokens.jsonl", "admin_key": "..."}

``kind: serve`` speaks the serve wire contract (``/v1/serve``: the node answers with a receipt and an exact-greedy parity
verdict, which this side checks); ``kind: openai`` speaks ``/chat/completions``; ``kind: pool`` puts several OpenAI-speaking
replicas behind one adapter id with session affinity and saturation handling.  A model without a plan row uses ``"*"``, then the
router's built-in plan for its class.

Reference: the worker that owns these routes is apps/openagents.com/workers/api/src/index.ts (``/v1/chat/completions`` wired
at :16272 to inference/chat-completions-routes.ts:2550); the pieces it strings together are restated in ``chat_route``,
``router``, ``fabric`` and ``hydralisk`` of this package.
"""
from __future__ import annotations

import argparse
import hmac
import json
import time
import urllib.parse
from http.server import BaseHTTPRequestHandler, ThreadingHTTPServer

from ..utils.cli import cli_entry
from .chat_route import ApiKey, ChatGateway, ModelGate
from .fabric import OpenAgentsNetworkAdapter, ProviderRegistry, dispatch_psionic_serve, make_http_transport
from .hydralisk import HydraliskAdapter, HydraliskPoolAdapter
from .observability import ServedTokensLedger
from .router import PricingEntry, PricingTable, select_adapter_plan

MAX_BODY_BYTES = 8 << 20


class ConfigError(ValueError):
    """The configuration file is malformed; the message names the entry."""


def _need(d, key: str, kinds, where: str):
    if not isinstance(d, dict) or not isinstance(d.get(key), kinds) or (isinstance(d.get(key), str) and not d[key].strip()):
        raise ConfigError(f"{where}: {key} is required")
    return d[key]


def build_adapter(node: dict, opener=None):
    """One ``nodes`` entry -> an adapter for the provider registry."""
    where = f"nodes[{node.get('id')!r}]" if isinstance(node, dict) else "nodes[?]"
    nid, kind = _need(node, "id", str, where), _need(node, "kind", str, where)
    kw = {"opener": opener} if opener is not None else {}
    timeout = float(node.get("timeout_s", 120.0))
    if kind == "serve":
        if nid != OpenAgentsNetworkAdapter.id:
            raise ConfigError(f"{where}: a serve-contract node is registered as {OpenAgentsNetworkAdapter.id!r}")
        endpoint = _need(node, "endpoint", str, where).rstrip("/")
        if not endpoint.endswith("/v1/serve"):
            endpoint += "/v1/serve"
        return OpenAgentsNetworkAdapter(dispatch=dispatch_psionic_serve(make_http_transport(endpoint, node.get("bearer") or "", timeout_s=timeout, **kw)))
    if kind == "openai":
        return HydraliskAdapter(nid, node.get("bearer") or "", _need(node, "endpoint", str, where), upstream_model=node.get("upstream_model"),
                                timeout_s=timeout, **kw)
    if kind == "pool":
        reps = _need(node, "replicas", list, where)
        if not reps:
            raise ConfigError(f"{where}: a pool needs at least one replica")
        out = []
        for i, r in enumerate(reps):
            rw = f"{where}.replicas[{i}]"
            rid = _need(r, "replicaId", str, rw)
            out.append({**{k: v for k, v in r.items() if k not in ("endpoint", "bearer", "upstream_model")},
                        "replicaId": rid, "maxInflight": int(r.get("maxInflight", 8)),
                        "adapter": HydraliskAdapter(f"{nid}.{rid}", r.get("bearer") or "", _need(r, "endpoint", str, rw),
                                                    upstream_model=r.get("upstream_model"), timeout_s=timeout, **kw)})
        return HydraliskPoolAdapter(nid, out, saturation_policy=node.get("saturation_policy"))
    raise ConfigError(f"{where}: kind must be serve, openai or pool")


def build_gateway(cfg: dict, opener=None) -> ChatGateway:
    if not isinstance(cfg, dict):
        raise ConfigError("the configuration must be a JSON object")
    keys = []
    for i, k in enumerate(_need(cfg, "keys", list, "config")):
        where = f"keys[{i}]"
        allowed = k.get("allowed_models") if isinstance(k, dict) else None
        if allowed is not None and not (isinstance(allowed, list) and all(isinstance(m, str) for m in allowed)):
            raise ConfigError(f"{where}: allowed_models must be a list of model ids or null")
        keys.append(ApiKey(_need(k, "key", str, where), _need(k, "account", str, where), int(k.get("balance_msat", 0)),
                           tuple(allowed) if allowed is not None else None, int(k.get("max_inflight", 4)), byok=k.get("byok"),
                           premium=bool(k.get("premium")), no_meter=bool(k.get("no_meter"))))
    if len({k.key for k in keys}) != len(keys):
        raise ConfigError("keys: the same key appears twice")
    reg = ProviderRegistry()
    for node in _need(cfg, "nodes", list, "config"):
        reg.register(build_adapter(node, opener))
    ids = list(reg.ids())
    if not ids:
        raise ConfigError("nodes: at least one node is required")
    pricing = None
    if cfg.get("pricing"):
        try:
            pricing = PricingTable([PricingEntry(**e) for e in cfg["pricing"]])
        except TypeError as e:
            raise ConfigError(f"pricing: {e}")
    plans = cfg.get("plans") or {}
    if not isinstance(plans, dict) or not all(isinstance(v, list) and all(a in ids for a in v) for v in plans.values()):
        raise ConfigError(f"plans: every plan is a list of node ids ({', '.join(ids)})")

    def plan(model: str):
        if model in plans:
            return tuple(plans[model])
        if "*" in plans:
            return tuple(plans["*"])
        built_in = tuple(a for a in select_adapter_plan(model, pricing) if a in ids)
        return built_in or tuple(ids)

    gates = []
    for i, g in enumerate(cfg.get("gates") or []):
        gates.append(ModelGate(_need(g, "model", str, f"gates[{i}]"), premium=bool(g.get("premium")), internal_only=bool(g.get("internal_only")),
                               servable=bool(g.get("servable", True)), alias_of=g.get("alias_of")))
    ledger = ServedTokensLedger(cfg.get("ledger") or None)
    return ChatGateway(reg, keys, pricing=pricing, plan=plan, sleep=lambda ms: time.sleep(ms / 1000.0), gates=gates,
                       internal_accounts=tuple(cfg.get("internal_accounts") or ()), ledger=ledger,
                       platform_funded=bool(cfg.get("platform_funded", True)))


def metrics_text(gw: ChatGateway) -> str:
    with gw.lock:
        by_route = {k: list(v) for k, v in gw.route_totals.items()}
    out = []
    for route, (n, pt, ct, msat) in sorted(by_route.items()):
        lab = f'{{route="{route}"}}'
        out += [f"b200_gateway_requests_total{lab} {n}", f"b200_gateway_prompt_tokens_total{lab} {pt}",
                f"b200_gateway_completion_tokens_total{lab} {ct}", f"b200_gateway_price_msat_total{lab} {msat}"]
    out.append(f"b200_gateway_keys {len(gw.keys)}")
    out.append(f"b200_gateway_inflight {sum(k.inflight for k in gw.keys.values())}")
    if gw.ledger is not None:
        out.append(f"b200_gateway_tokens_served_total {gw.ledger.total()}")
    return "\n".join(out) + "\n"


def make_handler(gw: ChatGateway, admin_key: str | None = None):
    class H(BaseHTTPRequestHandler):
        protocol_version = "HTTP/1.1"

        def log_message(self, *a):
            pass

        def _send(self, code: int, data: bytes, ctype: str, headers: dict | None = None):
            self.send_response(code)
            self.send_header("Content-Type", ctype)
            self.send_header("Content-Length", str(len(data)))
            for k, v in (headers or {}).items():
                self.send_header(k, v)
            self.end_headers()
            self.wfile.write(data)

        def _json(self, code: int, obj, headers: dict | None = None):
            self._send(code, json.dumps(obj).encode(), "application/json", headers)

        def _err(self, code: int, kind: str, msg: str):
            self._json(code, {"error": {"message": msg, "type": kind, "code": kind}})

        def do_GET(self):
            url = urllib.parse.urlsplit(self.path)
            q = urllib.parse.parse_qs(url.query)
            try:
                if url.path == "/health":
                    return self._json(200, {"status": "ok", "adapters": list(gw.registry.ids())})
                if url.path == "/v1/models":
                    return self._json(200, gw.models())
                if url.path == "/metrics":
                    return self._send(200, metrics_text(gw).encode(), "text/plain; version=0.0.4")
                if url.path == "/v1/quote":
                    try:
                        model = q["model"][0]
                        pt, mt = int(q.get("prompt_tokens", ["0"])[0]), int(q.get("max_tokens", ["0"])[0])
                    except (KeyError, ValueError):
                        return self._err(400, "invalid_request", "quote needs model, prompt_tokens and max_tokens")
                    if pt < 0 or mt < 0:
                        return self._err(400, "invalid_request", "token counts cannot be negative")
                    return self._json(200, gw.quote(model, pt, mt))
                if url.path == "/admin/telemetry":
                    given = (self.headers.get("Authorization") or "").encode()
                    if not admin_key or not hmac.compare_digest(given, f"Bearer {admin_key}".encode()):
                        return self._err(404, "not_found", "not found")
                    with gw.lock:
                        recs = gw.telemetry[-100:]
                    return self._json(200, {"records": recs})
            except Exception as e:      # noqa: BLE001 - a handler that raises would close the connection without an answer
                return self._err(500, "gateway_error", f"{type(e).__name__}: {e}")
            self._err(404, "not_found", f"no route {url.path}")

        def do_POST(self):
            path = self.path.split("?")[0]
            try:
                n = int(self.headers.get("Content-Length") or 0)
            except ValueError:
                n = -1
            if n < 0 or n > MAX_BODY_BYTES:
                self.close_connection = True
                return self._err(413 if n > 0 else 400, "invalid_request", f"the body must be at most {MAX_BODY_BYTES} bytes with a Content-Length")
            raw = self.rfile.read(n) if n else b""
            if path != "/v1/chat/completions":
                return self._err(404, "not_found", f"no route {path}")
            try:
                body = raw.decode()
            except UnicodeDecodeError:
                return self._err(400, "invalid_json", "request body is not UTF-8")
            try:
                headers = {k.lower(): v for k, v in self.headers.items()}
                status, extra, out = gw.handle_with_headers(self.headers.get("Authorization"), body,
                                                            session=headers.get("x-openagents-session"), headers=headers)
            except Exception as e:      # noqa: BLE001
                return self._err(500, "gateway_error", f"{type(e).__name__}: {e}")
            if isinstance(out, list):       # server-sent events, already framed
                return self._send(status, "".join(out).encode(), "text/event-stream", {**extra, "Cache-Control": "no-cache"})
            self._json(status, out, extra)

    return H


class _Server(ThreadingHTTPServer):
    request_queue_size = 1024
    daemon_threads = True

    def handle_error(self, request, client_address):
        """A client that goes away mid-request is routine, not a traceback on stderr; anything else is still reported."""
        import sys
        if isinstance(sys.exc_info()[1], (ConnectionError, TimeoutError)):
            return
        super().handle_error(request, client_address)


def serve(gw: ChatGateway, host: str = "127.0.0.1", port: int = 8787, admin_key: str | None = None) -> ThreadingHTTPServer:
    return _Server((host, port), make_handler(gw, admin_key))


@cli_entry("b200-gateway")
def main(argv=None):
    ap = argparse.ArgumentParser(prog="b200-gateway", description=__doc__.split("\n\n")[0])
    ap.add_argument("--config", required=True, help="JSON configuration (keys, nodes, plans, pricing, gates)")
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--port", type=int, default=8787)
    ap.add_argument("--check", action="store_true", help="validate the configuration and exit")
    a = ap.parse_args(argv)
    try:
        with open(a.config) as f:
            cfg = json.load(f)
        gw = build_gateway(cfg)
    except (OSError, ValueError) as e:
        ap.exit(2, f"b200-gateway: {a.config}: {e}\n")
    if a.check:
        print(json.dumps({"ok": True, "adapters": list(gw.registry.ids()), "keys": len(gw.keys)}))
        return 0
    httpd = serve(gw, a.host, a.port, cfg.get("admin_key"))
    print(json.dumps({"event": "listening", "host": a.host, "port": httpd.server_address[1], "adapters": list(gw.registry.ids())}), flush=True)
    try:
        httpd.serve_forever()
    except KeyboardInterrupt:
        pass
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
