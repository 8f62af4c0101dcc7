"""The serving lane as an installable service with a durable root.

What the reference says about the upstream service (docs/teardowns/2026-07-21-buzz-teardown.md:660-688): it installs as a
service with ``systemd`` and ``launchd`` artifacts; a lane root keeps configuration, node identity, network state, logs and
model paths across restarts; reinstalling the service artifacts does not rotate the identity; changing the namespace or the
admission token once durable state exists is refused; the management API states the realized topology as one of
``remote_whole_request`` / ``replicated`` / ``dense_split`` / ``sparse_expert`` with a stable placement digest, host
elections carry a term, the active host, the standby set, a promotion reason and the lease state, and an unsupported
topology is a typed refusal, not "unavailable".  This module is that shell around ``b200-serve`` for one box:

    python -m openagents_b200.serve.mesh_lane install --root /var/lib/b200-lane --namespace lab --admission-token-file tok -m model.gguf --tp 4
    python -m openagents_b200.serve.mesh_lane status --root /var/lib/b200-lane
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import stat
import sys
import time
from pathlib import Path

from ..control.coordination import MeshElection
from ..utils.cli import cli_entry

ROOT_SCHEMA = "b200.mesh_lane.root.v1"
DIRS = ("config", "identity", "network", "logs", "models", "service")
CLAIM_SHAPES = {"replicated": "replicated", "tensor_sharded": "dense_split", "layer_sharded": "dense_split", "pipeline_sharded": "dense_split",
                "sparse_expert": "sparse_expert", "remote": "remote_whole_request"}
SERVICE_NAME = "b200-mesh-lane"


class MeshLaneRefusal(Exception):
    """A typed refusal: ``code`` is stable, ``detail`` is for the operator."""

    def __init__(self, code: str, detail: str = ""):
        super().__init__(f"{code}: {detail}" if detail else code)
        self.code, self.detail = code, detail


def _sha(data: bytes) -> str:
    return "sha256:" + hashlib.sha256(data).hexdigest()


def _write_private(path: Path, data: bytes):
    fd = os.open(str(path), os.O_WRONLY | os.O_CREAT | os.O_TRUNC, 0o600)
    with os.fdopen(fd, "wb") as f:
        f.write(data)


class MeshLaneRoot:
    def __init__(self, root):
        self.root = Path(root)

    # ---- identity: created once, never rotated by a reinstall
    def _identity(self) -> dict:
        key_path, pub_path = self.root / "identity" / "node_key.pem", self.root / "identity" / "node.json"
        if pub_path.exists():
            return json.loads(pub_path.read_text())
        from cryptography.hazmat.primitives import serialization
        from cryptography.hazmat.primitives.asymmetric.ed25519 import Ed25519PrivateKey
        key = Ed25519PrivateKey.generate()
        pub = key.public_key().public_bytes(serialization.Encoding.Raw, serialization.PublicFormat.Raw)
        _write_private(key_path, key.private_bytes(serialization.Encoding.PEM, serialization.PrivateFormat.PKCS8, serialization.NoEncryption()))
        ident = {"nodeId": "node." + hashlib.sha256(pub).hexdigest()[:32], "publicKeyHex": pub.hex(), "algorithm": "ed25519",
                 "createdAt": time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime())}
        pub_path.write_text(json.dumps(ident, indent=1))
        return ident

    def sign(self, message: bytes) -> str:
        from cryptography.hazmat.primitives import serialization
        key = serialization.load_pem_private_key((self.root / "identity" / "node_key.pem").read_bytes(), password=None)
        return key.sign(message).hex()

    # ---- install / reinstall
    def install(self, namespace: str, admission_token: str, model_paths: list[str], host: str = "127.0.0.1", port: int = 8080, tp: int = 1, ep: int = 1,
                python: str = sys.executable, user: str | None = None) -> dict:
        if not namespace or not admission_token:
            raise MeshLaneRefusal("admission_material_missing", "a namespace and an admission token are required")
        if tp > 1 and ep > 1:
            raise MeshLaneRefusal("unsupported_topology", "tensor and expert sharding cannot be combined in one lane")
        for d in DIRS:
            (self.root / d).mkdir(parents=True, exist_ok=True)
        os.chmod(self.root / "identity", stat.S_IRWXU)
        cfg_path = self.root / "config" / "lane.json"
        token_digest = _sha(admission_token.encode())
        if cfg_path.exists():
            old = json.loads(cfg_path.read_text())
            if old["namespace"] != namespace:
                raise MeshLaneRefusal("namespace_change_refused", f"this root belongs to namespace {old['namespace']!r}")
            if old["admissionTokenDigest"] != token_digest:
                raise MeshLaneRefusal("admission_token_change_refused", "the admission token differs from the one the durable state was created with")
        ident = self._identity()
        models = []
        for p in model_paths:
            link = self.root / "models" / Path(p).name
            if not link.exists():
                try:
                    link.symlink_to(Path(p).resolve())
                except OSError:
                    pass
            models.append({"path": str(Path(p).resolve()), "name": Path(p).name})
        topology = "tensor_sharded" if tp > 1 else ("sparse_expert" if ep > 1 else "replicated")
        cfg = {"schema": ROOT_SCHEMA, "namespace": namespace, "admissionTokenDigest": token_digest, "nodeId": ident["nodeId"], "host": host, "port": port,
               "tp": tp, "ep": ep, "topology": topology, "models": models, "python": python, "user": user,
               "installedAt": json.loads(cfg_path.read_text())["installedAt"] if cfg_path.exists() else time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()),
               "reinstalls": (json.loads(cfg_path.read_text())["reinstalls"] + 1) if cfg_path.exists() else 0}
        cfg_path.write_text(json.dumps(cfg, indent=1))
        arts = self.service_artifacts(cfg)
        for name, text in arts.items():
            (self.root / "service" / name).write_text(text)
        join = self.root / "network" / "join_state.json"
        if not join.exists():
            join.write_text(json.dumps({"sessionGeneration": 0, "joinedNamespace": namespace, "election": {"term": 0, "activeHost": None, "standby": [], "leaseExpiresMs": 0},
                                        "promotionReason": None}, indent=1))
        return {"root": str(self.root), "nodeId": ident["nodeId"], "topology": topology, "serviceArtifacts": sorted(arts), "reinstalls": cfg["reinstalls"]}

    def config(self) -> dict:
        p = self.root / "config" / "lane.json"
        if not p.exists():
            raise MeshLaneRefusal("root_not_installed", str(self.root))
        return json.loads(p.read_text())

    def command(self, cfg: dict | None = None) -> list[str]:
        c = cfg or self.config()
        cmd = [c["python"], "-m", "openagents_b200.serve.server", "--host", c["host"], "--port", str(c["port"])]
        for m in c["models"]:
            cmd += ["-m", m["path"]]
        if c["tp"] > 1:
            cmd += ["--tp", str(c["tp"])]
        if c["ep"] > 1:
            cmd += ["--ep", str(c["ep"])]
        return cmd + ["--mesh-coordination", "enabled"]

    def service_artifacts(self, cfg: dict | None = None) -> dict[str, str]:
        c = cfg or self.config()
        cmd = self.command(c)
        unit = "\n".join([
            "[Unit]", f"Description=B200 serving lane ({c['namespace']})", "After=network-online.target", "Wants=network-online.target", "",
            "[Service]", "Type=simple", f"WorkingDirectory={self.root}", "ExecStart=" + " ".join(cmd),
            f"Environment=B200_MESH_LANE_ROOT={self.root}", f"Environment=B200_MESH_LANE_NAMESPACE={c['namespace']}",
            f"StandardOutput=append:{self.root / 'logs' / 'lane.out.log'}", f"StandardError=append:{self.root / 'logs' / 'lane.err.log'}",
            "Restart=on-failure", "RestartSec=5", "LimitMEMLOCK=infinity", *([f"User={c['user']}"] if c.get("user") else []), "",
            "[Install]", "WantedBy=multi-user.target", ""])
        args = "".join(f"    <string>{a}</string>\n" for a in cmd)
        plist = ('<?xml version="1.0" encoding="UTF-8"?>\n<!DOCTYPE plist PUBLIC "-//Apple//DTD PLIST 1.0//EN" "http://www.apple.com/DTDs/PropertyList-1.0.dtd">\n'
                 '<plist version="1.0">\n<dict>\n  <key>Label</key>\n  <string>com.openagents.' + SERVICE_NAME + '</string>\n  <key>ProgramArguments</key>\n  <array>\n' + args +
                 '  </array>\n  <key>WorkingDirectory</key>\n  <string>' + str(self.root) + '</string>\n  <key>KeepAlive</key>\n  <true/>\n  <key>StandardOutPath</key>\n  <string>' +
                 str(self.root / "logs" / "lane.out.log") + '</string>\n  <key>StandardErrorPath</key>\n  <string>' + str(self.root / "logs" / "lane.err.log") +
                 '</string>\n</dict>\n</plist>\n')
        return {SERVICE_NAME + ".service": unit, "com.openagents." + SERVICE_NAME + ".plist": plist}

    # ---- durable network state
    def begin_session(self, now_ms: int | None = None, lease_ms: int = 10_000) -> dict:
        """Called at every service start: a new session generation, and this node's heartbeat into the host election."""
        cfg = self.config()
        p = self.root / "network" / "join_state.json"
        st = json.loads(p.read_text())
        now_ms = int(time.time() * 1000) if now_ms is None else now_ms
        e = st["election"]
        el = MeshElection(e["term"], e["activeHost"], list(e["standby"]), e["leaseExpiresMs"])
        before = el.term
        role = el.heartbeat(cfg["nodeId"], now_ms, lease_ms)
        st["sessionGeneration"] += 1
        st["election"] = {"term": el.term, "activeHost": el.active_host, "standby": el.standby, "leaseExpiresMs": el.lease_expires_ms}
        if el.term != before:
            st["promotionReason"] = "first_host" if before == 0 else "lease_expired"
        p.write_text(json.dumps(st, indent=1))
        return {"sessionGeneration": st["sessionGeneration"], "role": role, "term": el.term, "promotionReason": st["promotionReason"]}

    # ---- management view
    def management_status(self, realized_topology: dict | None = None, now_ms: int | None = None) -> dict:
        """``realized_topology``: what the engine reports (``Backend.topology()``); None = the installed plan."""
        cfg = self.config()
        st = json.loads((self.root / "network" / "join_state.json").read_text())
        topo = realized_topology or {"mode": cfg["topology"], "ranks": max(cfg["tp"], cfg["ep"])}
        mode = topo.get("mode", topo.get("topology"))
        if mode not in CLAIM_SHAPES:
            raise MeshLaneRefusal("unsupported_topology", f"{mode!r} is not a topology this lane can claim")
        now_ms = int(time.time() * 1000) if now_ms is None else now_ms
        e = st["election"]
        placement = {k: topo[k] for k in sorted(topo) if k in ("mode", "topology", "ranks", "stages", "expertRanges")}
        return {"schema": "b200.mesh_lane.management_status.v1", "nodeId": cfg["nodeId"], "namespace": cfg["namespace"], "claimShape": CLAIM_SHAPES[mode],
                "realizedTopology": placement, "placementDigest": _sha(json.dumps(placement, sort_keys=True).encode()),
                "routeProvenance": {"servedBy": cfg["nodeId"], "endpoint": f"http://{cfg['host']}:{cfg['port']}", "localServedTruth": True},
                "election": {"term": e["term"], "activeHost": e["activeHost"], "standbySet": e["standby"], "promotionReason": st["promotionReason"],
                             "leaseState": "none" if e["activeHost"] is None else ("held" if now_ms < e["leaseExpiresMs"] else "expired")},
                "sessionGeneration": st["sessionGeneration"], "models": [m["name"] for m in cfg["models"]]}


@cli_entry("b200-lane")
def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m openagents_b200.serve.mesh_lane")
    sub = ap.add_subparsers(dest="cmd", required=True)
    i = sub.add_parser("install")
    i.add_argument("--root", required=True)
    i.add_argument("--namespace", required=True)
    i.add_argument("--admission-token-file", required=True)
    i.add_argument("-m", "--model", action="append", required=True)
    i.add_argument("--host", default="127.0.0.1")
    i.add_argument("--port", type=int, default=8080)
    i.add_argument("--tp", type=int, default=1)
    i.add_argument("--ep", type=int, default=1)
    i.add_argument("--user", default=None)
    for name in ("status", "unit", "start-session"):
        sub.add_parser(name).add_argument("--root", required=True)
    a = ap.parse_args(argv)
    lane = MeshLaneRoot(a.root)
    try:
        if a.cmd == "install":
            out = lane.install(a.namespace, Path(a.admission_token_file).read_text().strip(), a.model, a.host, a.port, a.tp, a.ep, user=a.user)
        elif a.cmd == "status":
            out = lane.management_status()
        elif a.cmd == "start-session":
            out = lane.begin_session()
        else:
            print(lane.service_artifacts()[SERVICE_NAME + ".service"], end="")
            return 0
    except MeshLaneRefusal as e:
        print(json.dumps({"refused": e.code, "detail": e.detail}))
        return 3
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
