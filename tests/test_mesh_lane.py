"""The serving lane's durable root: identity survives a reinstall, namespace and token changes are refused, service
artifacts, session generations with the host election, and the management view with typed refusals."""
import json
import os
import stat

import pytest

from openagents_b200.serve.mesh_lane import MeshLaneRefusal, MeshLaneRoot, main


def test_install_reinstall_and_refusals(tmp_path):
    lane = MeshLaneRoot(tmp_path / "lane")
    (tmp_path / "m.gguf").write_bytes(b"x")
    a = lane.install("lab", "secret-token", [str(tmp_path / "m.gguf")], port=9001, tp=4)
    assert a["topology"] == "tensor_sharded" and a["reinstalls"] == 0 and a["nodeId"].startswith("node.")
    key = (tmp_path / "lane" / "identity" / "node_key.pem")
    assert stat.S_IMODE(os.stat(key).st_mode) == 0o600 and b"PRIVATE KEY" in key.read_bytes()
    assert "secret-token" not in (tmp_path / "lane" / "config" / "lane.json").read_text()          # only its digest is kept
    b = lane.install("lab", "secret-token", [str(tmp_path / "m.gguf")], port=9002, tp=2)           # reinstall: new port, same identity
    assert b["nodeId"] == a["nodeId"] and b["reinstalls"] == 1 and lane.config()["port"] == 9002
    with pytest.raises(MeshLaneRefusal) as e:
        lane.install("other", "secret-token", [str(tmp_path / "m.gguf")])
    assert e.value.code == "namespace_change_refused"
    with pytest.raises(MeshLaneRefusal) as e:
        lane.install("lab", "another-token", [str(tmp_path / "m.gguf")])
    assert e.value.code == "admission_token_change_refused"
    with pytest.raises(MeshLaneRefusal) as e:
        lane.install("lab", "secret-token", [str(tmp_path / "m.gguf")], tp=2, ep=2)
    assert e.value.code == "unsupported_topology"
    with pytest.raises(MeshLaneRefusal) as e:
        MeshLaneRoot(tmp_path / "nothing").config()
    assert e.value.code == "root_not_installed"
    # a signature by the node key verifies under the published public key
    from cryptography.hazmat.primitives.asymmetric.ed25519 import Ed25519PublicKey
    ident = json.loads((tmp_path / "lane" / "identity" / "node.json").read_text())
    Ed25519PublicKey.from_public_bytes(bytes.fromhex(ident["publicKeyHex"])).verify(bytes.fromhex(lane.sign(b"hello")), b"hello")


def test_service_artifacts_sessions_and_management_view(tmp_path, capsys):
    (tmp_path / "m.gguf").write_bytes(b"x")
    (tmp_path / "tok").write_text("secret-token\n")
    root = str(tmp_path / "lane")
    assert main(["install", "--root", root, "--namespace", "lab", "--admission-token-file", str(tmp_path / "tok"), "-m", str(tmp_path / "m.gguf"), "--ep", "8"]) == 0
    capsys.readouterr()
    lane = MeshLaneRoot(root)
    unit = (tmp_path / "lane" / "service" / "b200-mesh-lane.service").read_text()
    assert "-m openagents_b200.serve.server" in unit and "--ep 8" in unit and f"WorkingDirectory={root}" in unit and "Restart=on-failure" in unit
    assert "<key>ProgramArguments</key>" in (tmp_path / "lane" / "service" / "com.openagents.b200-mesh-lane.plist").read_text()
    s1 = lane.begin_session(now_ms=1_000)
    assert s1 == {"sessionGeneration": 1, "role": "elected", "term": 1, "promotionReason": "first_host"}
    s2 = lane.begin_session(now_ms=5_000)
    assert s2["sessionGeneration"] == 2 and s2["role"] == "active" and s2["term"] == 1
    st = lane.management_status(now_ms=6_000)
    assert st["claimShape"] == "sparse_expert" and st["election"]["leaseState"] == "held" and st["election"]["activeHost"] == st["nodeId"]
    assert st["placementDigest"].startswith("sha256:") and st["sessionGeneration"] == 2
    assert lane.management_status(now_ms=10 ** 9)["election"]["leaseState"] == "expired"
    tp = lane.management_status({"mode": "tensor_sharded", "ranks": 4, "stages": [{"nodeRef": "box", "layerStart": 0, "layerEnd": 32, "role": "stage"}]})
    assert tp["claimShape"] == "dense_split" and tp["placementDigest"] != st["placementDigest"]
    with pytest.raises(MeshLaneRefusal) as e:
        lane.management_status({"mode": "ring_of_phones"})
    assert e.value.code == "unsupported_topology"
    assert main(["install", "--root", root, "--namespace", "elsewhere", "--admission-token-file", str(tmp_path / "tok"), "-m", str(tmp_path / "m.gguf")]) == 3
    assert json.loads(capsys.readouterr().out)["refused"] == "namespace_change_refused"
    assert main(["status", "--root", root]) == 0 and json.loads(capsys.readouterr().out)["namespace"] == "lab"
