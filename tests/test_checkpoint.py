"""Checkpoint layout: digests, tamper detection, aborted saves, re-sharding (CPU)."""
import os

import pytest
import torch

from openagents_b200.control import seal
from openagents_b200.train import checkpoint as ck


def _save(d, world=2, shard=64):
    g = torch.Generator().manual_seed(0)
    files, state = {}, []
    for r in range(world):
        w, m, v = (torch.randn(shard, generator=g) for _ in range(3))
        state.append((w, m, v))
        files.update(ck.save_shard(d, r, w, m, v))
    man = ck.write_manifest(d, files, run_ref="run.t", window_ref="run.t.w0", step=7, world_size=world, zero_stage=2,
                            n_total=world * shard, shard=shard, term=1, train_config={"lr": 1e-3}, model_config={"d": 8})
    return man, state


def test_roundtrip_and_reshard(tmp_path):
    d = str(tmp_path / "ck")
    man, state = _save(d)
    assert sorted(os.listdir(d)) == ["manifest.json", "model-rank0.bin", "model-rank1.bin", "optim-rank0.bin", "optim-rank1.bin"]
    assert all(seal.DIGEST_PATTERN.match(v["digest"]) for v in man["files"].values())
    man2, master, m, v = ck.load_full(d)
    assert man2["step"] == 7 and man2["term"] == 1 and man2["checkpointDigestRef"] == man["checkpointDigestRef"]
    assert torch.equal(master, torch.cat([s[0] for s in state])) and torch.equal(v, torch.cat([s[2] for s in state]))
    # 2 ranks -> 4 ranks
    parts = [ck.reshard(master, 128, 4, r) for r in range(4)]
    assert torch.equal(torch.cat(parts), master)
    # padding when the new layout is longer
    assert ck.reshard(master, 160, 4, 3).shape == (40,) and float(ck.reshard(master, 160, 4, 3)[-8:].abs().sum()) == 0.0


def test_tamper_and_abort_are_detected(tmp_path):
    d = str(tmp_path / "ck")
    _save(d)
    p = os.path.join(d, "optim-rank1.bin")
    b = bytearray(open(p, "rb").read())
    b[10] ^= 1
    open(p, "wb").write(bytes(b))
    with pytest.raises(ck.CheckpointError, match="digest mismatch"):
        ck.verify(d)
    d2 = str(tmp_path / "aborted")
    ck.save_shard(d2, 0, torch.zeros(8), torch.zeros(8), torch.zeros(8))     # shards but no manifest
    with pytest.raises(ck.CheckpointError, match="no manifest"):
        ck.load_manifest(d2)


def test_local_checkpoint_holds_until_replicated(tmp_path):
    d = str(tmp_path / "ck")
    man, _ = _save(d)
    local = ck.seal_descriptor(man, d)
    g = seal.evaluate(local)
    assert g.decision == seal.HOLD and "replication_factor_below_durable_minimum" in g.reasons
    durable = ck.seal_descriptor(man, d, replication_factor=2, storage_class="content_addressed_object_store",
                                 remote_store_ref="store.replicated")
    assert seal.evaluate(durable).decision == seal.SEAL
