"""The training assignment manifest: pinning, validation, lowering to launcher flags, receipts, and the refusal paths."""
import json
import os

import pytest

from openagents_b200.train import assignment_manifest as am
from openagents_b200.train.launcher import parse, run_manifest


def _files(tmp_path):
    (tmp_path / "chats.jsonl").write_text(json.dumps({"messages": [{"role": "user", "content": "hi"}, {"role": "assistant", "content": "hello"}]}) + "\n")
    (tmp_path / "pairs.jsonl").write_text(json.dumps({"messages": [{"role": "user", "content": "pick"}], "chosen": "a", "rejected": "b"}) + "\n")
    (tmp_path / "train-00000.b2tk").write_bytes(b"B2TK" + b"\x00" * 60)
    return tmp_path


def test_manifest_pins_inputs_and_lowers_to_flags(tmp_path):
    d = _files(tmp_path)
    m = am.make_manifest("assignment.sft.1", "sft", [{"role": "records", "path": str(d / "chats.jsonl")}], steps=12, layers=2, global_batch=8, micro_batch=4, seq_len=64)
    assert am.validate(m) == [] and am.verify_inputs(m) == [] and m["inputs"][0]["sha256"].startswith("sha256:") and m["manifestDigest"].startswith("sha256:")
    argv = am.launcher_argv(m, str(d / "work"))
    a = parse(argv)                                         # the flags are ones the launcher really has
    assert a.lane == "sft" and a.steps == 12 and a.layers == 2 and a.sft_records == str(d / "chats.jsonl") and a.export_gguf.endswith("model.gguf") and a.total_steps == 12
    pre = am.make_manifest("assignment.pre.1", "pretrain", [{"role": "shard", "path": str(d / "train-00000.b2tk")}], steps=3, global_batch=32, micro_batch=16)
    ap = parse(am.launcher_argv(pre, str(d / "w2")))
    assert ap.data == [str(d / "train-00000.b2tk")] and ap.lane == "pretrain"
    dpo = am.make_manifest("assignment.dpo.1", "dpo", [{"role": "pairs", "path": str(d / "pairs.jsonl")}], steps=3, global_batch=32, micro_batch=16, beta=0.3)
    ad = parse(am.launcher_argv(dpo, str(d / "w3")))
    assert ad.beta == 0.3 and ad.dpo_pairs.endswith("pairs.jsonl") and not ad.export_gguf
    # refusals
    assert am.validate({"schema": "other"}) == ["blocker.training_assignment.schema"]
    assert "blocker.training_assignment.missing_input.pairs" in am.validate({**dpo, "inputs": []})
    tampered = {**m, "budget": {"steps": 99, "maxWallSeconds": 10}}
    assert am.validate(tampered) == ["blocker.training_assignment.manifest_digest_mismatch"]
    bad_geo = am.make_manifest("assignment.x", "pretrain", [], steps=1, global_batch=10, micro_batch=4)
    assert "blocker.training_assignment.batch_geometry" in am.validate(bad_geo)
    (d / "chats.jsonl").write_text("changed\n")
    assert am.verify_inputs(m) == [f"blocker.training_assignment.input_digest_mismatch.{m['inputs'][0]['ref']}"]


def test_refused_assignment_still_closes_with_a_receipt(tmp_path, capsys):
    d = _files(tmp_path)
    m = am.make_manifest("assignment.sft.2", "sft", [{"role": "records", "path": str(d / "chats.jsonl")}], steps=2, global_batch=8, micro_batch=4, seq_len=64)
    (d / "chats.jsonl").write_text("someone swapped the data\n")
    (d / "m.json").write_text(json.dumps(m))
    rc = run_manifest(str(d / "m.json"), str(d / "work"))
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rc == 3 and line["status"] == "refused" and line["blockerRefs"][0].startswith("blocker.training_assignment.input_digest_mismatch")
    out = json.loads((d / "work" / "receipts.json").read_text())
    assert out["workerReceipt"]["status"] == "refused" and out["workerReceipt"]["assignmentId"] == "assignment.sft.2"
    assert out["trainingWorkerReceipt"]["trainingConfigDigest"] == m["manifestDigest"] and out["evidence"]["stepsLogged"] == 0


def test_receipts_read_the_run_directory(tmp_path):
    d = _files(tmp_path)
    m = am.make_manifest("assignment.pre.2", "pretrain", [], steps=2, global_batch=8, micro_batch=4, seq_len=64, max_wall_seconds=100)
    work = d / "work"
    (work / "ckpt" / "step00000002").mkdir(parents=True)
    (work / "ckpt" / "step00000002" / "manifest.json").write_text(json.dumps({"checkpointDigestRef": "sha256:" + "ab" * 32, "step": 2}))
    (work / "steps.jsonl").write_text("\n".join(json.dumps({"event": "step", "step": i, "loss": 10.0 - i}) for i in (1, 2)) + "\n")
    (work / "model.gguf").write_bytes(b"GGUFxxxx")
    r = am.receipts(m, str(work), "succeeded", wall_seconds=12.5)
    assert r["workerReceipt"]["status"] == "succeeded" and r["evidence"]["lastStep"] == 2 and r["evidence"]["outputs"]["checkpoint"]["dir"] == "step00000002"
    assert r["trainingWorkerReceipt"]["checkpointDigest"] == "sha256:" + "ab" * 32 and r["trainingWorkerReceipt"]["loss"] == 8.0
    assert r["trainingWorkerReceipt"]["tokensProcessed"] == 2 * 8 * 64 and r["evidence"]["outputs"]["gguf"]["bytes"] == 8
    late = am.receipts(m, str(work), "succeeded", wall_seconds=1000.0)
    assert late["workerReceipt"]["status"] == "failed" and late["evidence"]["overWallBudget"]


def test_receipts_take_the_tuning_lane_report(tmp_path):
    m = am.make_manifest("assignment.sft.3", "sft", [], steps=2, global_batch=8, micro_batch=4, seq_len=64)
    work = tmp_path / "work"
    work.mkdir()
    (work / "lane_report.json").write_text(json.dumps({"stepReceipts": [{"step": 1, "loss": 5.0, "batch": 0, "trainableTokens": 9}, {"step": 2, "loss": 4.5, "batch": 1, "trainableTokens": 9}]}))
    r = am.receipts(m, str(work), "succeeded", 3.0)
    assert r["evidence"]["lastStep"] == 2 and r["evidence"]["lastLoss"] == 4.5 and r["evidence"]["outputs"]["laneReport"]["sha256"].startswith("sha256:")


def test_accepted_assignment_runs_the_launcher_and_closes(tmp_path, capsys, monkeypatch):
    """The success path with the GPU worker replaced by a stand-in that does what a worker does to the run directory."""
    from openagents_b200.train import launcher
    d = _files(tmp_path)
    m = am.make_manifest("assignment.pre.3", "pretrain", [{"role": "shard", "path": str(d / "train-00000.b2tk")}], steps=3, layers=2, global_batch=8, micro_batch=4, seq_len=64)
    (d / "m.json").write_text(json.dumps(m))
    seen = {}

    def fake_worker(args):
        seen["args"] = args
        os.makedirs(os.path.join(args.ckpt_dir, "step00000003"), exist_ok=True)
        with open(os.path.join(args.ckpt_dir, "step00000003", "manifest.json"), "w") as f:
            json.dump({"checkpointDigestRef": "sha256:" + "cd" * 32, "step": 3}, f)
        with open(args.log_jsonl, "a") as f:
            for i in range(1, args.steps + 1):
                f.write(json.dumps({"event": "step", "step": i, "loss": 11.0 - i}) + "\n")
        with open(args.export_gguf, "wb") as f:
            f.write(b"GGUF")
    monkeypatch.setattr(launcher, "worker", fake_worker)
    with pytest.raises(SystemExit) as e:
        launcher.main(["--manifest", str(d / "m.json"), "--work-dir", str(d / "work")])
    assert e.value.code == 0
    a = seen["args"]
    assert a.steps == 3 and a.layers == 2 and a.data == [str(d / "train-00000.b2tk")] and a.global_batch == 8 and a.seq_len == 64
    line = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert line["status"] == "succeeded" and line["blockerRefs"] == []
    out = json.loads((d / "work" / "receipts.json").read_text())
    assert out["workerReceipt"]["status"] == "succeeded" and out["evidence"]["lastStep"] == 3 and out["evidence"]["outputs"]["gguf"]["bytes"] == 4
    assert out["trainingWorkerReceipt"]["checkpointDigest"] == "sha256:" + "cd" * 32 and out["trainingWorkerReceipt"]["tokensProcessed"] == 3 * 8 * 64

    def failing_worker(args):
        raise RuntimeError("device lost")
    monkeypatch.setattr(launcher, "worker", failing_worker)
    with pytest.raises(SystemExit) as e:
        launcher.main(["--manifest", str(d / "m.json"), "--work-dir", str(d / "work2")])
    assert e.value.code == 3
    out = json.loads((d / "work2" / "receipts.json").read_text())
    assert out["workerReceipt"]["status"] == "failed" and out["blockerRefs"] == ["blocker.training_assignment.run_failed.RuntimeError"]
