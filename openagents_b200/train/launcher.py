"""``b200-train``: the distributed-training launcher.

    python -m openagents_b200.train.launcher --nproc 8 --steps 20 [--ckpt-dir DIR] [--resume DIR]

With ``--nproc N > 1`` it re-executes itself under ``torch.distributed.run`` (one process per GPU,
rendezvous on 127.0.0.1); each worker then builds the trainer, walks the run/window state machine
(plan -> active -> seal -> reconcile) around its steps and, at the end of a window, writes a
checkpoint whose seal descriptor goes through the durable-seal predicate.

``--sync-profile diloco`` makes every rank a replica of its own (local-update rounds: ``--inner-steps`` optimizer steps
per round, then one outer step over all replicas; one window per round).

Flags follow the trainer contract (``--zero-stage --global-batch --seq-len --lr --betas --wd --clip
--ckpt-dir --resume``); the run/window semantics are the reference's
(apps/openagents.com/workers/api/src/training-run-window-authority.ts:43-56, 219-231).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

from ..utils.cli import cli_entry


def parse(argv=None):
    ap = argparse.ArgumentParser(prog="b200-train")
    ap.add_argument("--nproc", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--window-steps", type=int, default=0, help="optimizer steps per window (0 = one window)")
    ap.add_argument("--model", default="gpt2-small-shape")
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--zero-stage", type=int, default=2)
    ap.add_argument("--global-batch", type=int, default=512)
    ap.add_argument("--micro-batch", type=int, default=16)
    ap.add_argument("--seq-len", type=int, default=1024)
    ap.add_argument("--lr", type=float, default=6e-4)
    ap.add_argument("--betas", type=float, nargs=2, default=(0.9, 0.95))
    ap.add_argument("--wd", type=float, default=0.1)
    ap.add_argument("--clip", type=float, default=1.0)
    ap.add_argument("--schedule", default="cosine", choices=["cosine", "wsd", "constant"], help="learning-rate schedule over --total-steps")
    ap.add_argument("--total-steps", type=int, default=0, help="length of the schedule (0 = constant after warm-up)")
    ap.add_argument("--warmup-steps", type=int, default=0)
    ap.add_argument("--decay-fraction", type=float, default=0.2, help="wsd: share of the run spent decaying")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--ckpt-dir", default="")
    ap.add_argument("--resume", default="")
    ap.add_argument("--max-allowed-stale", type=int, default=5)
    ap.add_argument("--master-port", type=int, default=29517)
    ap.add_argument("--log-jsonl", default="")
    ap.add_argument("--export-gguf", default="", help="write the final weights as a GGUF file the server and the evaluator load")
    ap.add_argument("--tokenizer", default="", help="tokenizer.json of the data preparation; travels inside the exported file")
    ap.add_argument("--data", nargs="*", default=[], help="token shards (data.write_token_shard); default: synthetic uniform ids")
    ap.add_argument("--data-raw-width", type=int, default=0, choices=[0, 2, 4], help="read files without a shard header as raw ids of this width")
    ap.add_argument("--lane", default="pretrain", choices=["pretrain", "sft", "dpo"],
                    help="sft: instruction tuning on --sft-records (JSON lines of {messages: [...]}) with the assistant-token mask, "
                         "cosine schedule and a checkpoint/resume drill; prints the lane report")
    ap.add_argument("--dpo-pairs", default="", help="--lane dpo: JSON lines of {messages, chosen, rejected}")
    ap.add_argument("--beta", type=float, default=0.1, help="--lane dpo: strength of the implicit reward")
    ap.add_argument("--sft-records", default="")
    ap.add_argument("--sft-merges", type=int, default=512, help="merges of the byte-level BPE trained on the records")
    ap.add_argument("--sft-repeat", type=int, default=0, help="tile the packed corpus this many times (0 = enough for the run)")
    ap.add_argument("--checkpoint-at", type=int, default=0, help="step of the resume drill (0 = a third of the run)")
    ap.add_argument("--report", default="", help="write the lane report here as JSON")
    ap.add_argument("--sync-profile", default="sync", choices=["sync", "diloco"],
                    help="sync: every step is data-parallel over all ranks; diloco: every rank is a replica that takes "
                         "--inner-steps local steps per round, then one outer step over all replicas")
    ap.add_argument("--inner-steps", type=int, default=16)
    ap.add_argument("--outer-lr", type=float, default=0.7)
    ap.add_argument("--outer-momentum", type=float, default=0.9)
    ap.add_argument("--min-participants", type=int, default=1)
    return ap.parse_args(argv)


def worker(args):
    import torch
    import torch.distributed as dist
    from ..control import run_window as rw
    from ..models.config import PRESETS
    from .checkpoint import seal_descriptor
    from .trainer import TrainConfig, Trainer, synthetic_batch

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    model = PRESETS[args.model]
    if args.layers:
        model = model.with_(n_layers=args.layers)
    cfg = TrainConfig(model=model, global_batch=args.global_batch, micro_batch=args.micro_batch, seq_len=args.seq_len,
                      lr=args.lr, betas=tuple(args.betas), weight_decay=args.wd, grad_clip=args.clip, seed=args.seed,
                      zero_stage=args.zero_stage, schedule=args.schedule, total_steps=args.total_steps, warmup_steps=args.warmup_steps,
                      decay_fraction=args.decay_fraction)
    if args.sync_profile == "diloco":
        return diloco_worker(args, cfg, dev, rank, world)
    if args.lane == "sft":
        return sft_worker(args, cfg, dev, rank, world)
    if args.lane == "dpo":
        return dpo_worker(args, cfg, dev, rank, world)
    tr = Trainer(cfg, dev, rank, world)
    if args.resume:
        man = tr.load_checkpoint(args.resume)
        if rank == 0:
            print(json.dumps({"event": "resumed", "step": man["step"], "checkpointDigestRef": man["checkpointDigestRef"]}))
    auth = rw.Authority()
    run = auth.plan_run("promise.local.train", max_allowed_stale=args.max_allowed_stale)
    auth.advance_run(run.run_ref, "active")
    wsteps = args.window_steps or args.steps
    log = open(args.log_jsonl, "a") if (args.log_jsonl and rank == 0) else None
    loader = None
    if args.data:
        from ..data import BatchLoader, TokenDataset
        ds = TokenDataset(args.data, cfg.seq_len, args.data_raw_width)
        # the sampler is a function of the batch index, so a resumed run continues the stream at its step count
        loader = BatchLoader(ds, tr.accum, cfg.micro_batch, rank, world, seed=cfg.seed, start_batch=tr.step_count)
        if rank == 0:
            print(json.dumps({"event": "data", "shards": len(args.data), "tokens": ds.tokens, "windows": ds.windows,
                              "batchesPerEpoch": loader.batches_per_epoch}))
    step0 = tr.step_count
    done = 0
    while done < args.steps:
        n = min(wsteps, args.steps - done)
        w = auth.plan_window(run.run_ref, step0 + done, step0 + done + n)
        auth.activate_window(w.window_ref)
        auth.claim_lease(w.window_ref, f"worker.rank{rank}")
        t_train = 0.0
        for _ in range(n):
            n_valid = None
            if loader is not None:
                tok, tgt, nv, _ = loader.next()
                n_valid = nv if nv < tok.numel() else None           # only masked data changes the normalisation
                # the slot goes back to the loader at the next call, after this step's loss has been read (a stream sync)
                tok, tgt = tok.to(dev, non_blocking=True), tgt.to(dev, non_blocking=True)
            else:
                tok, tgt = synthetic_batch(cfg, tr.accum, tr.step_count, rank, dev)
                tok, tgt = tok.pin_memory().to(dev, non_blocking=True), tgt.pin_memory().to(dev, non_blocking=True)
            t0 = time.perf_counter()
            loss = tr.train_step(tok, tgt, n_valid)
            lv = float(loss.item())
            dt = time.perf_counter() - t0
            t_train += dt
            rec = {"event": "step", "step": tr.step_count, "loss": round(lv, 5), "grad_norm": round(tr.grad_norm(), 5),
                   "step_s": round(dt, 4), "tokens_per_s": round(cfg.global_batch * cfg.seq_len / dt, 1), "lr": tr.lr_at(tr.step_count - 1)}
            if rank == 0:
                print(json.dumps(rec), flush=True)
                if log:
                    log.write(json.dumps(rec) + "\n")
        tr.check_status()
        done += n
        meta = rw.SealMetadata(verification_overhead={"verificationSeconds": 0.0, "trainingSeconds": t_train})
        if args.ckpt_dir:
            d = os.path.join(args.ckpt_dir, f"step{tr.step_count:08d}")
            man = tr.save_checkpoint(d, run_ref=run.run_ref, window_ref=w.window_ref, term=run.term)
            if rank == 0:
                meta.checkpoint_digest_ref = man["checkpointDigestRef"]
                meta.durable_checkpoint_seal = seal_descriptor(man, d)
        _, gate = auth.seal_window(w.window_ref, meta)
        if rank == 0:
            print(json.dumps({"event": "window", "windowRef": w.window_ref, "state": auth._window(w.window_ref).state,
                              "sealDecision": gate.decision if gate else None, "reasons": list(gate.reasons) if gate else []}))
        if auth._window(w.window_ref).state == "sealed":
            auth.reconcile_window(w.window_ref)
        else:
            # HOLD: the checkpoint is not durable (one local replica).  Training goes on; the window
            # stays open for an operator to seal once a replicated store has confirmed the copy.
            pass
    if log:
        log.close()
    if args.export_gguf:
        _export(tr, args, rank)
    if world > 1:
        dist.destroy_process_group()


def _export(tr, args, rank, tokenizer=None):
    if tokenizer is None and args.tokenizer:
        from ..data import ByteBpe
        with open(args.tokenizer) as f:
            tokenizer = ByteBpe.from_json(f.read())
    tr.export_gguf(args.export_gguf, tokenizer=tokenizer)
    if rank == 0:
        print(json.dumps({"event": "exported", "path": args.export_gguf, "tokenizer": tokenizer is not None}))


def diloco_worker(args, cfg, dev, rank, world):
    """Local-update rounds: one replica per rank (its own trainer and optimizer state, a ``world``-th of the global batch),
    one window per round; rank 0 prints the round records and the window's coordination tags."""
    import dataclasses
    import torch
    import torch.distributed as dist
    from ..control import run_window as rw
    from .diloco import DilocoConfig, DilocoReplica
    from .trainer import Trainer, synthetic_batch
    if cfg.global_batch % world:
        raise SystemExit("--global-batch must be a multiple of the number of replicas")
    rcfg = dataclasses.replace(cfg, global_batch=cfg.global_batch // world)
    groups = [dist.new_group([r]) for r in range(world)] if world > 1 else [None]
    tr = Trainer(rcfg, dev, rank=0, world=1, group=groups[rank])
    dcfg = DilocoConfig(inner_steps=args.inner_steps, outer_lr=args.outer_lr, outer_momentum=args.outer_momentum,
                        min_participants=min(args.min_participants, world))
    rep = DilocoReplica(tr, dcfg, f"replica.rank{rank}")
    auth = rw.Authority()
    run = auth.plan_run("promise.local.train.diloco", max_allowed_stale=args.max_allowed_stale)
    auth.advance_run(run.run_ref, "active")
    done = 0
    while done < args.steps:
        n = min(args.inner_steps, args.steps - done)
        w = auth.plan_window(run.run_ref, done, done + n)
        auth.activate_window(w.window_ref)
        auth.claim_lease(w.window_ref, f"worker.rank{rank}")
        batches = []
        for i in range(n):
            tok, tgt = synthetic_batch(rcfg, tr.accum, done + i, rank, dev)
            batches.append((tok.pin_memory().to(dev, non_blocking=True), tgt.pin_memory().to(dev, non_blocking=True)))
        t0 = time.perf_counter()
        tags = dcfg.window_tags(rep.round_index, rep.base_checkpoint)
        rec = rep.run_round(batches)
        torch.cuda.synchronize(dev)
        dt = time.perf_counter() - t0
        tr.check_status()
        done += n
        if rank == 0:
            print(json.dumps({"event": "round", **rec, "round_s": round(dt, 4), "windowRef": w.window_ref, "replicas": world,
                              "tokens_per_s": round(rec["tokensAllReplicas"] / dt, 1), "windowTags": tags}), flush=True)
        auth.seal_window(w.window_ref, rw.SealMetadata(verification_overhead={"verificationSeconds": 0.0, "trainingSeconds": dt}))
    if world > 1:
        dist.destroy_process_group()


def sft_worker(args, cfg, dev, rank, world):
    """Instruction tuning on a file of chat records: tokenizer, masked shard, the run and its resume drill."""
    import dataclasses
    import tempfile
    import torch.distributed as dist
    from ..data import BatchLoader, ByteBpe, TokenDataset
    from . import sft
    from .trainer import Trainer
    if not args.sft_records:
        raise SystemExit("--lane sft needs --sft-records")
    records = sft.load_records(args.sft_records)
    text = "\n".join(m["content"] for r in records for m in r["messages"]).encode()
    tok = ByteBpe.train(text, args.sft_merges, special=sft.SPECIAL_TOKENS)
    if tok.vocab_size > cfg.model.vocab:
        raise SystemExit(f"the tokenizer has {tok.vocab_size} ids, the model {cfg.model.vocab}")
    corpus = sft.build_corpus(records, tok, os.path.basename(args.sft_records))
    cfg = dataclasses.replace(cfg, total_steps=args.steps)
    work = args.ckpt_dir or tempfile.mkdtemp(prefix="b200_sft_")
    os.makedirs(work, exist_ok=True)
    shard = os.path.join(work, "sft.b2tk")
    accum = cfg.global_batch // (cfg.micro_batch * world)
    need = (cfg.global_batch * cfg.seq_len + 1) * 2
    repeat = args.sft_repeat or max(1, -(-need // len(corpus.ids)))
    if rank == 0:
        sft.pack(corpus, shard, repeat)
    if world > 1:
        dist.barrier()
    ds = TokenDataset(shard, cfg.seq_len)
    rep = sft.run_lane(lambda: Trainer(cfg, dev, rank, world),
                       lambda start: BatchLoader(ds, accum, cfg.micro_batch, rank, world, seed=cfg.seed, start_batch=start),
                       steps=args.steps, checkpoint_at=args.checkpoint_at or max(1, args.steps // 3), ckpt_dir=os.path.join(work, "drill"),
                       corpus_manifest=corpus.manifest, device=dev,
                       on_finished=(lambda tr: _export(tr, args, rank, tokenizer=tok)) if args.export_gguf else None)
    if rank == 0:
        print(json.dumps(rep))
        if args.report:
            with open(args.report, "w") as f:
                json.dump(rep, f, indent=1)
    if world > 1:
        dist.destroy_process_group()


def dpo_worker(args, cfg, dev, rank, world):
    """Preference optimisation on a file of pairs: every step takes the next ``global_batch / 2`` pairs (cycling), the
    reference log-probabilities are computed once with the starting weights."""
    import torch
    import torch.distributed as dist
    from ..data import ByteBpe
    from . import dpo, sft
    from .trainer import Trainer
    if not args.dpo_pairs:
        raise SystemExit("--lane dpo needs --dpo-pairs")
    pairs = sft.load_records(args.dpo_pairs, preference=True)
    text = "\n".join([m["content"] for p in pairs for m in p["messages"]] + [p[k] for p in pairs for k in ("chosen", "rejected")]).encode()
    tok = ByteBpe.train(text, args.sft_merges, special=sft.SPECIAL_TOKENS)
    if tok.vocab_size > cfg.model.vocab:
        raise SystemExit(f"the tokenizer has {tok.vocab_size} ids, the model {cfg.model.vocab}")
    tr = Trainer(cfg, dev, rank, world)
    if args.resume:
        tr.load_checkpoint(args.resume)
    d = dpo.DpoTrainer(tr, beta=args.beta)
    P = cfg.micro_batch // 2                       # pairs per micro-batch on this rank
    per_step = P * tr.accum * world

    def batch(step):
        toks, tgts = [], []
        for a in range(tr.accum):
            at = step * per_step + (a * world + rank) * P
            t, g, _ = dpo.build_preference_batch([pairs[(at + i) % len(pairs)] for i in range(P)], tok, cfg.seq_len)
            toks.append(t)
            tgts.append(g)
        return torch.stack(toks).pin_memory().to(dev, non_blocking=True), torch.stack(tgts).pin_memory().to(dev, non_blocking=True)

    distinct = min(args.steps, -(-len(pairs) // per_step))
    refs = {}
    for s in range(distinct):                      # before the first update: the starting weights are the reference policy
        t, g = batch(s)
        refs[s] = d.reference_logps(t, g)
    for s in range(args.steps):
        t, g = batch(s % distinct)
        t0 = time.perf_counter()
        loss = float(d.train_step(t, g, refs[s % distinct]).item())
        dt = time.perf_counter() - t0
        if rank == 0:
            rec = {"event": "step", "step": tr.step_count, "pair_loss": round(loss, 5), "reward_accuracy": round(d.reward_accuracy(), 4),
                   "grad_norm": round(tr.grad_norm(), 5), "step_s": round(dt, 4), "pairs_per_s": round(per_step / dt, 1)}
            print(json.dumps(rec), flush=True)
            if args.log_jsonl:
                with open(args.log_jsonl, "a") as f:
                    f.write(json.dumps(rec) + "\n")
    tr.check_status()
    if args.ckpt_dir:
        tr.save_checkpoint(os.path.join(args.ckpt_dir, f"step{tr.step_count:08d}"))
    if world > 1:
        dist.destroy_process_group()


def run_manifest(path: str, work_dir: str | None = None) -> int:
    """Zero-touch: validate the assignment, pin its inputs, run it with the flags it stands for, write the receipts."""
    import tempfile
    from . import assignment_manifest as am
    with open(path) as f:
        m = json.load(f)
    work = work_dir or tempfile.mkdtemp(prefix="b200_assignment_")
    os.makedirs(work, exist_ok=True)
    blockers = am.validate(m) or am.verify_inputs(m)
    t0 = time.time()
    status = "refused" if blockers else "succeeded"
    if not blockers:
        try:
            main(am.launcher_argv(m, work))
        except SystemExit as e:
            status = "succeeded" if e.code in (0, None) else "failed"
        except Exception as e:      # noqa: BLE001 - whatever ended the run goes into the receipt, not up the stack
            status, blockers = "failed", [f"blocker.training_assignment.run_failed.{type(e).__name__}"]
    out = am.receipts(m if isinstance(m, dict) and "budget" in m else {"budget": {"maxWallSeconds": 1}, "batch": {"global": 0, "seqLen": 0}, "assignmentId": "unknown",
                                                                        "runRef": "run.unknown", "manifestDigest": "sha256:" + "0" * 64},
                      work, status, time.time() - t0)
    out["blockerRefs"] = blockers
    with open(os.path.join(work, "receipts.json"), "w") as f:
        json.dump(out, f, indent=1)
    print(json.dumps({"event": "assignment_closed", "status": out["workerReceipt"]["status"], "workDir": work, "blockerRefs": blockers,
                      "receiptDigest": out["workerReceipt"]["receiptDigest"]}))
    return 0 if out["workerReceipt"]["status"] == "succeeded" else 3


@cli_entry("b200-train")
def main(argv=None):
    if "RANK" in os.environ and os.environ.get("B200_TRAIN_ARGV"):      # a worker started by the re-execution below
        return worker(parse(json.loads(os.environ["B200_TRAIN_ARGV"])))
    raw = list(sys.argv[1:] if argv is None else argv)
    if "--manifest" in raw:                                              # the zero-touch path: every other flag comes from the manifest
        i = raw.index("--manifest")
        wd = raw[raw.index("--work-dir") + 1] if "--work-dir" in raw else None
        raise SystemExit(run_manifest(raw[i + 1], wd))
    args = parse(argv)
    if args.nproc > 1 and "RANK" not in os.environ:
        # The worker's flags travel in the environment: torch.distributed.run parses abbreviations of its own options
        # (``--nproc`` matches ``--nproc-per-node``) even behind the module name.
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.nproc}",
               "--master-addr", "127.0.0.1", "--master-port", str(args.master_port), "-m", "openagents_b200.train.launcher"]
        env = dict(os.environ, B200_TRAIN_ARGV=json.dumps(sys.argv[1:] if argv is None else list(argv)))
        raise SystemExit(subprocess.call(cmd, env=env))
    worker(args)


if __name__ == "__main__":
    main()
