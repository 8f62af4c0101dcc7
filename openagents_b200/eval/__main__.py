"""``python -m openagents_b200.eval``: run an evaluation pack against a GGUF checkpoint and print the decision.

    python -m openagents_b200.eval --model ckpt.gguf --heldout val.b2tk --seq-len 1024 \\
        --gate heldout.loss:<=:3.2 --gate heldout.loss:<=:4.0:rollback --choices mc.jsonl --gate mc.accuracy:>=:0.3
"""
from __future__ import annotations

import argparse
import json
import sys
import time

from ..utils.cli import cli_entry


def parse_gate(text: str):
    from .pack import MetricGate
    parts = text.split(":")
    if len(parts) not in (3, 4):
        raise argparse.ArgumentTypeError("a gate is metric:comparator:threshold[:rollback|optional]")
    flag = parts[3] if len(parts) == 4 else ""
    if flag not in ("", "rollback", "optional"):
        raise argparse.ArgumentTypeError(f"unknown gate flag {flag!r}")
    return MetricGate(parts[0], parts[1], float(parts[2]), required=flag != "optional", rollback_on_fail=flag == "rollback")


@cli_entry("b200-eval")
def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m openagents_b200.eval")
    ap.add_argument("--model", required=True, help="GGUF checkpoint")
    ap.add_argument("--backend", default="cuda", choices=["cuda", "cpu"])
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--heldout", nargs="*", default=[], help="token shards for the perplexity task")
    ap.add_argument("--raw-width", type=int, default=0, choices=[0, 2, 4])
    ap.add_argument("--seq-len", type=int, default=1024)
    ap.add_argument("--max-windows", type=int, default=0)
    ap.add_argument("--choices", default="", help="JSON lines of {context, choices, answer} for the multiple-choice task")
    ap.add_argument("--exact", default="", help="JSON lines of {prompt, answer} for the exact-match task")
    ap.add_argument("--max-new-tokens", type=int, default=32)
    ap.add_argument("--gate", type=parse_gate, action="append", default=[])
    ap.add_argument("--package-ref", default="benchmark://b200/local/checkpoint_eval@1")
    ap.add_argument("--checkpoint-ref", default="")
    ap.add_argument("--out", default="")
    args = ap.parse_args(argv)

    from ..data import TokenDataset
    from ..serve.backend import open_backend
    from ..serve.server import load_tokenizer
    from .pack import EvalPack, eval_run_evidence, run_pack
    from .scorers import load_items

    backend = open_backend(args.model, args.backend, args.device, max_num_seqs=4, max_ctx=max(args.seq_len, 512) + 64,
                           max_tokens=max(args.seq_len, 512) + 64)
    tok, _ = load_tokenizer(args.model, backend.cfg.vocab)
    tasks = []
    if args.heldout:
        tasks.append({"name": "heldout", "kind": "perplexity", "dataset": TokenDataset(args.heldout, args.seq_len, args.raw_width),
                      "max_windows": args.max_windows or None, "shards": len(args.heldout), "seq_len": args.seq_len})
    if args.choices:
        tasks.append({"name": "mc", "kind": "multiple_choice", "items": load_items(args.choices, "multiple_choice")})
    if args.exact:
        tasks.append({"name": "em", "kind": "exact_match", "items": load_items(args.exact, "exact_match"), "max_new_tokens": args.max_new_tokens,
                      "stop_ids": [tok.eos_id] if getattr(tok, "eos_id", None) is not None else []})
    if not tasks:
        ap.error("nothing to evaluate: give --heldout, --choices or --exact")
    t0 = time.perf_counter()
    decision = run_pack(EvalPack(args.package_ref, tasks, args.gate), backend, tok, args.checkpoint_ref or f"checkpoint://local/{args.model.rsplit('/', 1)[-1]}")
    decision["wallSeconds"] = round(time.perf_counter() - t0, 3)
    decision["evidence"] = eval_run_evidence(decision, time.strftime("%Y-%m-%dT%H:%M:%SZ", time.gmtime()))
    text = json.dumps(decision)
    print(text)
    if args.out:
        with open(args.out, "w") as f:
            f.write(text + "\n")
    return {"continue": 0, "hold": 3, "rollback": 4}[decision["decisionState"]]


if __name__ == "__main__":
    sys.exit(main())
