"""``python -m openagents_b200.data``: text -> refined, tokenized, sharded training data.

    python -m openagents_b200.data prepare --text corpus/*.txt --out data/run1 --merges 8192 --val-fraction 0.01
    python -m openagents_b200.data traces --in served.jsonl --out sft_records.jsonl

``prepare`` treats every input file as documents separated by blank lines (one JSON object with a ``text`` field per line for
``.jsonl``; the HTML responses of ``.warc`` / ``.warc.gz`` crawl files and ``.html`` files go through the text extractor), runs the refinery, trains a byte-level BPE on the refined text (or loads ``--tokenizer``), writes
``train-*.b2tk`` / ``val.b2tk`` with an end-of-text id between documents, and a manifest with every stage's counters.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import sys

from ..utils.cli import cli_entry


def _read_documents(paths) -> list[str]:
    texts = []
    for p in paths:
        if p.endswith((".warc", ".warc.gz")):                     # crawl files: HTML responses -> extracted text
            from .extract import warc_to_documents
            texts += ["\n".join(d["lines"]) for d in warc_to_documents(p)]
            continue
        if p.endswith((".html", ".htm")):
            from .extract import html_to_text
            with open(p, "rb") as f:
                texts.append(html_to_text(f.read()))
            continue
        with open(p, encoding="utf-8", errors="replace") as f:
            if p.endswith(".jsonl"):
                texts += [json.loads(line)["text"] for line in f if line.strip()]
            else:
                texts += [b for b in f.read().split("\n\n") if b.strip()]
    return texts


def prepare(args) -> dict:
    import numpy as np
    from . import ByteBpe, write_token_shard
    from .refinery import STAGES, documents_from_texts, refine
    texts = _read_documents(args.text)
    docs, report = refine(documents_from_texts(texts), stages=() if args.no_refine else STAGES, seed=args.seed, max_line_repeats=args.max_line_repeats)
    for flag, stage in ((args.language_id, "language_id"), (args.quality_classifier, "quality_classifier")):
        if flag:                                                  # MODEL.json:LABEL[:MIN_CONFIDENCE]
            from .classifiers import HashedNgramClassifier, classifier_stage
            parts = flag.split(":")
            docs, rep = classifier_stage(docs, HashedNgramClassifier.load(parts[0]), parts[1], float(parts[2]) if len(parts) > 2 else 0.5, stage=stage)
            report["stages"].append({"stage": stage, "stats": rep, "documentsAfter": len(docs)})
            report["outputDocuments"] = len(docs)
    bodies = ["\n".join(d["lines"]) for d in docs]
    if not bodies:
        raise SystemExit("the refinery kept no document")
    eot = "<|endoftext|>"
    if args.tokenizer:
        with open(args.tokenizer) as f:
            tok = ByteBpe.from_json(f.read())
        if eot not in tok.special_ids:
            raise SystemExit("the tokenizer has no <|endoftext|> id")
    else:
        tok = ByteBpe.train("\n".join(bodies).encode(), args.merges, special=[eot])
    os.makedirs(args.out, exist_ok=True)
    with open(os.path.join(args.out, "tokenizer.json"), "w") as f:
        f.write(tok.to_json())
    n_val = int(len(bodies) * args.val_fraction)
    order = sorted(range(len(bodies)), key=lambda i: hashlib.sha256(f"{args.seed}:{docs[i]['documentRef']}".encode()).digest())
    val_set = set(order[:n_val])
    streams = {"train": [], "val": []}
    for i, body in enumerate(bodies):
        streams["val" if i in val_set else "train"] += tok.encode(body) + [tok.special_ids[eot]]
    files = []
    train = np.asarray(streams["train"], dtype=np.int64)
    per = max(1, args.shard_tokens)
    for k in range(0, max(1, len(train)), per):
        files.append(write_token_shard(os.path.join(args.out, f"train-{k // per:05d}.b2tk"), train[k: k + per]))
    if streams["val"]:
        files.append(write_token_shard(os.path.join(args.out, "val.b2tk"), np.asarray(streams["val"], dtype=np.int64)))
    chars = sum(len(b) for b in bodies)
    manifest = {"schema": "b200.data.prepared.v1", "documents": len(bodies), "valDocuments": n_val, "vocabSize": tok.vocab_size,
                "merges": len(tok.merges), "trainTokens": len(streams["train"]), "valTokens": len(streams["val"]),
                "bytesPerToken": round(len("\n".join(bodies).encode()) / max(1, len(streams["train"]) + len(streams["val"])), 4),
                "characters": chars, "refinery": report, "files": [{**f, "path": os.path.basename(f["path"])} for f in files]}
    with open(os.path.join(args.out, "manifest.json"), "w") as f:
        json.dump(manifest, f, indent=1)
    return manifest


def traces(args) -> dict:
    from .traces import traces_to_records
    with open(args.inp) as f:
        rows = [json.loads(line) for line in f if line.strip()]
    records, report = traces_to_records(rows, args.max_chars)
    with open(args.out, "w") as f:
        for r in records:
            f.write(json.dumps(r) + "\n")
    return report


@cli_entry("b200-data")
def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m openagents_b200.data")
    sub = ap.add_subparsers(dest="cmd", required=True)
    p = sub.add_parser("prepare")
    p.add_argument("--text", nargs="+", required=True)
    p.add_argument("--out", required=True)
    p.add_argument("--merges", type=int, default=8192)
    p.add_argument("--tokenizer", default="")
    p.add_argument("--val-fraction", type=float, default=0.01)
    p.add_argument("--shard-tokens", type=int, default=100_000_000)
    p.add_argument("--max-line-repeats", type=int, default=1)
    p.add_argument("--no-refine", action="store_true")
    p.add_argument("--language-id", default="", help="MODEL.json:LABEL[:MIN_CONFIDENCE] keeps the documents a hashed n-gram classifier assigns to LABEL")
    p.add_argument("--quality-classifier", default="", help="same form, for a learned quality filter")
    p.add_argument("--seed", default="refinery")
    t = sub.add_parser("traces")
    t.add_argument("--in", dest="inp", required=True)
    t.add_argument("--out", required=True)
    t.add_argument("--max-chars", type=int, default=200_000)
    args = ap.parse_args(argv)
    out = prepare(args) if args.cmd == "prepare" else traces(args)
    print(json.dumps({k: v for k, v in out.items() if k != "refinery"} if args.cmd == "prepare" else out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
