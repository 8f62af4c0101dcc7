"""``python -m openagents_b200.gguf``: look into a GGUF file, re-quantize it, digest it.

    python -m openagents_b200.gguf inspect model.gguf             # architecture, shape, tensor types and bytes, tokenizer kind
    python -m openagents_b200.gguf quantize in.gguf out.gguf --plan q4_k     # every tensor through fp32 into the plan's block types
    python -m openagents_b200.gguf digest model.gguf              # the artifact digest receipts and manifests cite

``quantize`` keeps every metadata key that is not a shape or file-type key (tokenizer, chat template, the tokenizer a tuned
checkpoint carries) and reports the relative RMS error of each re-quantized tensor against the input.
"""
from __future__ import annotations

import argparse
import json
import sys

import numpy as np

from ..utils.cli import cli_entry


def inspect(path: str) -> dict:
    from . import GGUFFile
    with GGUFFile(path) as f:
        by_type: dict[str, dict] = {}
        total = 0
        for t in f.tensors.values():
            e = by_type.setdefault(t.type.name, {"tensors": 0, "bytes": 0, "elements": 0})
            e["tensors"] += 1
            e["bytes"] += t.nbytes
            e["elements"] += int(np.prod(t.shape)) if t.shape else 1
            total += t.nbytes
        meta = f.metadata
        arch = f.architecture
        tok = ("b200-byte-bpe" if "tokenizer.b200.byte_bpe" in meta else meta.get("tokenizer.ggml.model", "ggml-tokens") if "tokenizer.ggml.tokens" in meta else "none (bytes)")
        shape = {k.split(".", 1)[1]: v for k, v in meta.items() if k.startswith(arch + ".") and not isinstance(v, (list, dict))}
        elements = sum(e["elements"] for e in by_type.values())
        return {"path": path, "version": f.version, "alignment": f.alignment, "architecture": arch, "shape": shape, "tensorCount": len(f.tensors),
                "tensorBytes": total, "parameters": elements, "bitsPerWeight": round(8.0 * total / max(1, elements), 3), "byType": by_type,
                "tokenizer": tok, "chatTemplate": "tokenizer.chat_template" in meta,
                "metadataKeys": sorted(k for k in meta if not k.startswith(("tokenizer.ggml.tokens", "tokenizer.ggml.merges", "tokenizer.ggml.token_type")))}


def quantize(src: str, dst: str, plan_name: str) -> dict:
    import torch
    from ..models import weights as W
    from ..models.config import ModelConfig
    from . import GGUFFile
    plans = {"q8_0": W.PLAN_Q8_0, "q4_k": W.PLAN_Q4_K, "bf16": W.PLAN_BF16, "f32": W.PLAN_F32, "moe": W.PLAN_MOE}
    if plan_name not in plans:
        raise SystemExit(f"unknown plan {plan_name!r}; choose from {sorted(plans)}")
    with GGUFFile(src) as f:
        cfg = ModelConfig.from_gguf_metadata(f.metadata)
        drop = set(cfg.to_gguf_metadata()) | {"general.file_type", "general.alignment"}
        extra = {k: v for k, v in f.metadata.items() if k not in drop}
        floats = {n: torch.from_numpy(t.to_float().copy()) for n, t in f.tensors.items()}
        before = {n: t.type.name for n, t in f.tensors.items()}
    W.save_gguf(dst, cfg, floats, plans[plan_name], extra_meta=extra)
    rows, worst = [], 0.0
    with GGUFFile(dst) as g:
        for n, t in g.tensors.items():
            a, b = floats[n].numpy().astype(np.float64).reshape(-1), t.to_float().astype(np.float64).reshape(-1)
            err = float(np.sqrt(np.mean((a - b) ** 2)) / (np.sqrt(np.mean(a ** 2)) + 1e-30))
            worst = max(worst, err)
            rows.append({"tensor": n, "from": before[n], "to": t.type.name, "relativeRmsError": round(err, 6)})
        out_bytes = sum(t.nbytes for t in g.tensors.values())
    return {"source": src, "output": dst, "plan": plan_name, "tensorBytes": out_bytes, "worstRelativeRmsError": round(worst, 6),
            "keptMetadataKeys": sorted(k for k in extra if not k.startswith("tokenizer.ggml.")), "tensors": rows}


@cli_entry("b200-gguf")
def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m openagents_b200.gguf")
    sub = ap.add_subparsers(dest="cmd", required=True)
    sub.add_parser("inspect").add_argument("path")
    q = sub.add_parser("quantize")
    q.add_argument("src")
    q.add_argument("dst")
    q.add_argument("--plan", default="q4_k")
    q.add_argument("--quiet", action="store_true", help="leave the per-tensor rows out of the printed report")
    sub.add_parser("digest").add_argument("path")
    args = ap.parse_args(argv)
    if args.cmd == "inspect":
        out = inspect(args.path)
    elif args.cmd == "quantize":
        out = quantize(args.src, args.dst, args.plan)
        if args.quiet:
            out.pop("tensors")
    else:
        from ..receipts.manifests import artifact_digest
        out = {"path": args.path, "artifactDigest": artifact_digest(args.path)}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
