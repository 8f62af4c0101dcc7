"""Distill to fit: a smaller student learns from a served teacher's own answers.

The reference's private-deployment contracts name the stage and its receipt (a smaller distilled model from a captured input
distribution, accepted on an evaluated quality delta and a cost reduction, the router swap gated separately;
packages/reactor-contracts/src/index.ts:857-890) and leave the run itself to the training stack.  This is the sequence-level
form of that run, built from parts the framework already has:

1. ``teacher_records``: the teacher, any serving backend, answers the captured prompts through the ordinary scheduler (greedy
   or sampled, several answers per prompt if wanted); each answer becomes a chat record;
2. the records go through ``train.sft`` (assistant-token mask, corpus manifest, lane report with the resume drill) on the
   student's trainer: the student is trained to put its probability on the teacher's tokens, which is the hard-label limit of
   matching the teacher's distribution and needs no teacher logits to cross a process boundary;
3. ``quality_delta`` scores both models on held-out prompts with the evaluation scorers, in basis points, for the receipt
   (``control.reactor.distill_to_fit_receipt``).
"""
from __future__ import annotations

import hashlib
import json

from . import sft


def teacher_records(backend, tokenizer, prompts: list[str], max_new_tokens: int = 64, answers_per_prompt: int = 1, temperature: float = 0.0,
                    top_k: int = 0, seed: int = 0, system: str | None = None, max_num_seqs: int = 8) -> tuple[list[dict], dict]:
    """``prompts``: user turns.  The teacher sees each one under the instruction-tuning template (``sft.generation_prompt``) and stops
    at the end-of-turn marker when its vocabulary has one.  Returns the records and a capture manifest (digests, counts)."""
    from ..serve.generation import SamplingParams, Scheduler
    sch = Scheduler(backend, tokenizer, max_num_seqs=max_num_seqs)
    reqs = []
    for p_i, prompt in enumerate(prompts):
        msgs = ([{"role": "system", "content": system}] if system else []) + [{"role": "user", "content": prompt}]
        ids = tokenizer.encode(sft.generation_prompt(msgs))
        for k in range(answers_per_prompt):
            params = SamplingParams(max_tokens=max_new_tokens, temperature=temperature if answers_per_prompt > 1 or temperature > 0 else 0.0, top_k=top_k,
                                    stop=(sft.TEMPLATE["endOfTurn"],), seed=(seed * 1_000_003 + p_i * 101 + k) & 0x7FFFFFFF)
            reqs.append((msgs, sch.submit(ids, params)))
    sch.run_until_done([r for _, r in reqs])
    records, dropped, seen = [], 0, set()
    for msgs, r in reqs:
        eos = getattr(tokenizer, "eos_id", None)
        text = tokenizer.decode([t for t in r.output if t != eos]).split(sft.TEMPLATE["endOfTurn"])[0].strip()
        key = hashlib.sha256(json.dumps([msgs, text]).encode()).hexdigest()
        if not text or r.finish_reason == "error" or key in seen:
            dropped += 1
            continue
        seen.add(key)
        records.append({"messages": msgs + [{"role": "assistant", "content": text}]})
    manifest = {"schema": "b200.training.distillation_capture.v1", "prompts": len(prompts), "answersPerPrompt": answers_per_prompt, "records": len(records),
                "dropped": dropped, "teacherBackend": backend.name,
                "inputDistributionDigest": "sha256:" + hashlib.sha256(json.dumps(prompts, sort_keys=True).encode()).hexdigest(),
                "recordsDigest": "sha256:" + hashlib.sha256(json.dumps(records, sort_keys=True).encode()).hexdigest()}
    return records, manifest


def quality_delta(teacher_backend, student_backend, teacher_tok, student_tok, items, max_new_tokens: int = 32) -> dict:
    """Exact-match quality of both models on the same ``{"prompt", "answer"}`` items, in basis points, and the delta."""
    from ..eval.scorers import exact_match
    out = {}
    for name, be, tok in (("baseline", teacher_backend, teacher_tok), ("candidate", student_backend, student_tok)):
        stop = [tok.eos_id] if getattr(tok, "eos_id", None) is not None else []
        r = exact_match(be, items, tok, max_new_tokens=max_new_tokens, stop_ids=stop)
        out[name + "QualityScoreBps"] = round(r["exactMatch"] * 10_000)
    out["qualityDeltaBps"] = out["candidateQualityScoreBps"] - out["baselineQualityScoreBps"]
    out["items"] = len(items)
    return out
