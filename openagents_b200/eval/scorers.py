"""Scorers that run on any serving backend (``serve.backend.Backend`` with ``score``; the fp32 CPU backend is the oracle).

* ``perplexity``: mean negative log-likelihood per target token over windows of a token data set (masked targets are
  skipped), reported as loss, perplexity and, when the byte count is known, bits per byte;
* ``multiple_choice``: log-likelihood ranking: the context is fed once, every choice is scored after it and cut off
  again (``truncate``), so the context's keys and values are computed once per item;
* ``exact_match``: greedy generation until a stop token or the length limit, compared with the expected answer after
  normalisation.

Each scorer opens its own sequences under ids taken from ``seq_base`` upward and closes them.
"""
from __future__ import annotations

import math


def _open(backend, seq_id: int, tokens: list[int]) -> None:
    """Open a sequence that will be fed ``tokens`` from position 0 (a prefix-cache hit is undone: scoring needs the logits of
    every position)."""
    cached = backend.begin(seq_id, list(tokens))
    if cached:
        backend.truncate(seq_id, 0)


def perplexity(backend, dataset, max_windows: int | None = None, seq_base: int = 1 << 40, bytes_per_token: float | None = None) -> dict:
    if not backend.supports_score:
        raise ValueError(f"backend {backend.name} cannot score")
    nll, n = 0.0, 0
    windows = len(dataset) if max_windows is None else min(len(dataset), max_windows)
    for w in range(windows):
        tok, tgt, valid = dataset.window(w)
        if valid == 0:
            continue
        sid = seq_base + w
        _open(backend, sid, tok.tolist())
        try:
            lp = backend.score(sid, tok.tolist(), tgt.tolist())
        finally:
            backend.end(sid)
        nll -= sum(lp)
        n += valid
    if n == 0:
        raise ValueError("no unmasked target in the evaluated windows")
    loss = nll / n
    out = {"windows": windows, "targets": n, "loss": loss, "perplexity": math.exp(min(loss, 700.0))}
    if bytes_per_token:
        out["bitsPerByte"] = loss / math.log(2.0) / bytes_per_token
    return out


def load_items(path: str, kind: str) -> list[dict]:
    """The items of a JSON-lines task file, each checked before any model time is spent: ``multiple_choice`` items are
    ``{"context": text, "choices": [two or more texts], "answer": index}``, ``exact_match`` items ``{"prompt": text, "answer": text}``.
    A bad line raises ``ValueError`` with the file name and line number."""
    import json
    if kind not in ("multiple_choice", "exact_match"):
        raise ValueError(f"unknown task kind {kind!r}")
    text = lambda v: isinstance(v, str) and v.strip() != ""      # noqa: E731
    out = []
    with open(path, encoding="utf-8") as f:
        for n, line in enumerate(f, 1):
            if not line.strip():
                continue
            where = f"{path}:{n}"
            try:
                it = json.loads(line)
            except ValueError as e:
                raise ValueError(f"{where}: not JSON ({e})") from None
            if not isinstance(it, dict):
                raise ValueError(f"{where}: an item is a JSON object")
            if kind == "multiple_choice":
                ch = it.get("choices")
                if not text(it.get("context")) or not isinstance(ch, list) or len(ch) < 2 or not all(text(c) for c in ch):
                    raise ValueError(f"{where}: an item is {{\"context\": text, \"choices\": [two or more texts], \"answer\": index}}")
                a = it.get("answer")
                if not isinstance(a, int) or isinstance(a, bool) or not 0 <= a < len(ch):
                    raise ValueError(f"{where}: answer must be the index of one of the {len(ch)} choices")
            elif not text(it.get("prompt")) or not isinstance(it.get("answer"), str):
                raise ValueError(f"{where}: an item is {{\"prompt\": text, \"answer\": text}}")
            out.append(it)
    if not out:
        raise ValueError(f"{path}: no items")
    return out


def multiple_choice(backend, items, tokenizer, length_normalised: bool = True, seq_base: int = 1 << 41) -> dict:
    """``items``: ``{"context": str, "choices": [str, ...], "answer": index}``.  Returns accuracy and the per-item picks."""
    if not (backend.supports_score and backend.supports_verify):
        raise ValueError(f"backend {backend.name} cannot score and cut a sequence")
    picks, correct = [], 0
    for k, it in enumerate(items):
        ctx = tokenizer.encode(it["context"])
        if not ctx:
            raise ValueError("empty context")
        sid = seq_base + k
        _open(backend, sid, ctx)
        try:
            # everything but the context's last token is fed once; that token leads every choice so that its logits score the
            # choice's first token
            if len(ctx) > 1:
                backend.score(sid, ctx[:-1], [-1] * (len(ctx) - 1))
            keep = len(ctx) - 1
            scores = []
            for ch in it["choices"]:
                c = tokenizer.encode(ch)
                if not c:
                    raise ValueError("empty choice")
                feed = [ctx[-1]] + c[:-1]
                lp = backend.score(sid, feed, c)
                backend.truncate(sid, keep)
                s = sum(lp)
                scores.append(s / len(c) if length_normalised else s)
        finally:
            backend.end(sid)
        pick = max(range(len(scores)), key=lambda i: scores[i])
        picks.append({"pick": pick, "answer": it["answer"], "scores": scores})
        correct += int(pick == it["answer"])
    return {"items": len(picks), "accuracy": correct / max(1, len(picks)), "picks": picks}


def _norm(s: str) -> str:
    return " ".join(s.strip().lower().split())


def exact_match(backend, items, tokenizer, max_new_tokens: int = 32, stop_ids=(), seq_base: int = 1 << 42) -> dict:
    """``items``: ``{"prompt": str, "answer": str}``; greedy decoding."""
    rows, correct = [], 0
    stop = set(stop_ids)
    for k, it in enumerate(items):
        prompt = tokenizer.encode(it["prompt"])
        sid = seq_base + k
        cached = backend.begin(sid, prompt)
        out: list[int] = []
        try:
            feed = prompt[cached:]
            for _ in range(max_new_tokens):
                nxt = int(backend.forward([sid], [feed])[0].argmax())
                if nxt in stop:
                    break
                out.append(nxt)
                feed = [nxt]
        finally:
            backend.end(sid)
        text = tokenizer.decode(out)
        ok = _norm(text) == _norm(it["answer"]) or _norm(text).startswith(_norm(it["answer"]))
        rows.append({"generated": text, "answer": it["answer"], "match": ok})
        correct += int(ok)
    return {"items": len(rows), "exactMatch": correct / max(1, len(rows)), "rows": rows}
