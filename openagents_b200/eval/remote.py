"""The same scorers against a running server: log-likelihoods through ``/v1/completions`` (``echo`` + ``logprobs`` with
``max_tokens: 0``), the request evaluation harnesses send.  Token ids travel as the prompt, so client and server cannot
disagree about tokenisation."""
from __future__ import annotations

import json
import math
import urllib.request


def _score(base_url: str, model: str, token_ids: list[int], timeout: float = 300.0, api_key: str | None = None) -> list:
    req = urllib.request.Request(base_url.rstrip("/") + "/v1/completions",
                                 data=json.dumps({"model": model, "prompt": token_ids, "max_tokens": 0, "echo": True, "logprobs": 1}).encode(),
                                 headers={"Content-Type": "application/json", **({"Authorization": f"Bearer {api_key}"} if api_key else {})})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        lp = json.loads(r.read())["choices"][0]["logprobs"]
    if lp["token_ids"] != list(token_ids):
        raise RuntimeError("the server scored other tokens than were sent")
    return lp["token_logprobs"]


def loglikelihood(base_url: str, model: str, context_ids: list[int], continuation_ids: list[int], **kw) -> float:
    """log p(continuation | context) in nats."""
    if not context_ids or not continuation_ids:
        raise ValueError("context and continuation must be non-empty")
    lps = _score(base_url, model, list(context_ids) + list(continuation_ids), **kw)
    return float(sum(lps[len(context_ids):]))


def perplexity_http(base_url: str, model: str, dataset, max_windows: int | None = None, **kw) -> dict:
    """``scorers.perplexity`` over HTTP: a window's inputs plus its final target go out as one prompt of ``seq_len + 1`` ids, and
    the log-probabilities of ids 1.. are the window's ``seq_len`` predictions (masked targets are skipped)."""
    nll, n = 0.0, 0
    windows = len(dataset) if max_windows is None else min(len(dataset), max_windows)
    for w in range(windows):
        tok, tgt, _ = dataset.window(w)
        ids = tok.tolist() + [int(tgt[-1])] if int(tgt[-1]) >= 0 else tok.tolist()
        lps = _score(base_url, model, ids, **kw)
        keep = [i for i in range(1, len(ids)) if int(tgt[i - 1]) >= 0]
        nll -= sum(lps[i] for i in keep)
        n += len(keep)
    if n == 0:
        raise ValueError("no unmasked target in the evaluated windows")
    return {"windows": windows, "targets": n, "loss": nll / n, "perplexity": math.exp(min(nll / n, 700.0))}


def multiple_choice_http(base_url: str, model: str, items, tokenizer, length_normalised: bool = True, **kw) -> dict:
    picks, correct = [], 0
    for it in items:
        ctx = tokenizer.encode(it["context"])
        scores = []
        for ch in it["choices"]:
            c = tokenizer.encode(ch)
            s = loglikelihood(base_url, model, ctx, c, **kw)
            scores.append(s / len(c) if length_normalised else s)
        pick = max(range(len(scores)), key=lambda i: scores[i])
        picks.append({"pick": pick, "answer": it["answer"], "scores": scores})
        correct += int(pick == it["answer"])
    return {"items": len(picks), "accuracy": correct / max(1, len(picks)), "picks": picks}
