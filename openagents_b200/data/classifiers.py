"""Small text classifiers for the refinery: language identification and a learned quality filter.

Both are the same model, the one the course's data assignment uses off the shelf: a bag of hashed character n-grams into a
linear softmax layer (the "fastText supervised" shape), trained here with plain mini-batch SGD in ``torch`` on whatever
labelled texts the caller brings (the reference's continuation audit names language ID and model-backed quality, NSFW and
toxicity classifiers as the refinery stages still planned upstream;
docs/2026-06-10-cs336-distributed-homework-continuation-audit.md:280-295).  Features are byte n-grams hashed with FNV-1a
into ``buckets`` slots and L2-normalised, so the model is language-agnostic, has no vocabulary file and is a single matrix.
"""
from __future__ import annotations

import json

import numpy as np
import torch


def _features(text: str, n_min: int, n_max: int, buckets: int) -> tuple[np.ndarray, np.ndarray]:
    data = (" " + " ".join(text.lower().split()) + " ").encode("utf-8")[:4096]
    idx: dict[int, float] = {}
    for n in range(n_min, n_max + 1):
        for i in range(len(data) - n + 1):
            h = 0x811C9DC5
            for b in data[i: i + n]:
                h = ((h ^ b) * 0x01000193) & 0xFFFFFFFF
            k = (h ^ n) % buckets
            idx[k] = idx.get(k, 0.0) + 1.0
    if not idx:
        return np.zeros(0, np.int64), np.zeros(0, np.float32)
    keys = np.fromiter(idx.keys(), np.int64, len(idx))
    vals = np.fromiter(idx.values(), np.float32, len(idx))
    return keys, vals / np.linalg.norm(vals)


class HashedNgramClassifier:
    def __init__(self, labels: list[str], n_min: int = 1, n_max: int = 3, buckets: int = 1 << 15, weights: torch.Tensor | None = None,
                 bias: torch.Tensor | None = None):
        self.labels, self.n_min, self.n_max, self.buckets = list(labels), n_min, n_max, buckets
        self.W = weights if weights is not None else torch.zeros(buckets, len(labels))
        self.b = bias if bias is not None else torch.zeros(len(labels))

    def _dense(self, texts) -> torch.Tensor:
        X = torch.zeros(len(texts), self.buckets)
        for r, t in enumerate(texts):
            k, v = _features(t, self.n_min, self.n_max, self.buckets)
            if len(k):
                X[r, torch.from_numpy(k)] = torch.from_numpy(v)
        return X

    @classmethod
    def fit(cls, texts: list[str], labels: list[str], epochs: int = 30, lr: float = 0.5, seed: int = 0, **kw) -> "HashedNgramClassifier":
        names = sorted(set(labels))
        if len(names) < 2:
            raise ValueError("a classifier needs at least two classes")
        m = cls(names, **kw)
        X = m._dense(texts)
        y = torch.tensor([names.index(l) for l in labels])
        W, b = m.W.clone().requires_grad_(True), m.b.clone().requires_grad_(True)
        opt = torch.optim.SGD([W, b], lr=lr)
        g = torch.Generator().manual_seed(seed)
        for _ in range(epochs):
            perm = torch.randperm(len(texts), generator=g)
            for lo in range(0, len(texts), 32):
                sel = perm[lo: lo + 32]
                loss = torch.nn.functional.cross_entropy(X[sel] @ W + b, y[sel])
                opt.zero_grad()
                loss.backward()
                opt.step()
        m.W, m.b = W.detach(), b.detach()
        return m

    @torch.no_grad()
    def predict_proba(self, texts: list[str]) -> torch.Tensor:
        return torch.softmax(self._dense(texts) @ self.W + self.b, -1)

    def predict(self, text: str) -> tuple[str, float]:
        p = self.predict_proba([text])[0]
        i = int(p.argmax())
        return self.labels[i], float(p[i])

    def save(self, path: str):
        nz = self.W.abs().sum(1).nonzero().squeeze(1)                     # only the buckets training touched
        with open(path, "w") as f:
            json.dump({"schema": "b200.hashed_ngram_classifier.v1", "labels": self.labels, "nMin": self.n_min, "nMax": self.n_max, "buckets": self.buckets,
                       "rows": nz.tolist(), "weights": self.W[nz].tolist(), "bias": self.b.tolist()}, f)

    @classmethod
    def load(cls, path: str) -> "HashedNgramClassifier":
        with open(path) as f:
            o = json.load(f)
        if o.get("schema") != "b200.hashed_ngram_classifier.v1":
            raise ValueError("not a classifier file")
        W = torch.zeros(o["buckets"], len(o["labels"]))
        if o["rows"]:
            W[torch.tensor(o["rows"])] = torch.tensor(o["weights"])
        return cls(o["labels"], o["nMin"], o["nMax"], o["buckets"], W, torch.tensor(o["bias"]))


def classifier_stage(docs: list[dict], model: HashedNgramClassifier, keep_label: str, min_confidence: float = 0.5, stage: str = "quality_classifier"):
    """Refinery stage: keep the documents the model assigns to ``keep_label`` with at least ``min_confidence``."""
    texts = [" ".join(d["lines"]) for d in docs]
    if not texts:
        return [], {"stage": stage, "inputDocuments": 0, "keptDocuments": 0, "rejected": {}}
    P = model.predict_proba(texts)
    k = model.labels.index(keep_label)
    kept, rejected = [], {}
    for d, p in zip(docs, P):
        if float(p[k]) >= min_confidence and int(p.argmax()) == k:
            kept.append(d)
        else:
            lab = model.labels[int(p.argmax())]
            rejected[lab] = rejected.get(lab, 0) + 1
    return kept, {"stage": stage, "inputDocuments": len(docs), "keptDocuments": len(kept), "keepLabel": keep_label, "minConfidence": min_confidence,
                  "rejected": rejected}
