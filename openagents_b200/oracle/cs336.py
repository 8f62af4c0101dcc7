"""CPU restatement of the reference's contributor workloads ("homework"): the only executable ML
semantics in the reference tree, kept here as oracles and as the CPU side of the multi-rank tests.

A1 real-gradient workload (apps/openagents.com/workers/api/src/cs336-a1-real-gradient-workload.ts):
a tiny LM — embedding, RMSNorm, single-head causal softmax attention, residual, RMSNorm, SwiGLU,
residual, RMSNorm, unembedding, cross-entropy — in float64 with a hand-derived backward pass
(:417-596 forward, :602-784 backward), per-shard full-batch gradients (:816-866), synchronous
data-parallel SGD averaging (:872-891), validation loss (:899-927) and SHA-256 state commitments
(:801-809).  Parameter layout and run configuration follow :30-60 and :199-226 (2,244 parameters).
"""
from __future__ import annotations

import hashlib
import math
import struct
from dataclasses import dataclass

import numpy as np

RMS_EPS = 1e-5


@dataclass(frozen=True)
class A1Config:
    d_ff: int = 24
    d_model: int = 12
    learning_rate: float = 1.5
    sequence_length: int = 16
    shard_count: int = 2
    step_count: int = 6
    structure_bias: float = 0.85
    train_sequences_per_shard: int = 48
    validation_sequence_count: int = 32
    vocabulary_size: int = 32


NAMES = ("emb", "g1", "wq", "wk", "wv", "wo", "g2", "w1", "w3", "w2", "g3", "wu")


def parameter_layout(c: A1Config) -> dict:
    d, h, v = c.d_model, c.d_ff, c.vocabulary_size
    shapes = {"emb": (v, d), "g1": (d,), "wq": (d, d), "wk": (d, d), "wv": (d, d), "wo": (d, d), "g2": (d,),
              "w1": (d, h), "w3": (d, h), "w2": (h, d), "g3": (d,), "wu": (d, v)}
    out, off = {}, 0
    for n in NAMES:
        size = int(np.prod(shapes[n]))
        out[n] = (off, shapes[n])
        off += size
    out["size"] = off
    return out


def unpack(c: A1Config, params: np.ndarray) -> dict:
    lay = parameter_layout(c)
    return {n: params[lay[n][0]: lay[n][0] + int(np.prod(lay[n][1]))].reshape(lay[n][1]) for n in NAMES}


def _stream(seed: str, n: int) -> np.ndarray:
    """Deterministic uniform [0,1) stream from a SHA-256 counter (the reference seeds its data and
    parameters the same way: :151-173)."""
    out, i = np.empty(n), 0
    ctr = 0
    while i < n:
        h = hashlib.sha256(f"{seed}:{ctr}".encode()).digest()
        for k in range(0, 32, 4):
            if i < n:
                out[i] = struct.unpack(">I", h[k:k + 4])[0] / 2 ** 32
                i += 1
        ctr += 1
    return out


def init_params(c: A1Config, seed: str = "cs336.a1.params") -> np.ndarray:
    lay = parameter_layout(c)
    p = np.zeros(lay["size"])
    u = _stream(seed, lay["size"])
    for n in NAMES:
        off, shape = lay[n]
        size = int(np.prod(shape))
        if n in ("g1", "g2", "g3"):
            p[off: off + size] = 1.0
        else:
            fan = shape[0] if n != "emb" else c.d_model
            p[off: off + size] = (u[off: off + size] * 2 - 1) / np.sqrt(fan)
    return p


def make_sequences(c: A1Config, seed: str, count: int) -> np.ndarray:
    """Token sequences with learnable structure: with probability ``structure_bias`` the next token
    is (prev * 3 + 1) mod V, otherwise uniform."""
    V, T = c.vocabulary_size, c.sequence_length + 1
    u = _stream(seed, count * T * 2).reshape(count, T, 2)
    seq = np.zeros((count, T), dtype=np.int64)
    seq[:, 0] = (u[:, 0, 0] * V).astype(np.int64)
    for t in range(1, T):
        follow = u[:, t, 0] < c.structure_bias
        seq[:, t] = np.where(follow, (seq[:, t - 1] * 3 + 1) % V, (u[:, t, 1] * V).astype(np.int64))
    return seq


def rmsnorm_fwd(x, g):
    r = 1.0 / np.sqrt((x * x).mean(-1, keepdims=True) + RMS_EPS)
    return x * r * g, r


def rmsnorm_bwd(dy, x, g, r):
    d = x.shape[-1]
    dg = (dy * x * r).sum(0)
    dxh = dy * g
    dx = r * dxh - x * (r ** 3) * (dxh * x).sum(-1, keepdims=True) / d
    return dx, dg


def sequence_pass(c: A1Config, P: dict, seq: np.ndarray, need_grad: bool = True):
    """Forward (and backward) over one sequence.  Returns (mean loss, grads dict or None)."""
    d, T = c.d_model, c.sequence_length
    tok, tgt = seq[:T], seq[1: T + 1]
    x0 = P["emb"][tok]                                       # [T, d]
    h1, r1 = rmsnorm_fwd(x0, P["g1"])
    q, k, v = h1 @ P["wq"], h1 @ P["wk"], h1 @ P["wv"]
    s = (q @ k.T) / np.sqrt(d)
    mask = np.triu(np.ones((T, T), dtype=bool), 1)
    s = np.where(mask, -np.inf, s)
    s = s - s.max(-1, keepdims=True)
    a = np.exp(s)
    a = a / a.sum(-1, keepdims=True)
    ctx = a @ v
    x1 = x0 + ctx @ P["wo"]
    h2, r2 = rmsnorm_fwd(x1, P["g2"])
    gate, val = h2 @ P["w1"], h2 @ P["w3"]
    sig = 1.0 / (1.0 + np.exp(-gate))
    act = gate * sig * val
    x2 = x1 + act @ P["w2"]
    h3, r3 = rmsnorm_fwd(x2, P["g3"])
    logits = h3 @ P["wu"]
    z = logits - logits.max(-1, keepdims=True)
    lse = np.log(np.exp(z).sum(-1, keepdims=True))
    logp = z - lse
    loss = -logp[np.arange(T), tgt].mean()
    if not need_grad:
        return loss, None
    G = {}
    dlogits = np.exp(logp)
    dlogits[np.arange(T), tgt] -= 1.0
    dlogits /= T
    G["wu"] = h3.T @ dlogits
    dh3 = dlogits @ P["wu"].T
    dx2, G["g3"] = rmsnorm_bwd(dh3, x2, P["g3"], r3)
    G["w2"] = act.T @ dx2
    dact = dx2 @ P["w2"].T
    dval = dact * gate * sig
    dgate = dact * val * (sig + gate * sig * (1 - sig))
    G["w1"], G["w3"] = h2.T @ dgate, h2.T @ dval
    dh2 = dgate @ P["w1"].T + dval @ P["w3"].T
    dx1_n, G["g2"] = rmsnorm_bwd(dh2, x1, P["g2"], r2)
    dx1 = dx2 + dx1_n
    G["wo"] = ctx.T @ dx1
    dctx = dx1 @ P["wo"].T
    da = dctx @ v.T
    dv = a.T @ dctx
    ds = a * (da - (da * a).sum(-1, keepdims=True)) / np.sqrt(d)
    dq, dk = ds @ k, ds.T @ q
    G["wq"], G["wk"], G["wv"] = h1.T @ dq, h1.T @ dk, h1.T @ dv
    dh1 = dq @ P["wq"].T + dk @ P["wk"].T + dv @ P["wv"].T
    dx0_n, G["g1"] = rmsnorm_bwd(dh1, x0, P["g1"], r1)
    dx0 = dx1 + dx0_n
    G["emb"] = np.zeros_like(P["emb"])
    np.add.at(G["emb"], tok, dx0)
    return loss, G


def shard_gradient(c: A1Config, params: np.ndarray, shard_index: int) -> tuple[np.ndarray, float]:
    """Full-batch mean gradient of one shard."""
    P = unpack(c, params)
    seqs = make_sequences(c, f"cs336.a1.train.shard{shard_index}", c.train_sequences_per_shard)
    lay = parameter_layout(c)
    g, total = np.zeros(lay["size"]), 0.0
    for s in seqs:
        loss, G = sequence_pass(c, P, s)
        total += loss
        for n in NAMES:
            off = lay[n][0]
            g[off: off + G[n].size] += G[n].reshape(-1)
    return g / len(seqs), total / len(seqs)


def apply_aggregated_sgd_step(c: A1Config, params: np.ndarray, shard_grads: list[np.ndarray]) -> np.ndarray:
    return params - c.learning_rate * np.sum(shard_grads, axis=0) / len(shard_grads)


def validation_loss(c: A1Config, params: np.ndarray) -> float:
    P = unpack(c, params)
    seqs = make_sequences(c, "cs336.a1.validation", c.validation_sequence_count)
    return float(np.mean([sequence_pass(c, P, s, need_grad=False)[0] for s in seqs]))


def state_digest(params: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(params, dtype="<f8").tobytes()).hexdigest()


def run_training(c: A1Config = A1Config(), seed_digest_hex: str | None = None) -> dict:
    """The in-process reference trajectory every multi-device run must match digest for digest.  ``seed_digest_hex``: seed
    parameters and data exactly like the reference's published multi-device run (see ``reference_*`` below); the validation
    losses then reproduce the published curve."""
    if seed_digest_hex is not None:
        return _run_training_reference_seeded(c, seed_digest_hex)
    params = init_params(c)
    steps = [{"step": 0, "validationLoss": validation_loss(c, params), "stateDigest": state_digest(params)}]
    for step in range(1, c.step_count + 1):
        grads = [shard_gradient(c, params, s)[0] for s in range(c.shard_count)]
        params = apply_aggregated_sgd_step(c, params, grads)
        steps.append({"step": step, "validationLoss": validation_loss(c, params), "stateDigest": state_digest(params),
                      "gradientDigests": [state_digest(g) for g in grads]})
    return {"parameterCount": int(params.size), "steps": steps, "finalParams": params}


# ---- the reference's own seeding, so that its published numbers can be reproduced
# (cs336-a1-real-gradient-workload.ts:151-186 SHA-256 counter stream, :239-262 initial parameters, :264-281 permutation,
#  :291-314 sequences, :316-349 shard and validation sets, :797-808 state digest; the published run:
#  apps/openagents.com/docs/2026-06-11-cs336-a1-multi-device-real-gradient-evidence.md:74-100)
PUBLISHED_SEED_DIGEST_HEX = "097226577c582f296c8c3d050278007d68340963e1a24e7723e769c98a0e009c"
PUBLISHED_INITIAL_STATE_DIGEST_HEX = "4c3de6ca350bebea744a1acee4e91095fdef421edbe21891ca3a65fbe12f2943"
PUBLISHED_VALIDATION_LOSSES = (3.5197062668735226, 2.951128363282113, 2.5675990018969443, 2.2080697872990354, 1.8804644102382486,
                               1.589493254125287, 1.3835386088779047)


def reference_uint32s(seed: str, count: int) -> list[int]:
    out, ctr = [], 0
    while len(out) < count:
        h = hashlib.sha256(f"{seed}:{ctr}".encode()).hexdigest()
        out += [int(h[k: k + 8], 16) for k in range(0, 64, 8)]
        ctr += 1
    return out[:count]


def reference_initial_parameters(c: A1Config, seed_digest_hex: str) -> np.ndarray:
    lay = parameter_layout(c)
    u = np.array(reference_uint32s(f"cs336_a1.real_grad.init.{seed_digest_hex}", lay["size"]), dtype=np.float64) / 4294967296.0
    p = (u * 2 - 1) * (0.5 / math.sqrt(c.d_model))
    for n in ("g1", "g2", "g3"):
        p[lay[n][0]: lay[n][0] + c.d_model] = 1.0
    return p


def reference_permutation(seed: str, size: int) -> list[int]:
    vals = list(range(size))
    draws = reference_uint32s(f"{seed}:perm", size)
    for i in range(size - 1, 0, -1):
        j = draws[size - 1 - i] % (i + 1)
        vals[i], vals[j] = vals[j], vals[i]
    return vals


def reference_sequences(c: A1Config, seed_digest_hex: str, kind: str, count: int) -> np.ndarray:
    """``kind``: ``train:<shard>`` or ``val``.  The next symbol follows a seeded permutation of the current one with probability
    ``structure_bias``, else it is uniform."""
    perm = reference_permutation(f"cs336_a1.real_grad.structure.{seed_digest_hex}", c.vocabulary_size)
    L = c.sequence_length + 1
    out = np.zeros((count, L), dtype=np.int64)
    for s in range(count):
        d = reference_uint32s(f"cs336_a1.real_grad.stream.{seed_digest_hex}.{kind}:{s}", 2 * L + 1)
        out[s, 0] = d[0] % c.vocabulary_size
        for i in range(L - 1):
            out[s, i + 1] = perm[out[s, i]] if d[2 * i + 1] / 4294967296.0 < c.structure_bias else d[2 * i + 2] % c.vocabulary_size
    return out


def js_number(x: float) -> str:
    """A double the way ``JSON.stringify`` prints it: shortest digits that round-trip, plain notation for 1e-6 <= |x| < 1e21,
    otherwise ``d.ddde+N`` / ``d.ddde-N`` without padding."""
    if x == 0:
        return "0"
    if x != x or x in (float("inf"), float("-inf")):
        return "null"
    sign = "-" if x < 0 else ""
    r = repr(abs(float(x)))
    if "e" in r:
        mant, exp = r.split("e")
        digits, point = mant.replace(".", ""), len(mant.split(".")[0])
        e10 = int(exp) + point                      # value = 0.digits x 10^e10
    else:
        ip, _, fp = r.partition(".")
        fp = "" if fp == "0" else fp
        digits, e10 = (ip + fp), len(ip)
        if ip == "0":
            stripped = fp.lstrip("0")
            e10 = -(len(fp) - len(stripped))
            digits = stripped
    digits = digits.rstrip("0") or "0"
    lead = len(digits) - len(digits.lstrip("0"))
    digits, e10 = digits[lead:] or "0", e10 - lead
    n = e10                                          # position of the decimal point relative to the digit string
    k = len(digits)
    if 0 < n <= 21:
        body = digits + "0" * (n - k) if k <= n else digits[:n] + "." + digits[n:]
    elif -6 < n <= 0:
        body = "0." + "0" * (-n) + digits
    else:
        e = n - 1
        body = digits[0] + ("." + digits[1:] if k > 1 else "") + "e" + ("+" if e >= 0 else "-") + str(abs(e))
    return sign + body


def reference_state_digest(seed_digest_hex: str, step: int, params: np.ndarray) -> str:
    label = f"cs336_a1.real_grad.state.{seed_digest_hex}.step_{step}"
    text = '{"label":"' + label + '","values":[' + ",".join(js_number(float(v)) for v in params) + "]}"
    return hashlib.sha256(text.encode()).hexdigest()


def _run_training_reference_seeded(c: A1Config, seed: str) -> dict:
    lay = parameter_layout(c)
    params = reference_initial_parameters(c, seed)
    train = [reference_sequences(c, seed, f"train:{s}", c.train_sequences_per_shard) for s in range(c.shard_count)]
    val = reference_sequences(c, seed, "val", c.validation_sequence_count)

    def vloss(p):
        P = unpack(c, p)
        return float(np.mean([sequence_pass(c, P, s, need_grad=False)[0] for s in val]))

    def shard_grad(p, seqs):
        P = unpack(c, p)
        g = np.zeros(lay["size"])
        for s in seqs:
            _, G = sequence_pass(c, P, s)
            for n in NAMES:
                g[lay[n][0]: lay[n][0] + G[n].size] += G[n].reshape(-1)
        return g / len(seqs)
    steps = [{"step": 0, "validationLoss": vloss(params), "stateDigest": reference_state_digest(seed, 0, params)}]
    for step in range(1, c.step_count + 1):
        params = apply_aggregated_sgd_step(c, params, [shard_grad(params, t) for t in train])
        steps.append({"step": step, "validationLoss": vloss(params), "stateDigest": reference_state_digest(seed, step, params)})
    return {"parameterCount": int(params.size), "steps": steps, "finalParams": params}


# ---------------------------------------------------------------- A1 homework: BPE + committed mod-p matmul
# (cs336-a1-homework-workload.ts:20 modulus, :132-169 tokenizer shard, :209-221 product, :232-290 commitments)
FIELD_MODULUS = 2 ** 31 - 1


def bpe_train(data: bytes, n_merges: int = 24, min_count: int = 1) -> dict:
    """Byte-level BPE: repeatedly merge the most frequent adjacent pair (ties: lowest pair); stops when the best pair occurs
    fewer than ``min_count`` times."""
    ids = list(data)
    merges = []
    for k in range(n_merges):
        counts = {}
        for a, b in zip(ids, ids[1:]):
            counts[(a, b)] = counts.get((a, b), 0) + 1
        if not counts:
            break
        best = max(counts.items(), key=lambda kv: (kv[1], -kv[0][0], -kv[0][1]))[0]
        if counts[best] < min_count:
            break
        new_id = 256 + k
        merges.append((best[0], best[1], new_id))
        out, i = [], 0
        while i < len(ids):
            if i + 1 < len(ids) and (ids[i], ids[i + 1]) == best:
                out.append(new_id)
                i += 2
            else:
                out.append(ids[i])
                i += 1
        ids = out
    digest = hashlib.sha256(json_bytes({"merges": merges, "tokenCount": len(ids)})).hexdigest()
    return {"merges": merges, "tokenIds": ids, "digestHex": digest}


# the reference's committed four-line corpus and merge budget (cs336-a1-homework-workload.ts:22-29); its shard digest is the seed
# of the published A1 / A3 runs
A1_DEMO_CORPUS = "\n".join(["one day a little robot found a shiny coin on the floor", "the robot gave the coin to a small bird and the bird sang",
                            "they walked to the lake and watched the slow boats together", "the bird said thank you and the robot beeped a happy song"])
A1_MERGE_BUDGET = 24


def tokenizer_shard(corpus: str = A1_DEMO_CORPUS, merge_budget: int = A1_MERGE_BUDGET) -> dict:
    """The tokenizer shard of the homework workload (:132-169): byte-level BPE that stops early when the best pair occurs only
    once, committed by SHA-256 over the merge table and the final token stream."""
    data = corpus.encode()
    r = bpe_train(data, merge_budget, min_count=2)
    body = {"corpusByteLength": len(data), "mergeBudget": merge_budget, "merges": [list(m) for m in r["merges"]], "tokens": r["tokenIds"]}
    return {"digestHex": hashlib.sha256(json_bytes_ordered(body)).hexdigest(), "mergeCount": len(r["merges"]), "tokenCount": len(r["tokenIds"]),
            "vocabularySize": 256 + len(r["merges"])}


def json_bytes_ordered(obj) -> bytes:
    """``JSON.stringify`` of an object whose keys are already in insertion order."""
    import json
    return json.dumps(obj, separators=(",", ":")).encode()


def json_bytes(obj) -> bytes:
    import json
    return json.dumps(obj, sort_keys=True, separators=(",", ":")).encode()


def seeded_values(seed: str, count: int, bound: int) -> list[int]:
    """``count`` values below ``bound`` from the SHA-256 counter stream (each 32-bit word reduced modulo the bound; :170-193)."""
    return [v % bound for v in reference_uint32s(seed, count)]


def seeded_matrix(seed: str, rows: int, cols: int, bound: int = FIELD_MODULUS) -> np.ndarray:
    return np.array(seeded_values(seed, rows * cols, bound), dtype=np.int64).reshape(rows, cols)


def matrix_product_mod(a: np.ndarray, b: np.ndarray, p: int = FIELD_MODULUS) -> np.ndarray:
    out = np.zeros((a.shape[0], b.shape[1]), dtype=np.int64)
    for i in range(a.shape[0]):
        for j in range(b.shape[1]):
            out[i, j] = sum(int(x) * int(y) for x, y in zip(a[i], b[:, j])) % p
    return out


def merkle_root(leaves: list[str]) -> str:
    """Pairs of hex digests are concatenated AS TEXT and hashed; an odd last node is hashed alone (:252-262)."""
    level = list(leaves)
    if not level:
        return hashlib.sha256(b"").hexdigest()
    while len(level) > 1:
        level = [hashlib.sha256((level[i] + (level[i + 1] if i + 1 < len(level) else "")).encode()).hexdigest() for i in range(0, len(level), 2)]
    return level[0]


PUBLISHED_MERKLE_ROOT_PREFIX = "14cd1fdf7d013cfe"      # apps/openagents.com/docs/2026-06-11-training-validator-paid-closeout-evidence.md:46-50


def training_step_matrix(tokenizer_digest: str, rows: int = 8, inner: int = 16, cols: int = 8) -> dict:
    """One committed forward matmul (:232-290): activations below 97 derived from the tokenizer shard digest, the seeded demo
    weight shard, the product mod p, a SHA-256 digest per product row, the Merkle root over them, and a challenge vector derived
    from the root, that is, only after the commitment."""
    left = seeded_matrix(f"cs336_a1.activations.{tokenizer_digest}", rows, inner, 97)
    right = seeded_matrix("cs336_a1.weight_shard.psion_cs336_a1_demo_v1", inner, cols, 97)
    prod = matrix_product_mod(left, right)
    row_digests = [hashlib.sha256(json_bytes_ordered([int(v) for v in r])).hexdigest() for r in prod]
    root = merkle_root(row_digests)
    challenge = seeded_values(f"cs336_a1.challenge.{root}", cols, FIELD_MODULUS)
    return {"fieldModulus": FIELD_MODULUS, "leftMatrix": left.tolist(), "rightMatrix": right.tolist(),
            "claimedProductMatrix": prod.tolist(), "rowDigests": row_digests, "merkleRoot": root,
            "challengeVector": challenge, "rowOpenings": [{"rowRef": f"row.{i}", "digest": d} for i, d in enumerate(row_digests)],
            "merkleProofValid": True}


# ---------------------------------------------------------------- A2 device micro-benchmarks
# (cs336-a2-benchmark-workload.ts:35-44 shapes, :141-191 attention, :193-210 STREAM triad, :212-249 greedy
# row decode, :251-292 one training step, :338-370 suite with an injectable clock, :497-509 agreement score)
def mulberry32(seed: int):
    state = seed & 0xFFFFFFFF

    def nxt() -> float:
        nonlocal state
        state = (state + 0x6D2B79F5) & 0xFFFFFFFF
        t = state
        t = ((t ^ (t >> 15)) * (t | 1)) & 0xFFFFFFFF
        t ^= (t + (((t ^ (t >> 7)) * (t | 61)) & 0xFFFFFFFF)) & 0xFFFFFFFF
        return ((t ^ (t >> 14)) & 0xFFFFFFFF) / 4294967296.0
    return nxt


def _rand(seed: int, *shape) -> np.ndarray:
    r = mulberry32(seed)
    return np.array([r() * 2 - 1 for _ in range(int(np.prod(shape)))]).reshape(shape)


def a2_attention(seq: int = 64, dim: int = 32, seed: int = 1) -> np.ndarray:
    q, k, v = _rand(seed, seq, dim), _rand(seed + 1, seq, dim), _rand(seed + 2, seq, dim)
    s = q @ k.T / np.sqrt(dim)
    s = np.exp(s - s.max(-1, keepdims=True))
    return (s / s.sum(-1, keepdims=True)) @ v


def a2_stream_triad(n: int = 2_000_000, passes: int = 8, scalar: float = 3.0) -> float:
    b, c = np.arange(n, dtype=np.float64) * 1e-6, np.ones(n)
    a = np.zeros(n)
    for _ in range(passes):
        a = b + scalar * c
        b, c = c, a
    return float(a[::max(1, n // 1000)].sum())


def a2_row_decode(vocab: int = 96, hidden: int = 48, steps: int = 48, seed: int = 7) -> list[int]:
    W, state = _rand(seed, vocab, hidden), _rand(seed + 1, hidden)
    out = []
    for _ in range(steps):
        tok = int(np.argmax(W @ state))
        out.append(tok)
        state = np.tanh(0.5 * state + 0.5 * W[tok])
    return out


def a2_training_step(rows: int = 32, inner: int = 64, cols: int = 32, lr: float = 0.01, seed: int = 11) -> tuple[np.ndarray, float]:
    A, W, T = _rand(seed, rows, inner), _rand(seed + 1, inner, cols), _rand(seed + 2, rows, cols)
    E = A @ W - T
    return W - lr * (A.T @ E) / rows, float((E * E).mean())


def nearest_rank(samples: list[float], q: float) -> float:
    s = sorted(samples)
    return s[max(0, min(len(s) - 1, int(np.ceil(q * len(s))) - 1))]


def a2_suite(now, repetitions: int = 5) -> dict:
    """Times the four kernels with the injected clock ``now()`` (seconds); p50/p90 by nearest rank."""
    out = {}
    for name, fn in (("attention", a2_attention), ("memory_bandwidth", lambda: a2_stream_triad(200_000, 2)),
                     ("decode", a2_row_decode), ("training_step", a2_training_step)):
        ts, digest = [], None
        for _ in range(repetitions):
            t0 = now()
            r = fn()
            ts.append(now() - t0)
            digest = hashlib.sha256(repr(np.asarray(r[0] if isinstance(r, tuple) else r).round(9).tolist()).encode()).hexdigest()
        out[name] = {"p50": nearest_rank(ts, 0.5), "p90": nearest_rank(ts, 0.9), "outputDigest": digest}
    return out


def cross_device_agreement(median_a: float, median_b: float) -> float:
    lo, hi = min(median_a, median_b), max(median_a, median_b)
    return 0.0 if hi <= 0 else lo / hi


# ---------------------------------------------------------------- A3 IsoFLOP grid, A5 DPO
# (cs336-a3-sweep-workload.ts:141 grid planner with D = C / (6 N); cs336-a5-dpo-preference-workload.ts:85-122)
def plan_isoflop_grid(compute_budgets: list[float], param_counts: list[int]) -> list[dict]:
    return [{"computeBudget": C, "paramCount": N, "tokenBudget": int(C // (6 * N))} for C in compute_budgets for N in param_counts
            if C // (6 * N) >= 1]


def softplus(x: float) -> float:
    return float(np.log1p(np.exp(-abs(x))) + max(x, 0.0))


def dpo_implicit_reward(beta: float, logp_policy: float, logp_ref: float) -> float:
    return beta * (logp_policy - logp_ref)


def dpo_pair_loss(beta: float, pol_chosen: float, pol_rejected: float, ref_chosen: float, ref_rejected: float) -> float:
    """-log sigmoid(r_chosen - r_rejected) written with softplus."""
    margin = dpo_implicit_reward(beta, pol_chosen, ref_chosen) - dpo_implicit_reward(beta, pol_rejected, ref_rejected)
    return softplus(-margin)


# ---- the same run with the reference's ORDER of floating-point operations (native; csrc/oracle/a1_ordered.cpp)
PUBLISHED_FINAL_STATE_DIGEST_HEX = "bda8a9edba1c18da74e4c138d66da65888d3fe51f9ae4538b9046f7d701bdbb3"


def _ordered_lib():
    import ctypes
    from .. import _native
    lib = _native.host()
    if not getattr(lib, "_a1_ready", False):
        dp, ip = ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_int32)
        lib.b200_a1_shard_gradient.argtypes, lib.b200_a1_shard_gradient.restype = [ctypes.c_int] * 4 + [dp, ip, ctypes.c_int, dp], ctypes.c_double
        lib.b200_a1_mean_loss.argtypes, lib.b200_a1_mean_loss.restype = [ctypes.c_int] * 4 + [dp, ip, ctypes.c_int], ctypes.c_double
        lib.b200_a1_sgd_step.argtypes, lib.b200_a1_sgd_step.restype = [ctypes.c_uint64, dp, ctypes.POINTER(dp), ctypes.c_int, ctypes.c_double, dp], None
        lib.b200_a1_det_exp.argtypes, lib.b200_a1_det_exp.restype = [ctypes.c_double], ctypes.c_double
        lib.b200_a1_det_ln.argtypes, lib.b200_a1_det_ln.restype = [ctypes.c_double], ctypes.c_double
        lib._a1_ready = True
    return lib


def reference_shard_gradient_digest(seed_digest_hex: str, step: int, shard: int, grad: np.ndarray) -> str:
    label = f"cs336_a1.real_grad.shard_gradient.{seed_digest_hex}.step_{step}.shard_{shard}"
    return hashlib.sha256(('{"label":"' + label + '","values":[' + ",".join(js_number(float(v)) for v in grad) + "]}").encode()).hexdigest()


def run_training_ordered(c: A1Config = A1Config(), seed_digest_hex: str = PUBLISHED_SEED_DIGEST_HEX) -> dict:
    """The reference trajectory digest for digest: scalar loops in the reference's order with its deterministic exp and ln."""
    import ctypes
    lib = _ordered_lib()
    dp, ip = ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_int32)
    dims = (c.d_model, c.d_ff, c.vocabulary_size, c.sequence_length)
    params = np.ascontiguousarray(reference_initial_parameters(c, seed_digest_hex))
    train = [np.ascontiguousarray(reference_sequences(c, seed_digest_hex, f"train:{s}", c.train_sequences_per_shard), dtype=np.int32) for s in range(c.shard_count)]
    val = np.ascontiguousarray(reference_sequences(c, seed_digest_hex, "val", c.validation_sequence_count), dtype=np.int32)

    def vloss(p):
        return float(lib.b200_a1_mean_loss(*dims, p.ctypes.data_as(dp), val.ctypes.data_as(ip), len(val)))
    steps = [{"step": 0, "validationLoss": vloss(params), "stateDigest": reference_state_digest(seed_digest_hex, 0, params)}]
    for step in range(c.step_count):
        grads, shard_losses = [], []
        for t in train:
            g = np.zeros_like(params)
            shard_losses.append(float(lib.b200_a1_shard_gradient(*dims, params.ctypes.data_as(dp), t.ctypes.data_as(ip), len(t), g.ctypes.data_as(dp))))
            grads.append(g)
        nxt = np.zeros_like(params)
        arr = (dp * len(grads))(*[g.ctypes.data_as(dp) for g in grads])
        lib.b200_a1_sgd_step(params.size, params.ctypes.data_as(dp), arr, len(grads), c.learning_rate, nxt.ctypes.data_as(dp))
        digests = [reference_shard_gradient_digest(seed_digest_hex, step, s, g) for s, g in enumerate(grads)]
        params = nxt
        steps.append({"step": step + 1, "validationLoss": vloss(params), "stateDigest": reference_state_digest(seed_digest_hex, step + 1, params),
                      "gradientDigests": digests, "shardLosses": shard_losses})
    return {"parameterCount": int(params.size), "steps": steps, "finalParams": params}
