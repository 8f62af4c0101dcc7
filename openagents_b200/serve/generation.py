"""Tokenizer, sampling parameters and the continuous-batching scheduler.

The scheduler admits requests up to ``max_num_seqs``, prefills prompts in chunks so a long prompt
does not monopolise a step, and decodes every running sequence together each step.  Sampling
options are the ones the reference's provider-neutral request carries (maxTokens, temperature,
topP, topK, stop: apps/pylon/packages/runtime/src/llm/request.ts:5-11).  Throughput levers named by
the reference's serving reports (``max_num_seqs``, prefix caching, chunked prefill:
apps/openagents.com/workers/api/src/inference/gym/throughput.ts:66-80) map to the constructor
arguments here.
"""
from __future__ import annotations

import hashlib
import itertools
import time
from dataclasses import dataclass, field

import torch

from .backend import Backend

CHAT_TEMPLATE = "{% for m in messages %}<|{{ m.role }}|>\n{{ m.content }}\n{% endfor %}<|assistant|>\n"
CHAT_TEMPLATE_DIGEST = "sha256:" + hashlib.sha256(CHAT_TEMPLATE.encode()).hexdigest()


class ByteTokenizer:
    """UTF-8 bytes as token ids 0..255; 256 = end of sequence.  Models with a GGUF vocabulary use
    ``VocabTokenizer``; synthetic models (random weights, no vocabulary) use this one."""
    eos_id = 256

    def __init__(self, vocab_size: int):
        if vocab_size < 257:
            raise ValueError("byte tokenizer needs a vocabulary of at least 257 ids")
        self.vocab_size = vocab_size

    def encode(self, text: str) -> list[int]:
        return list(text.encode("utf-8"))

    def decode(self, ids) -> str:
        return bytes(i for i in ids if 0 <= i < 256).decode("utf-8", "replace")


class VocabTokenizer:
    """Greedy longest-match over ``tokenizer.ggml.tokens`` (enough for round-tripping the
    vocabulary of a loaded GGUF file; merges-based BPE is ``oracle.cs336.bpe_train``'s domain)."""

    def __init__(self, tokens: list[str], eos_id: int):
        self.tokens, self.eos_id, self.vocab_size = tokens, eos_id, len(tokens)
        self.index = {t: i for i, t in enumerate(tokens)}
        self.maxlen = max((len(t) for t in tokens), default=1)

    def encode(self, text: str) -> list[int]:
        out, i = [], 0
        while i < len(text):
            for n in range(min(self.maxlen, len(text) - i), 0, -1):
                t = self.index.get(text[i:i + n])
                if t is not None:
                    out.append(t)
                    i += n
                    break
            else:
                i += 1
        return out

    def decode(self, ids) -> str:
        return "".join(self.tokens[i] for i in ids if 0 <= i < len(self.tokens))


def _byte_alphabet() -> dict[int, str]:
    """The printable stand-in for each byte that byte-level BPE vocabularies use (GPT-2 convention)."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    table, n = {}, 0
    for b in range(256):
        if b in keep:
            table[b] = chr(b)
        else:
            table[b] = chr(256 + n)
            n += 1
    return table


class BpeTokenizer:
    """Byte-level BPE from a GGUF file's ``tokenizer.ggml.tokens`` and ``tokenizer.ggml.merges`` (model ``gpt2``, the
    scheme of the llama-3, qwen and gpt-oss vocabularies): text is split into pre-token pieces, each piece's bytes are
    mapped to the printable alphabet, and adjacent symbols are merged in rank order.  Special tokens
    (``tokenizer.ggml.token_type`` 3 or 4, e.g. ``<|eot_id|>``) are matched verbatim before the split."""
    _SPLIT = r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+"

    def __init__(self, tokens: list[str], merges: list[str], eos_id: int, bos_id: int | None = None,
                 token_types: list[int] | None = None):
        import regex
        self.tokens, self.eos_id, self.bos_id, self.vocab_size = tokens, eos_id, bos_id, len(tokens)
        self.index = {t: i for i, t in enumerate(tokens)}
        self.rank = {tuple(m.split(" ", 1)): i for i, m in enumerate(merges)}
        self.b2u = _byte_alphabet()
        self.u2b = {u: b for b, u in self.b2u.items()}
        self.split = regex.compile(self._SPLIT)
        special = [t for i, t in enumerate(tokens) if token_types and i < len(token_types) and token_types[i] in (3, 4)]
        self.special = sorted(special, key=len, reverse=True)
        self.special_re = regex.compile("|".join(regex.escape(t) for t in self.special)) if self.special else None
        self._cache: dict[str, list[int]] = {}

    def _bpe(self, piece: str) -> list[int]:
        hit = self._cache.get(piece)
        if hit is not None:
            return hit
        sym = [self.b2u[b] for b in piece.encode("utf-8")]
        while len(sym) > 1:
            best, at = None, -1
            for i in range(len(sym) - 1):
                r = self.rank.get((sym[i], sym[i + 1]))
                if r is not None and (best is None or r < best):
                    best, at = r, i
            if best is None:
                break
            sym[at: at + 2] = [sym[at] + sym[at + 1]]
        ids = []
        for t in sym:
            i = self.index.get(t)
            if i is None:                      # a symbol the vocabulary lacks: fall back to its single-byte tokens
                ids += [self.index[c] for c in t if c in self.index]
            else:
                ids.append(i)
        if len(self._cache) < 65536:
            self._cache[piece] = ids
        return ids

    def _encode_plain(self, text: str) -> list[int]:
        out: list[int] = []
        for piece in self.split.findall(text):
            out += self._bpe(piece)
        return out

    def encode(self, text: str) -> list[int]:
        if not self.special_re:
            return self._encode_plain(text)
        out, pos = [], 0
        for m in self.special_re.finditer(text):
            out += self._encode_plain(text[pos: m.start()])
            out.append(self.index[m.group(0)])
            pos = m.end()
        return out + self._encode_plain(text[pos:])

    def decode(self, ids) -> str:
        buf = bytearray()
        for i in ids:
            if 0 <= i < len(self.tokens):
                t = self.tokens[i]
                if t in self.special:
                    buf += t.encode("utf-8")
                else:
                    buf += bytes(self.u2b[c] for c in t if c in self.u2b)
        return buf.decode("utf-8", "replace")


class ByteBpeTokenizer:
    """The native byte-level BPE (``data.bpe.ByteBpe``) behind the serving tokenizer interface.  End of sequence is the
    end-of-turn marker when the vocabulary has one (instruction-tuned checkpoints), else ``<|endoftext|>``."""

    def __init__(self, spec_json: str, vocab_size: int):
        from ..data.bpe import ByteBpe
        self.bpe = ByteBpe.from_json(spec_json)
        if self.bpe.vocab_size > vocab_size:
            raise ValueError("the tokenizer has more ids than the model")
        self.vocab_size = vocab_size
        ids = self.bpe.special_ids
        self.eos_id = ids.get("<|end|>", ids.get("<|endoftext|>", vocab_size - 1))
        self.bos_id = None

    def encode(self, text: str) -> list[int]:
        return self.bpe.encode(text)

    def decode(self, ids) -> str:
        return self.bpe.decode([i for i in ids if 0 <= i < self.bpe.vocab_size])

    def decode_bytes(self, ids) -> bytes:
        return self.bpe.decode_bytes([i for i in ids if 0 <= i < self.bpe.vocab_size])


def tokenizer_from_metadata(meta: dict, vocab_size: int):
    """The tokenizer a GGUF file describes: byte-level BPE when it carries merges, greedy longest match over the token
    list when it only has tokens, raw bytes when it has neither (synthetic models)."""
    own = meta.get("tokenizer.b200.byte_bpe")
    if own:                                        # a checkpoint tuned by this framework carries the tokenizer it was tuned with
        return ByteBpeTokenizer(own if isinstance(own, str) else bytes(own).decode(), vocab_size)
    tokens = meta.get("tokenizer.ggml.tokens")
    if not tokens:
        return ByteTokenizer(vocab_size)
    tokens = [t if isinstance(t, str) else bytes(t).decode("utf-8", "replace") for t in tokens]
    eos = int(meta.get("tokenizer.ggml.eos_token_id", len(tokens) - 1))
    merges = meta.get("tokenizer.ggml.merges")
    if merges:
        bos = meta.get("tokenizer.ggml.bos_token_id")
        types = meta.get("tokenizer.ggml.token_type")
        return BpeTokenizer(tokens, [m if isinstance(m, str) else bytes(m).decode() for m in merges], eos,
                            None if bos is None else int(bos), list(types) if types is not None else None)
    return VocabTokenizer(tokens, eos)


def render_chat(messages: list[dict], template: str | None = None, bos_token: str = "", eos_token: str = "", tools=None, **kwargs) -> str:
    """The prompt text for a list of chat messages.  ``template``: a GGUF ``tokenizer.chat_template`` that the caller has
    ADMITTED (digest allowlist); it is rendered in an immutable sandbox (no attribute access to Python internals, no
    mutation of the inputs) with the variables model templates expect (``messages``, ``add_generation_prompt``,
    ``bos_token``, ``eos_token``, ``tools``, plus ``kwargs`` such as ``reasoning_effort``).  A template that fails to
    render falls back to the built-in layout rather than failing the request."""
    if template:
        try:
            return _compiled_template(template).render(messages=[dict(m) for m in messages], add_generation_prompt=True,
                                                       bos_token=bos_token, eos_token=eos_token, tools=tools, **kwargs)
        except Exception:      # noqa: BLE001 - template errors (undefined names, raise_exception) must not take a request down
            pass
    return "".join(f"<|{m.get('role', 'user')}|>\n{m.get('content', '')}\n" for m in messages) + "<|assistant|>\n"


_TEMPLATES: dict[str, object] = {}


def _compiled_template(template: str):
    t = _TEMPLATES.get(template)
    if t is None:
        from jinja2.sandbox import ImmutableSandboxedEnvironment

        def raise_exception(msg):
            raise ValueError(msg)
        env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)
        env.globals["raise_exception"] = raise_exception
        env.globals["strftime_now"] = lambda fmt: time.strftime(fmt)
        t = _TEMPLATES[template] = env.from_string(template)
    return t


@dataclass
class SamplingParams:
    max_tokens: int = 128
    temperature: float = 0.0
    top_p: float = 1.0
    top_k: int = 0
    stop: tuple[str, ...] = ()
    seed: int | None = None

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 or self.top_k == 1


@dataclass
class SpeculationConfig:
    """Low-batch speculative decoding by n-gram lookup in the sequence's own tokens (prompt-lookup drafting): when at
    most ``max_batch`` sequences are decoding, a greedy request whose last ``ngram`` tokens occurred before proposes the
    up to ``draft`` tokens that followed them; one forward over last token + draft verifies all of them and yields one
    more token, the rejected tail is cut from the KV cache.  The output is exactly the greedy output.  The lever the
    gateway's throughput report calls ``lowBatchSpeculativeDecoding`` (inference/gym/throughput.ts:49-55, 114-135:
    ``enabled_below_batch``, ``maxBatchSize`` 4, mode ``n_gram``)."""
    mode: str = "n_gram"
    max_batch: int = 4
    ngram: int = 3
    draft: int = 4
    min_ngram: int = 2


def ngram_draft(context: list[int], ngram: int, draft: int, min_ngram: int = 2) -> list[int]:
    """The tokens that followed the most recent earlier occurrence of the context's last n tokens (longest n first)."""
    L = len(context)
    for n in range(min(ngram, L - 1), min_ngram - 1, -1):
        tail = context[L - n:]
        for start in range(L - n - 1, -1, -1):
            if context[start: start + n] == tail:
                out = context[start + n: start + n + draft]
                if out:
                    return out
    return []


@dataclass
class Request:
    request_id: str
    prompt: list[int]
    params: SamplingParams
    seq_id: int = -1
    spec_proposed: int = 0            # speculated tokens offered to the verifier / accepted by it, for this request
    spec_accepted: int = 0
    state: str = "waiting"            # waiting | prefill | running | finished
    prefilled: int = 0
    cached_prompt_tokens: int = 0
    output: list[int] = field(default_factory=list)
    finish_reason: str | None = None  # stop | length | error | cancelled
    error: Exception | None = None    # what ended the request when finish_reason is "error"
    next_token: int | None = None
    t_arrival: float = 0.0
    t_first_token: float | None = None
    t_done: float | None = None
    keep_sequence: bool = False       # session turns keep their KV for the next turn
    history: list[int] = field(default_factory=list)   # tokens the sequence already holds (a continued session)
    opened: bool = False              # this request opened its sequence (and closes it if it fails)
    gen: torch.Generator | None = None
    on_token: object = None           # callback(token_id) for streaming (called from the scheduling thread)
    on_done: object = None            # callback(request) when the request finishes, whatever the reason

    @property
    def ttft_s(self):
        return None if self.t_first_token is None else self.t_first_token - self.t_arrival

    def uniform(self) -> float:
        """The random number the sampler uses for this request's next token (seeded requests repeat)."""
        return float(torch.rand(1, generator=self.gen).item())


class RequestRejected(ValueError):
    """A request that can never run on this server (longer than the context window, empty, ...)."""


class Scheduler:
    """Continuous batching over one backend.  ``step()`` admits waiting requests while sequence slots are free,
    prefills their prompts in chunks (several requests share one forward call, up to ``prefill_chunk`` tokens), then
    runs ONE decode step for every running sequence.  A request that fails (out of KV pages, a backend error) is
    finished with ``finish_reason = "error"`` and leaves the queues, so it can never block the requests behind it.

    The object is not thread-safe: one thread calls ``submit`` / ``step`` at a time (the server serialises them with
    a lock and runs ``step`` on its scheduling thread)."""

    def __init__(self, backend: Backend, tokenizer, max_num_seqs: int = 64, prefill_chunk: int = 2048,
                 now=time.perf_counter, speculation: SpeculationConfig | None = None):
        self.backend, self.tok, self.max_num_seqs, self.prefill_chunk, self.now = backend, tokenizer, max_num_seqs, prefill_chunk, now
        self.speculation = speculation if (speculation and speculation.mode == "n_gram" and getattr(backend, "supports_verify", False)) else None
        self.waiting: list[Request] = []
        self.running: list[Request] = []
        self._seq_ids = itertools.count(1)
        self._req_ids = itertools.count(1)
        self.stats = {"requests": 0, "prompt_tokens": 0, "completion_tokens": 0, "cached_prompt_tokens": 0, "steps": 0,
                      "batch_size_sum": 0, "prefill_calls": 0, "prefill_seqs_sum": 0, "errors": 0, "rejected": 0,
                      "d2h_bytes": 0, "spec_steps": 0, "spec_drafted": 0, "spec_accepted": 0}

    @property
    def speculation_acceptance_rate(self) -> float | None:
        d = self.stats["spec_drafted"]
        return self.stats["spec_accepted"] / d if d else None

    @property
    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def submit(self, prompt: list[int], params: SamplingParams, seq_id: int | None = None, keep_sequence: bool = False,
               on_token=None, on_done=None, history: list[int] | None = None) -> Request:
        """``seq_id`` continues an existing sequence (a session turn): only the new tokens are run; ``history`` are the
        tokens that sequence already holds (needed to publish its pages to the prefix cache under the right keys)."""
        held = len(history) if history is not None else 0
        limit = getattr(self.backend, "max_context", None)
        if not prompt:
            self.stats["rejected"] += 1
            raise RequestRejected("the prompt is empty")
        if limit is not None and held + len(prompt) + max(1, params.max_tokens) > limit:
            self.stats["rejected"] += 1
            raise RequestRejected(f"prompt of {held + len(prompt)} tokens plus max_tokens {params.max_tokens} exceeds the "
                                  f"context window of {limit} tokens")
        r = Request(f"req-{next(self._req_ids)}", list(prompt), params, t_arrival=self.now(), keep_sequence=keep_sequence,
                    on_token=on_token, on_done=on_done, history=list(history or []))
        if params.seed is not None:
            r.gen = torch.Generator().manual_seed(params.seed)
        if seq_id is not None:
            r.seq_id, r.state = seq_id, "prefill"
        self.waiting.append(r)
        self.stats["requests"] += 1
        self.stats["prompt_tokens"] += len(r.prompt)
        return r

    def cancel(self, r: Request):
        """Drop a request (client went away); its sequence is closed unless a session keeps it."""
        if r.state != "finished":
            self._finish(r, "cancelled")

    def _finish(self, r: Request, reason: str, error: Exception | None = None):
        r.finish_reason, r.state, r.t_done, r.error = reason, "finished", self.now(), error
        if r in self.running:
            self.running.remove(r)
        if r in self.waiting:
            self.waiting.remove(r)
        self.stats["completion_tokens"] += len(r.output)
        if error is not None:
            self.stats["errors"] += 1
        # a failed or cancelled request gives its sequence back even inside a session: what the pages hold is unknown
        if r.seq_id >= 0 and (not r.keep_sequence or (reason in ("error", "cancelled") and r.opened)):
            try:
                self.backend.end(r.seq_id)
            except Exception:       # noqa: BLE001 - closing must not raise out of the scheduling loop
                pass
        if r.on_done:
            try:
                r.on_done(r)
            except Exception:       # noqa: BLE001 - a waiter's callback must not stop the scheduling loop
                pass

    def fail_all(self, error: Exception):
        """Finish every queued and running request with ``error``: the last resort of the thread that calls ``step`` when a step
        raised, so that no caller waits for ever on a request that a broken step left behind."""
        for r in list(self.running) + list(self.waiting):
            if r.state != "finished":
                self._finish(r, "error", error)

    def _accept(self, r: Request, tok: int):
        """Take one sampled token for ``r``.  Whatever goes wrong with this one request (its streaming callback, decoding its
        text for the stop strings) ends this request with an error and leaves the others, and the scheduling thread, alone."""
        try:
            self._accept_token(r, tok)
        except Exception as e:      # noqa: BLE001
            if r.state != "finished":
                self._finish(r, "error", e)

    def _accept_token(self, r: Request, tok: int):
        if r.t_first_token is None:
            r.t_first_token = self.now()
        if tok == self.tok.eos_id:
            return self._finish(r, "stop")
        r.output.append(tok)
        r.next_token = tok
        if r.on_token:
            r.on_token(tok)
        if r.params.stop:
            text = self.tok.decode(r.output)
            if any(s and s in text for s in r.params.stop):
                return self._finish(r, "stop")
        if len(r.output) >= r.params.max_tokens:
            return self._finish(r, "length")

    def _sample_batch(self, reqs: list[Request], seq_ids, new_tokens) -> list[int] | None:
        """One backend call for ``reqs`` and one sampled token per request; on a backend error the requests are retried
        one by one so that only the ones that really fail are finished with an error.  Returns ``None`` when every
        request of the batch has been dealt with that way."""
        try:
            toks = self.backend.step(seq_ids, new_tokens, [r.params for r in reqs], [r.uniform() if not r.params.greedy else 0.0 for r in reqs])
            self.stats["d2h_bytes"] += getattr(self.backend, "last_d2h_bytes", 0)
            return toks
        except Exception as e:       # noqa: BLE001 - any backend failure is turned into per-request errors
            if len(reqs) == 1:
                self._finish(reqs[0], "error", e)
                return None
            for r, s, t in zip(reqs, seq_ids, new_tokens):
                one = self._sample_batch([r], [s], [t])
                if one is not None:
                    self._after_forward(r, len(t), one[0])
            return None

    def _after_forward(self, r: Request, n_fed: int, tok: int):
        """Book ``n_fed`` tokens just run for ``r`` and, if that completed what it had to feed, take the sampled token."""
        if r.state == "running":
            return self._accept(r, tok)
        r.prefilled += n_fed
        if r.prefilled == len(r.prompt):
            if r in self.waiting:
                self.waiting.remove(r)
            r.state = "running"
            self.running.append(r)
            try:
                self.backend.publish(r.seq_id, r.history + r.prompt)
            except Exception:      # noqa: BLE001 - the prefix index is an optimisation
                pass
            self._accept(r, tok)
        else:
            r.state = "prefill"

    def step(self) -> int:
        """One scheduling step: admit + prefill chunks, then one decode step.  Returns the number
        of sequences that made progress."""
        progressed = 0
        # ---- admission and (chunked) prefill: several requests share the token budget of one forward call
        budget = self.prefill_chunk
        batch: list[tuple[Request, int]] = []
        slots = self.max_num_seqs - len(self.running)
        for r in list(self.waiting):
            if budget <= 0 or len(batch) >= slots:
                break
            if r.seq_id < 0:
                try:
                    r.seq_id = next(self._seq_ids)
                    r.cached_prompt_tokens = self.backend.begin(r.seq_id, r.prompt)
                    r.opened = True
                except Exception as e:      # noqa: BLE001
                    r.seq_id = -1
                    self._finish(r, "error", e)
                    continue
                r.prefilled = r.cached_prompt_tokens
                self.stats["cached_prompt_tokens"] += r.cached_prompt_tokens
            n = min(budget, len(r.prompt) - r.prefilled)
            batch.append((r, n))
            budget -= n
        if batch:
            reqs = [r for r, _ in batch]
            feeds = [r.prompt[r.prefilled: r.prefilled + n] for r, n in batch]
            toks = self._sample_batch(reqs, [r.seq_id for r in reqs], feeds)
            self.stats["prefill_calls"] += 1
            self.stats["prefill_seqs_sum"] += len(batch)
            if toks is not None:
                for (r, n), tok in zip(batch, toks):
                    self._after_forward(r, n, tok)
            progressed += len(batch)
        # ---- one decode step for everyone who has a token to feed
        dec = [r for r in self.running if r.next_token is not None]
        if dec and self.speculation is not None and len(dec) <= self.speculation.max_batch:
            rest = []
            for r in dec:
                if r.params.greedy and self._speculate(r):
                    progressed += 1
                else:
                    rest.append(r)
            dec = rest
        if dec:
            toks = self._sample_batch(dec, [r.seq_id for r in dec], [[r.next_token] for r in dec])
            self.stats["steps"] += 1
            self.stats["batch_size_sum"] += len(dec)
            if toks is not None:
                for r, tok in zip(dec, toks):
                    self._accept(r, tok)
            progressed += len(dec)
        return progressed

    def _speculate(self, r: Request) -> bool:
        """Draft, verify and accept for one greedy request; False when there was nothing to draft (the request then takes
        the normal decode step).  On a backend error the request is finished with that error, like in any other step."""
        sp, be = self.speculation, self.backend
        room = r.params.max_tokens - len(r.output) - 1            # drafts we could still emit before the bonus token
        limit = getattr(be, "max_context", None)
        try:
            base = be.seq_len(r.seq_id)
        except Exception:      # noqa: BLE001
            return False
        if limit is not None:
            room = min(room, limit - base - 2)
        if room < 1:
            return False
        draft = ngram_draft(r.history + r.prompt + r.output, sp.ngram, min(sp.draft, room), sp.min_ngram)
        if not draft:
            return False
        try:
            preds = be.verify(r.seq_id, [r.next_token] + draft)
            self.stats["d2h_bytes"] += getattr(be, "last_d2h_bytes", 0)
        except Exception as e:      # noqa: BLE001
            self._finish(r, "error", e)
            return True
        k = len(draft)
        n_acc = 0
        while n_acc < k and draft[n_acc] == preds[n_acc]:
            n_acc += 1
        self.stats["spec_steps"] += 1
        self.stats["spec_drafted"] += k
        self.stats["spec_accepted"] += n_acc
        r.spec_proposed += k
        r.spec_accepted += n_acc
        self.stats["steps"] += 1
        self.stats["batch_size_sum"] += 1
        i_last = n_acc
        for i, tok in enumerate(draft[:n_acc] + [preds[n_acc]]):
            self._accept(r, tok)
            if r.state == "finished":
                i_last = i
                break
        keep = base + 1 + i_last                  # the fed token plus the accepted tokens whose successors were used
        if keep < base + 1 + k and (r.state != "finished" or (r.keep_sequence and r.finish_reason not in ("error", "cancelled"))):
            try:
                be.truncate(r.seq_id, keep)
            except Exception as e:      # noqa: BLE001
                if r.state != "finished":
                    self._finish(r, "error", e)
        return True

    def run_until_done(self, reqs: list[Request], max_steps: int = 1_000_000):
        for _ in range(max_steps):
            if all(r.state == "finished" for r in reqs):
                return
            self.step()
        raise RuntimeError("scheduler did not finish")
