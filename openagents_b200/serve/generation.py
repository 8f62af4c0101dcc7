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


def render_chat(messages: list[dict]) -> str:
    return "".join(f"<|{m.get('role', 'user')}|>\n{m.get('content', '')}\n" for m in messages) + "<|assistant|>\n"


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


def sample(logits: torch.Tensor, p: SamplingParams, gen: torch.Generator | None) -> int:
    """One token from a [V] logits row (host-side; the engine's device sampler serves the
    graph-replayed greedy loop)."""
    if p.greedy:
        return int(torch.argmax(logits))
    x = logits.float() / max(p.temperature, 1e-6)
    k = p.top_k if p.top_k > 0 else min(64, x.numel())
    vals, idx = torch.topk(x, min(k, x.numel()))
    probs = torch.softmax(vals, dim=-1)
    if p.top_p < 1.0:
        keep = int((torch.cumsum(probs, 0) < p.top_p).sum().item()) + 1
        probs, idx = probs[:keep] / probs[:keep].sum(), idx[:keep]
    return int(idx[torch.multinomial(probs, 1, generator=gen)])


@dataclass
class Request:
    request_id: str
    prompt: list[int]
    params: SamplingParams
    seq_id: int = -1
    state: str = "waiting"            # waiting | prefill | running | finished
    prefilled: int = 0
    cached_prompt_tokens: int = 0
    output: list[int] = field(default_factory=list)
    finish_reason: str | None = None
    next_token: int | None = None
    t_arrival: float = 0.0
    t_first_token: float | None = None
    t_done: float | None = None
    keep_sequence: bool = False       # session turns keep their KV for the next turn
    gen: torch.Generator | None = None
    on_token: object = None           # callback(token_id) for streaming

    @property
    def ttft_s(self):
        return None if self.t_first_token is None else self.t_first_token - self.t_arrival


class Scheduler:
    def __init__(self, backend: Backend, tokenizer, max_num_seqs: int = 64, prefill_chunk: int = 2048,
                 now=time.perf_counter):
        self.backend, self.tok, self.max_num_seqs, self.prefill_chunk, self.now = backend, tokenizer, max_num_seqs, prefill_chunk, now
        self.waiting: list[Request] = []
        self.running: list[Request] = []
        self._seq_ids = itertools.count(1)
        self._req_ids = itertools.count(1)
        self.stats = {"requests": 0, "prompt_tokens": 0, "completion_tokens": 0, "cached_prompt_tokens": 0, "steps": 0,
                      "batch_size_sum": 0}

    def submit(self, prompt: list[int], params: SamplingParams, seq_id: int | None = None, keep_sequence: bool = False,
               on_token=None) -> Request:
        """``seq_id`` continues an existing sequence (a session turn): only the new tokens are run."""
        r = Request(f"req-{next(self._req_ids)}", list(prompt), params, t_arrival=self.now(), keep_sequence=keep_sequence,
                    on_token=on_token)
        if params.seed is not None:
            r.gen = torch.Generator().manual_seed(params.seed)
        if seq_id is not None:
            r.seq_id, r.state = seq_id, "prefill"
        self.waiting.append(r)
        self.stats["requests"] += 1
        self.stats["prompt_tokens"] += len(r.prompt)
        return r

    def _finish(self, r: Request, reason: str):
        r.finish_reason, r.state, r.t_done = reason, "finished", self.now()
        if r in self.running:
            self.running.remove(r)
        self.stats["completion_tokens"] += len(r.output)
        if not r.keep_sequence:
            self.backend.end(r.seq_id)

    def _accept(self, r: Request, logits_row: torch.Tensor):
        tok = sample(logits_row, r.params, r.gen)
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

    def step(self) -> int:
        """One scheduling step: admit + prefill chunks, then one decode step.  Returns the number
        of sequences that made progress."""
        progressed = 0
        # ---- admission and (chunked) prefill
        budget = self.prefill_chunk
        while self.waiting and len(self.running) < self.max_num_seqs and budget > 0:
            r = self.waiting[0]
            if r.seq_id < 0:
                r.seq_id = next(self._seq_ids)
                r.cached_prompt_tokens = self.backend.begin(r.seq_id, r.prompt)
                r.prefilled = r.cached_prompt_tokens
                self.stats["cached_prompt_tokens"] += r.cached_prompt_tokens
            n = min(budget, len(r.prompt) - r.prefilled)
            logits = self.backend.forward([r.seq_id], [r.prompt[r.prefilled: r.prefilled + n]])
            r.prefilled += n
            budget -= n
            progressed += 1
            if r.prefilled == len(r.prompt):
                self.waiting.pop(0)
                r.state = "running"
                self.running.append(r)
                self.backend.publish(r.seq_id, r.prompt)
                self._accept(r, logits[0])
            else:
                r.state = "prefill"
                break
        # ---- one decode step for everyone who has a token to feed
        batch = [r for r in self.running if r.next_token is not None]
        if batch:
            logits = self.backend.forward([r.seq_id for r in batch], [[r.next_token] for r in batch])
            self.stats["steps"] += 1
            self.stats["batch_size_sum"] += len(batch)
            for i, r in enumerate(batch):
                self._accept(r, logits[i])
            progressed += len(batch)
        return progressed

    def run_until_done(self, reqs: list[Request], max_steps: int = 1_000_000):
        for _ in range(max_steps):
            if all(r.state == "finished" for r in reqs):
                return
            self.step()
        raise RuntimeError("scheduler did not finish")
