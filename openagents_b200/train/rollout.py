"""Roll-outs with graded rewards and a group-relative policy-gradient step on the trainer.

The reference's A5 workload samples several roll-outs per task, grades each against the task's exact answer and summarises
rewards per task (apps/openagents.com/workers/api/src/cs336-a5-rollout-workload.ts:222 batch, :334 grading; restated in
``oracle.cs336_more``); its post-training receipt lists preference/roll-out work as the step after instruction tuning.
Here the roll-outs come from the weights being trained:

* sampling: ``serve.gpt2_backend.Gpt2CudaBackend.over_trainer`` serves the trainer's own parameter buffer through the
  ordinary scheduler (continuous batching, temperature / top-k sampling, seeds), ``group_size`` completions per prompt;
* grading: any ``reward_fn(task, completion_text, completion_ids) -> float`` (``exact_answer_reward`` grades the final
  integer of a completion the way the reference's grader does);
* advantages: reward minus the group mean, divided by the group's standard deviation (groups whose roll-outs all got
  the same reward carry no signal and are skipped);
* update: the completions become rows of a masked batch (prompt masked, completion trainable) and every row gets the
  factor ``advantage / (completion tokens x rows in the step)``; the fused cross-entropy then writes
  ``factor x (softmax - onehot)``, the gradient of ``-advantage x mean log-probability``, and the usual backward and
  optimizer step follow (the same per-row mechanism the preference lane uses).
"""
from __future__ import annotations

import math

import torch

from ..oracle.cs336_more import parse_final_value


def exact_answer_reward(task: dict, text: str, ids) -> float:
    """1.0 when the completion's last ``#### <integer>`` line equals ``task["answer"]`` (the reference grader's format), else 0.0."""
    return 1.0 if parse_final_value(text) == task.get("answer") else 0.0


def group_advantages(rewards: list[float], eps: float = 1e-6) -> list[float] | None:
    """Standardised within the group; None when every roll-out got the same reward."""
    mean = sum(rewards) / len(rewards)
    var = sum((r - mean) ** 2 for r in rewards) / len(rewards)
    if var <= eps * eps:
        return None
    sd = math.sqrt(var)
    return [(r - mean) / (sd + eps) for r in rewards]


def build_rollout_batch(samples, seq_len: int, rows: int, pad_id: int = 0):
    """``samples``: ``(prompt_ids, completion_ids, advantage)``.  Returns ``tokens`` / ``targets`` ``[accum, rows, seq_len]`` (int64),
    per-row factors ``[accum, rows * seq_len]`` (float32) and the number of rows that carry signal; rows beyond the samples are
    padding with every target masked."""
    n = len(samples)
    accum = max(1, -(-n // rows))
    tokens = torch.full((accum * rows, seq_len), pad_id, dtype=torch.int64)
    targets = torch.full((accum * rows, seq_len), -1, dtype=torch.int64)
    factors = torch.zeros((accum * rows, seq_len), dtype=torch.float32)
    for r, (prompt, completion, adv) in enumerate(samples):
        ids = list(prompt) + list(completion)
        if len(ids) > seq_len + 1 or not completion:
            raise ValueError("a roll-out does not fit the window or is empty")
        m = len(ids) - 1
        tokens[r, :m] = torch.tensor(ids[:-1])
        lo = len(prompt) - 1                                     # the position whose target is the first completion token
        targets[r, lo:m] = torch.tensor(ids[len(prompt):])
        factors[r, lo:m] = adv / (len(completion) * n)
    return (tokens.view(accum, rows, seq_len), targets.view(accum, rows, seq_len), factors.view(accum, rows * seq_len), n)


class RolloutTrainer:
    def __init__(self, trainer, tokenizer, reward_fn=exact_answer_reward, group_size: int = 4, max_new_tokens: int = 16,
                 temperature: float = 1.0, top_k: int = 64, seed: int = 0):
        from ..serve.generation import Scheduler
        from ..serve.gpt2_backend import Gpt2CudaBackend
        self.trainer, self.tok, self.reward_fn = trainer, tokenizer, reward_fn
        self.group_size, self.max_new, self.temperature, self.top_k, self.seed = group_size, max_new_tokens, temperature, top_k, seed
        self.backend = Gpt2CudaBackend.over_trainer(trainer)
        self.scheduler = Scheduler(self.backend, tokenizer, max_num_seqs=self.backend.rows)
        self.steps = 0

    def sample(self, tasks) -> list[dict]:
        """``tasks``: ``{"prompt": str, ...}``.  One record per task: its prompt ids, ``group_size`` completions, their rewards."""
        from ..serve.generation import SamplingParams
        reqs = []
        for t_i, task in enumerate(tasks):
            prompt = self.tok.encode(task["prompt"])
            for k in range(self.group_size):
                p = SamplingParams(max_tokens=self.max_new, temperature=self.temperature, top_k=self.top_k,
                                   seed=(self.seed * 1_000_003 + self.steps * 10_007 + t_i * 101 + k) & 0x7FFFFFFF)
                reqs.append((t_i, prompt, self.scheduler.submit(prompt, p)))
        self.scheduler.run_until_done([r for _, _, r in reqs])
        out = [{"task": t, "prompt": None, "completions": [], "rewards": []} for t in tasks]
        for t_i, prompt, r in reqs:
            ids = [i for i in r.output if i != getattr(self.tok, "eos_id", None)] or list(r.output)
            out[t_i]["prompt"] = prompt
            out[t_i]["completions"].append(ids)
            out[t_i]["rewards"].append(float(self.reward_fn(tasks[t_i], self.tok.decode(ids), ids)))
        return out

    def step(self, tasks) -> dict:
        """Sample, grade, and take one optimizer step on the groups that carry signal."""
        tr = self.trainer
        groups = self.sample(tasks)
        samples = []
        for g in groups:
            adv = group_advantages(g["rewards"])
            if adv is None:
                continue
            samples += [(g["prompt"], c, a) for c, a in zip(g["completions"], adv) if c]
        rewards = [r for g in groups for r in g["rewards"]]
        rec = {"step": self.steps, "tasks": len(tasks), "rollouts": len(rewards), "meanReward": sum(rewards) / max(1, len(rewards)),
               "groupsWithSignal": sum(group_advantages(g["rewards"]) is not None for g in groups), "trainedRows": len(samples), "objective": None}
        self.steps += 1
        if not samples:
            return rec
        tokens, targets, factors, _ = build_rollout_batch(samples, tr.cfg.seq_len, tr.cfg.micro_batch)
        dev = tr.device
        tokens, targets, factors = (x.pin_memory().to(dev, non_blocking=True) for x in (tokens, targets, factors))
        accum_needed = tokens.shape[0]
        if accum_needed != tr.accum:
            # the trainer accumulates a fixed number of micro-batches per step: pad with empty ones or split into several steps
            if accum_needed > tr.accum:
                raise ValueError(f"{len(samples)} roll-outs need {accum_needed} micro-batches, the trainer accumulates {tr.accum}")
            pad = tr.accum - accum_needed
            tokens = torch.cat([tokens, tokens.new_zeros((pad, *tokens.shape[1:]))])
            targets = torch.cat([targets, targets.new_full((pad, *targets.shape[1:]), -1)])
            factors = torch.cat([factors, factors.new_zeros((pad, factors.shape[1]))])
        fns = [(lambda rows, a=a: (factors[a], (rows * factors[a]).sum())) for a in range(tr.accum)]
        rec["objective"] = float(tr.train_step(tokens, targets, row_scale_fns=fns).item())
        return rec
