"""Group advantages and the roll-out batch layout (the policy-gradient step itself runs on the GPU trainer)."""
import pytest
import torch

from openagents_b200.train.rollout import build_rollout_batch, exact_answer_reward, group_advantages


def test_group_advantages_standardise_and_skip_flat_groups():
    a = group_advantages([1.0, 0.0, 0.0, 1.0])
    assert a == pytest.approx([1.0, -1.0, -1.0, 1.0], abs=1e-4) and abs(sum(a)) < 1e-9
    assert group_advantages([1.0, 1.0, 1.0]) is None and group_advantages([0.0] * 4) is None
    b = group_advantages([0.0, 0.0, 0.0, 1.0])
    assert b[3] > 0 > b[0] and b[0] == b[1] == b[2]


def test_batch_rows_mask_the_prompt_and_carry_the_factor():
    samples = [([5, 6, 7], [8, 9], 1.5), ([5, 6, 7], [10], -0.5), ([1], [2, 3, 4], 2.0)]
    tok, tgt, fac, n = build_rollout_batch(samples, seq_len=8, rows=2)
    assert tok.shape == tgt.shape == (2, 2, 8) and fac.shape == (2, 16) and n == 3
    assert tok[0, 0, :4].tolist() == [5, 6, 7, 8] and tgt[0, 0].tolist() == [-1, -1, 8, 9, -1, -1, -1, -1]
    assert fac[0, :8].tolist() == pytest.approx([0, 0, 1.5 / 6, 1.5 / 6, 0, 0, 0, 0])
    assert tgt[0, 1].tolist() == [-1, -1, 10, -1, -1, -1, -1, -1] and fac[0, 8 + 2].item() == pytest.approx(-0.5 / 3)
    assert tgt[1, 0].tolist() == [2, 3, 4, -1, -1, -1, -1, -1] and bool((tgt[1, 1] == -1).all())      # the fourth row is padding
    # the factors are the gradient weights of  -sum_i A_i * mean_t log p  / n
    logits = torch.randn(2 * 2 * 8, 12, dtype=torch.float64, requires_grad=True)
    nll = torch.nn.functional.cross_entropy(logits, tgt.reshape(-1), ignore_index=-1, reduction="none")
    (nll * fac.reshape(-1).double()).sum().backward()
    logits2 = logits.detach().clone().requires_grad_(True)
    nll2 = torch.nn.functional.cross_entropy(logits2, tgt.reshape(-1), ignore_index=-1, reduction="none").view(4, 8)
    (-(1.5 * (-nll2[0, 2:4]).mean() - 0.5 * (-nll2[1, 2]) + 2.0 * (-nll2[2, 0:3]).mean()) / 3).backward()
    assert torch.allclose(logits.grad, logits2.grad, atol=1e-9)
    with pytest.raises(ValueError):
        build_rollout_batch([([1] * 9, [2], 1.0)], seq_len=8, rows=2)


def test_exact_answer_reward_reads_the_final_integer():
    assert exact_answer_reward({"answer": 42}, "6 times 7\n#### 42", []) == 1.0          # the grader reads the "#### <integer>" line
    assert exact_answer_reward({"answer": 42}, "#### 41\n#### 43", []) == 0.0
    assert exact_answer_reward({"answer": 42}, "so the total is 42", []) == 0.0
