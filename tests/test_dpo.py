"""Preference batches and the row factors of the DPO objective against autograd and the reference's pair loss."""
import pytest
import torch
import torch.nn.functional as F

from openagents_b200.data import ByteBpe
from openagents_b200.oracle.cs336 import dpo_pair_loss
from openagents_b200.train import dpo, sft

PAIRS = [{"messages": [{"role": "user", "content": "Is water wet?"}], "chosen": "Yes, it is.", "rejected": "No."},
         {"messages": [{"role": "user", "content": "Name a fruit."}, {"role": "assistant", "content": "Apple."}, {"role": "user", "content": "Another."}],
          "chosen": "Pear.", "rejected": "Granite is a rock."}]


def _tok():
    return ByteBpe.train(b"Is water wet? Yes, it is. No. Name a fruit. Apple. Another. Pear. Granite is a rock.", 12, special=sft.SPECIAL_TOKENS)


def test_batch_layout_masks_prompt_earlier_turns_and_padding():
    tok = _tok()
    tokens, targets, counts = dpo.build_preference_batch(PAIRS, tok, seq_len=64)
    assert tokens.shape == targets.shape == (4, 64)
    for r, (pair, key) in enumerate([(PAIRS[0], "chosen"), (PAIRS[1], "chosen"), (PAIRS[0], "rejected"), (PAIRS[1], "rejected")]):
        kept = [int(t) for t in targets[r] if t >= 0]
        assert tok.decode(kept) == pair[key] + "<|end|>" and counts[r] == len(kept)
        first = int((targets[r] >= 0).nonzero()[0])
        assert int(tokens[r, first + 1]) == kept[0]                # targets are the inputs shifted by one
    assert "Apple" not in tok.decode([int(t) for t in targets[1] if t >= 0])     # the earlier assistant turn is prompt
    with pytest.raises(ValueError):
        dpo.build_preference_batch(PAIRS, tok, seq_len=8)


def test_row_factors_are_the_gradient_of_the_pair_loss():
    torch.manual_seed(0)
    B, T, V, beta = 4, 6, 11, 0.3
    logits = torch.randn(B * T, V, dtype=torch.float64, requires_grad=True)
    targets = torch.randint(0, V, (B, T))
    targets[:, :2] = -1
    ref = torch.randn(B, dtype=torch.float64)
    nll = F.cross_entropy(logits, targets.reshape(-1), ignore_index=-1, reduction="none")
    pol = -nll.view(B, T).sum(1)
    want = sum(dpo_pair_loss(beta, float(pol[i].detach()), float(pol[2 + i].detach()), float(ref[i]), float(ref[2 + i])) for i in range(2)) / 2
    stats = {}
    scale, loss = dpo.dpo_row_scales(nll.detach(), ref, beta, pairs_in_step=2, stats=stats)
    assert float(loss) == pytest.approx(want, rel=1e-9)
    # what the fused kernel writes: factor * (softmax - onehot) on unmasked rows
    t = targets.reshape(-1)
    onehot = F.one_hot(t.clamp(min=0), V).double()
    mine = scale.double().unsqueeze(1) * (torch.softmax(logits.detach(), -1) - onehot) * (t >= 0).unsqueeze(1)
    full = (F.softplus(-beta * ((pol[:2] - ref[:2]) - (pol[2:] - ref[2:])))).mean()
    full.backward()
    assert torch.allclose(mine, logits.grad, atol=1e-7)
    assert 0.0 <= float(stats["rewardAccuracy"]) <= 1.0 and stats["margins"].shape == (2,)
