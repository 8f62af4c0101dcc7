"""GPT-2-shape checkpoints through the serving interface (fp32 oracle backend), the backend factory and the tokenizer that
travels inside the file."""
import pytest
import torch

from openagents_b200.data import ByteBpe
from openagents_b200.eval import multiple_choice
from openagents_b200.models.config import GPT2_SMALL
from openagents_b200.models.weights import PLAN_BF16, random_weights, save_gguf
from openagents_b200.oracle.models import gpt2_forward
from openagents_b200.serve.backend import open_backend
from openagents_b200.serve.generation import SamplingParams, Scheduler
from openagents_b200.serve.server import load_tokenizer

CFG = GPT2_SMALL.with_(n_layers=2, d_model=64, n_heads=2, n_kv_heads=2, head_dim=32, ffn=128, vocab=320, context=64)


@pytest.fixture(scope="module")
def gguf(tmp_path_factory):
    p = str(tmp_path_factory.mktemp("g") / "gpt2.gguf")
    tok = ByteBpe.train(b"the cat sat on the mat " * 8, 20, special=["<|user|>", "<|assistant|>", "<|system|>", "<|end|>"])
    save_gguf(p, CFG, random_weights(CFG, 1), PLAN_BF16, extra_meta={"tokenizer.b200.byte_bpe": tok.to_json()})
    return p, tok


def test_factory_picks_the_gpt2_backend_and_matches_the_oracle(gguf):
    path, _ = gguf
    be = open_backend(path, "cpu")
    assert type(be).__name__ == "Gpt2CpuBackend" and be.max_context == 64
    toks = [5, 9, 200, 31, 7]
    want = gpt2_forward(CFG, be.W, torch.tensor(toks)[None])[0]
    be.begin(1, toks)
    assert torch.allclose(be.forward([1], [toks[:3]])[0], want[2], atol=1e-5)
    assert be.verify(1, toks[3:]) == want[3:].argmax(-1).tolist() and be.seq_len(1) == 5
    be.truncate(1, 3)
    lp = be.score(1, toks[3:], [4, -1])
    assert lp[0] == pytest.approx(float(torch.log_softmax(want[3].double(), -1)[4]), abs=1e-5) and lp[1] == 0.0
    be.end(1)
    with pytest.raises(ValueError, match="context"):
        be.begin(2, [])
        be.forward([2], [[1] * 65])


def test_tokenizer_travels_in_the_file_and_the_scheduler_runs(gguf):
    path, tok = gguf
    loaded, tpl = load_tokenizer(path, CFG.vocab)
    assert type(loaded).__name__ == "ByteBpeTokenizer" and tpl is None
    text = "the cat<|end|>"
    assert loaded.encode(text) == tok.encode(text) and loaded.decode(loaded.encode(text)) == text
    assert loaded.eos_id == tok.special_ids["<|end|>"]
    be = open_backend(path, "cpu")
    sch = Scheduler(be, loaded, max_num_seqs=2)
    r = sch.submit(loaded.encode("the cat sat"), SamplingParams(max_tokens=5))
    sch.run_until_done([r])
    assert 1 <= len(r.output) <= 5 and be.kv_stats()["sequences"] == 0
    res = multiple_choice(be, [{"context": "the cat", "choices": [" sat", " mat on"], "answer": 0}], loaded)
    assert res["items"] == 1
