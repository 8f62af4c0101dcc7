"""End-to-end engine checks on a GPU against the CPU oracle."""
import pytest
import torch

from openagents_b200.models.config import TINY_LLAMA
from openagents_b200.models.weights import PLAN_Q4_K, PLAN_Q8_0, load_gguf_float, random_weights, save_gguf
from openagents_b200.oracle.models import KVCacheRef, greedy_generate, llama_forward

pytestmark = pytest.mark.gpu


def _engine(path, **kw):
    from openagents_b200.models.engine import LlamaEngine
    from openagents_b200.models.qweight import GGUFSource
    src = GGUFSource(path, "cuda")
    return LlamaEngine(src.cfg, src, max_batch=8, max_ctx=256, max_tokens=256, **kw)


def test_tiny_llama_q8_greedy_matches_oracle(tmp_path):
    """Benchmark configuration 1 on the GPU: same GGUF, same prompt, token ids equal the oracle's."""
    cfg = TINY_LLAMA
    p = str(tmp_path / "tiny.gguf")
    save_gguf(p, cfg, random_weights(cfg, 0), PLAN_Q8_0)
    cfg2, W = load_gguf_float(p)
    prompt = torch.randint(0, cfg.vocab, (32,), generator=torch.Generator().manual_seed(1))
    ref_ids, ref_logits = greedy_generate(cfg2, W, prompt, 64)
    eng = _engine(p)
    scale = ref_logits.std().item()
    for use_graph in (False, True):
        ids, logits = eng.generate(prompt.tolist(), 64, seq_id=10 + int(use_graph), use_graph=use_graph)
        eng.check_status()
        # Compare step by step while both runs have produced the same tokens.  A first difference is
        # only acceptable where the oracle's top-2 margin is inside the kernel tolerance.
        for t, (a, b) in enumerate(zip(ids, ref_ids.tolist())):
            err = (logits[t] - ref_logits[t]).abs().max().item()
            assert err < 0.05 * scale, (use_graph, t, err, scale)
            if a != b:
                top2 = ref_logits[t].topk(2).values
                assert (top2[0] - top2[1]).item() < 2 * err, (t, a, b)
                break
    eng.end(10)
    eng.end(11)


def test_q4k_paths_agree(tmp_path):
    """Mat-vec path (<= 8 tokens), dense tensor-core path and the oracle agree on a Q4_K/Q6_K model."""
    cfg = TINY_LLAMA.with_(d_model=512, n_heads=8, n_kv_heads=2, head_dim=64, ffn=1024, vocab=4096, n_layers=3)
    p = str(tmp_path / "q4k.gguf")
    save_gguf(p, cfg, random_weights(cfg, 3), PLAN_Q4_K)
    cfg2, W = load_gguf_float(p)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g) for n in (40, 17, 33)]
    eng = _engine(p)
    # prefill all three together (dense path), then decode three steps (mat-vec path)
    for b in range(3):
        eng.begin(b)
    logits, nxt = eng.forward_tokens([0, 1, 2], [x.tolist() for x in prompts])
    caches = [KVCacheRef(cfg.n_layers) for _ in range(3)]
    ref = torch.stack([llama_forward(cfg2, W, prompts[b], caches[b])[-1] for b in range(3)])
    scale = ref.std().item()
    assert (logits.cpu() - ref).abs().max().item() < 0.08 * scale
    toks = ref.argmax(-1).tolist()
    for step in range(3):
        logits, nxt = eng.decode([0, 1, 2], toks, use_graph=(step > 0))
        ref = torch.stack([llama_forward(cfg2, W, torch.tensor([toks[b]]), caches[b])[-1] for b in range(3)])
        assert (logits.cpu() - ref).abs().max().item() < 0.08 * scale, step
        toks = ref.argmax(-1).tolist()
    eng.check_status()
    # a 12-sequence decode batch goes through the dense path and must match too
    from openagents_b200.models.engine import LlamaEngine
    from openagents_b200.models.qweight import GGUFSource
    src = GGUFSource(p, "cuda")
    eng2 = LlamaEngine(src.cfg, src, max_batch=16, max_ctx=128, max_tokens=256)
    ps = [torch.randint(0, cfg.vocab, (5 + b,), generator=g) for b in range(12)]
    for b in range(12):
        eng2.begin(b)
    logits, _ = eng2.forward_tokens(list(range(12)), [x.tolist() for x in ps])
    caches = [KVCacheRef(cfg.n_layers) for _ in range(12)]
    ref = torch.stack([llama_forward(cfg2, W, ps[b], caches[b])[-1] for b in range(12)])
    assert (logits.cpu() - ref).abs().max().item() < 0.08 * scale
    toks = ref.argmax(-1).tolist()
    logits, _ = eng2.decode(list(range(12)), toks)
    ref = torch.stack([llama_forward(cfg2, W, torch.tensor([toks[b]]), caches[b])[-1] for b in range(12)])
    assert (logits.cpu() - ref).abs().max().item() < 0.08 * scale
    eng2.check_status()


def test_prefix_reuse_gives_same_logits(tmp_path):
    cfg = TINY_LLAMA.with_(vocab=1000)
    p = str(tmp_path / "t.gguf")
    save_gguf(p, cfg, random_weights(cfg, 4), PLAN_Q8_0)
    eng = _engine(p)
    prompt = torch.randint(0, 1000, (50,), generator=torch.Generator().manual_seed(5)).tolist()
    assert eng.begin(1, prompt) == 0
    l1, _ = eng.forward_tokens([1], [prompt])
    l1 = l1.clone()
    eng.pool.publish(1, prompt)
    cached = eng.begin(2, prompt)
    assert cached == 48
    l2, _ = eng.forward_tokens([2], [prompt[cached:]])
    assert torch.allclose(l1, l2, atol=2e-2 * l1.std().item())


@pytest.mark.kv_retention
def test_prefix_pages_of_a_closed_sequence_still_serve_hits(tmp_path):
    """The published pages of a sequence that has ended stay in the prefix index: the same prompt later is prefilled on top of
    them and gives the same logits (to the tolerance of a different tiling), and they are given up when the pool needs pages."""
    cfg = TINY_LLAMA.with_(vocab=1000)
    p = str(tmp_path / "t.gguf")
    save_gguf(p, cfg, random_weights(cfg, 4), PLAN_Q8_0)
    eng = _engine(p)
    prompt = torch.randint(0, 1000, (50,), generator=torch.Generator().manual_seed(5)).tolist()
    assert eng.begin(1, prompt) == 0
    l1, _ = eng.forward_tokens([1], [prompt])
    l1 = l1.clone()
    eng.pool.publish(1, prompt)
    free0 = eng.pool.free_pages
    eng.end(1)
    assert eng.pool.retained_pages == 3 and eng.pool.free_pages == free0 + 4
    cached = eng.begin(2, prompt)
    assert cached == 48 and eng.pool.retained_pages == 0
    l2, _ = eng.forward_tokens([2], [prompt[cached:]])
    assert torch.allclose(l1, l2, atol=2e-2 * l1.std().item())
    eng.end(2)
    eng.pool.set_retention(False)
    assert eng.pool.retained_pages == 0 and eng.begin(3, prompt) == 0
    eng.end(3)
    eng.check_status()


def test_device_side_decode_loop_matches_stepwise(tmp_path):
    """The self-advancing decode graph produces the same ids as one host round trip per step."""
    cfg = TINY_LLAMA.with_(vocab=2048)
    p = str(tmp_path / "t.gguf")
    save_gguf(p, cfg, random_weights(cfg, 6), PLAN_Q8_0)
    eng = _engine(p)
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, 2048, (20 + 3 * b,), generator=g).tolist() for b in range(3)]
    outs = []
    for base in (0, 10):
        ids = [base + b for b in range(3)]
        for i in ids:
            eng.begin(i)
        _, nxt = eng.forward_tokens(ids, prompts)
        first = nxt.tolist()
        if base == 0:
            toks, hist = first, []
            for _ in range(20):
                _, nxt = eng.decode(ids, toks)
                toks = nxt.tolist()
                hist.append(toks)
            outs.append(torch.tensor(hist))
        else:
            outs.append(eng.decode_steps(ids, first, 20).cpu().long())
    assert torch.equal(outs[0], outs[1])
    assert eng.pool.length(10) == len(prompts[0]) + 20


def test_backend_samples_on_the_device(tmp_path):
    """The serving backend's step: greedy rows take the engine's fused arg-max, the others the device top-k / top-p
    kernel; four bytes per sequence come back.  Sampled ids must lie in the oracle's top-k, and a seeded request repeats."""
    from openagents_b200.serve.backend import CudaBackend
    from openagents_b200.serve.generation import ByteTokenizer, SamplingParams, Scheduler
    cfg = TINY_LLAMA.with_(vocab=1000)
    p = str(tmp_path / "t.gguf")
    save_gguf(p, cfg, random_weights(cfg, 5), PLAN_Q8_0)
    cfg2, W = load_gguf_float(p)
    be = CudaBackend.from_gguf(p, max_num_seqs=8, max_ctx=256, max_tokens=256)
    prompt = list(range(20, 45))
    ref = llama_forward(cfg2, W, torch.tensor(prompt), KVCacheRef(cfg.n_layers))[-1]
    be.begin(1, prompt)
    be.begin(2, prompt)
    hot = SamplingParams(temperature=0.9, top_k=5, top_p=1.0)
    ids = be.step([1, 2], [prompt, prompt], [SamplingParams(), hot], [0.0, 0.6])
    assert be.last_d2h_bytes == 8
    assert ids[0] == int(ref.argmax()) and ids[1] in ref.topk(5).indices.tolist()
    ids2 = be.step([1, 2], [[ids[0]], [ids[1]]], [SamplingParams(), hot], [0.0, 0.1])
    assert len(ids2) == 2 and be.last_d2h_bytes == 8
    be.end(1)
    be.end(2)
    # through the scheduler: a seeded sampled request repeats token for token
    outs = []
    for _ in range(2):
        sch = Scheduler(be, ByteTokenizer(cfg.vocab), max_num_seqs=4)
        r = sch.submit(prompt, SamplingParams(max_tokens=12, temperature=0.8, top_k=8, seed=7))
        g = sch.submit(prompt[:10], SamplingParams(max_tokens=12))
        sch.run_until_done([r, g])
        assert r.finish_reason in ("length", "stop") and g.finish_reason in ("length", "stop")
        outs.append(r.output)
    assert outs[0] == outs[1] and sch.stats["d2h_bytes"] > 0
    be.engine.check_status()


def test_workspace_canaries_stay_intact(tmp_path):
    """Every engine workspace between guard zones of a known byte: after prefill at the workspace's full token count,
    mat-vec decode, batched fused-dequant decode (eager and from a graph) and the device-side decode loop, no kernel
    has written a byte outside its buffers; and a deliberate stray write on the host is reported."""
    from openagents_b200.models.engine import LlamaEngine
    from openagents_b200.models.qweight import GGUFSource
    cfg = TINY_LLAMA.with_(d_model=512, n_heads=8, n_kv_heads=2, head_dim=64, ffn=1024, vocab=4096, n_layers=2)
    p = str(tmp_path / "q4k.gguf")
    save_gguf(p, cfg, random_weights(cfg, 5), PLAN_Q4_K)
    src = GGUFSource(p, "cuda")
    eng = LlamaEngine(src.cfg, src, max_batch=16, max_ctx=256, max_tokens=192, canaries=True)
    assert len(eng._guards) > 20 and eng.check_canaries() == []
    g = torch.Generator().manual_seed(4)
    ids = list(range(12))
    for b in ids:
        eng.begin(b)
    # 12 x 16 = 192 tokens: the prefill fills the token workspaces to the last row
    _, nxt = eng.forward_tokens(ids, [torch.randint(0, cfg.vocab, (16,), generator=g).tolist() for _ in ids])
    toks = nxt.tolist()
    for step in range(3):
        _, nxt = eng.decode(ids, toks, use_graph=(step > 0))
        toks = nxt.tolist()
    eng.decode_steps(ids, toks, 4)
    _, nxt = eng.decode([0, 1], toks[:2])                 # mat-vec path
    eng.decode_steps([3], [5], 3)
    eng.check_status()
    assert eng.check_canaries() == []
    raw, nbytes = eng._guards["gu"]
    raw[eng._GUARD_BYTES + nbytes + 3] = 0                 # one byte past the end of `gu`
    raw_q, _ = eng._guards["qkv"]
    raw_q[eng._GUARD_BYTES - 1] = 7                        # one byte before the start of `qkv`
    assert sorted(eng.check_canaries()) == ["gu:after", "qkv:before"]


def test_speculative_decoding_matches_greedy_on_the_engine(tmp_path):
    """N-gram drafts verified by one multi-token forward with logits at every position, rejected tails cut from the
    paged cache: the tokens are exactly those of plain greedy decoding, also across a second turn on the same sequence."""
    from openagents_b200.serve.backend import CudaBackend
    from openagents_b200.serve.generation import ByteTokenizer, SamplingParams, Scheduler, SpeculationConfig
    cfg = TINY_LLAMA.with_(d_model=512, n_heads=8, n_kv_heads=2, head_dim=64, ffn=1024, vocab=4096, n_layers=2)
    p = str(tmp_path / "q4k.gguf")
    save_gguf(p, cfg, random_weights(cfg, 9), PLAN_Q4_K)
    prompt = list(b"abcabcabcabc the cat sat on the mat the cat sat on")
    outs = {}
    for name, spec in (("plain", None), ("spec", SpeculationConfig(max_batch=4, ngram=3, draft=4))):
        be = CudaBackend.from_gguf(p, max_num_seqs=8, max_ctx=512, max_tokens=512)
        sch = Scheduler(be, ByteTokenizer(be.cfg.vocab), max_num_seqs=4, speculation=spec)
        r = sch.submit(prompt, SamplingParams(max_tokens=48), keep_sequence=True)
        sch.run_until_done([r])
        feed = [r.output[-1]] + list(b" again")
        r2 = sch.submit(feed, SamplingParams(max_tokens=16), seq_id=r.seq_id, keep_sequence=True, history=prompt + r.output[:-1])
        sch.run_until_done([r2])
        outs[name] = (r.output, r2.output)
        be.engine.check_status()
        if spec:
            assert sch.stats["spec_steps"] > 0
            print("speculation:", {k: v for k, v in sch.stats.items() if k.startswith("spec")}, "steps", sch.stats["steps"])
    assert outs["spec"] == outs["plain"]
    # the verify call itself: predictions at every position equal stepping one token at a time
    be = CudaBackend.from_gguf(p, max_num_seqs=8, max_ctx=512, max_tokens=512)
    be.begin(1, prompt)
    be.begin(2, prompt)
    be.forward([1, 2], [prompt[:-5], prompt[:-5]])
    tail = prompt[-5:]
    all_at_once = be.verify(1, tail)
    one_by_one = [be.step([2], [[t]], [SamplingParams()], [0.0])[0] for t in tail]
    assert all_at_once == one_by_one and be.seq_len(1) == len(prompt)
    be.truncate(1, len(prompt) - 3)
    assert be.seq_len(1) == len(prompt) - 3 and be.verify(1, tail[2:]) == all_at_once[2:]


def test_scoring_on_the_engine_matches_the_cpu_backend(tmp_path):
    """Log-probabilities of given continuations (evaluation packs): the engine's multi-position logits against the fp32 CPU
    backend on the same quantized file, in chunks longer than the logits workspace, and a multiple-choice item that reuses
    the context's keys and values through ``truncate``."""
    from openagents_b200.eval import multiple_choice
    from openagents_b200.serve.backend import CpuBackend, CudaBackend
    from openagents_b200.serve.generation import ByteTokenizer
    cfg = TINY_LLAMA.with_(d_model=512, n_heads=8, n_kv_heads=2, head_dim=64, ffn=1024, vocab=4096, n_layers=2)
    p = str(tmp_path / "q8.gguf")
    save_gguf(p, cfg, random_weights(cfg, 4), PLAN_Q8_0)
    gpu = CudaBackend.from_gguf(p, max_num_seqs=8, max_ctx=512, max_tokens=512)
    cpu = CpuBackend.from_gguf(p)
    free0 = gpu.kv_stats()["pages_free"]
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, cfg.vocab, (151,), generator=g).tolist()          # more than two chunks of 64 rows
    feed, tgt = toks[:-1], toks[1:]
    tgt[7] = -1
    gpu.begin(1, feed)
    cpu.begin(1, feed)
    a, b = gpu.score(1, feed, tgt), cpu.score(1, feed, tgt)
    gpu.engine.check_status()
    assert a[7] == 0.0 and gpu.seq_len(1) == 150
    worst = max(abs(x - y) for x, y in zip(a, b))
    assert worst < 0.15, worst                                                   # bf16 activations against fp32
    assert abs(sum(a) - sum(b)) / 150 < 0.02
    gpu.end(1)
    cpu.end(1)
    items = [{"context": "the cat sat on the", "choices": [" mat", " moon and stars", " q"], "answer": 0}]
    tok = ByteTokenizer(cfg.vocab)
    rg, rc = multiple_choice(gpu, items, tok), multiple_choice(cpu, items, tok)
    gpu.engine.check_status()
    assert all(abs(x - y) < 0.1 for x, y in zip(rg["picks"][0]["scores"], rc["picks"][0]["scores"]))
    assert gpu.kv_stats()["pages_free"] == free0                                 # every sequence was closed
