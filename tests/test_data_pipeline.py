"""Token shards, the stateless shuffled sampler, the prefetching loader and the native BPE."""
import numpy as np
import pytest
import torch

from openagents_b200.data import BatchLoader, ByteBpe, TokenDataset, permute, write_token_shard
from openagents_b200.data.bpe import split_pieces
from openagents_b200.oracle.cs336 import bpe_train


def _shards(tmp_path, sizes=(1000, 517), vocab=50000, mask=False):
    rng = np.random.default_rng(0)
    paths, all_tok = [], []
    for i, n in enumerate(sizes):
        t = rng.integers(0, vocab, n)
        m = (rng.random(n) < 0.5).astype(np.uint8) if mask else None
        p = tmp_path / f"s{i}.b2tk"
        write_token_shard(p, t, m)
        paths.append(p)
        all_tok.append((t, m))
    return paths, all_tok


def test_windows_and_targets(tmp_path):
    paths, toks = _shards(tmp_path)
    ds = TokenDataset(paths, seq_len=16)
    assert ds.tokens == 1517 and len(ds) == (999 // 16) + (516 // 16)
    tok, tgt, n = ds.window(3)
    assert n == 16 and tok.tolist() == toks[0][0][48:64].tolist() and tgt.tolist() == toks[0][0][49:65].tolist()
    first_of_second = 999 // 16
    tok, tgt, _ = ds.window(first_of_second)
    assert tok.tolist() == toks[1][0][:16].tolist()            # windows never straddle two shards
    with pytest.raises(IndexError):
        ds.window(len(ds))


def test_masked_targets_and_wide_ids(tmp_path):
    paths, toks = _shards(tmp_path, sizes=(400,), vocab=200000, mask=True)
    ds = TokenDataset(paths, seq_len=8)
    t, m = toks[0]
    tok, tgt, n = ds.window(5)
    want = [int(t[41 + i]) if m[41 + i] else -1 for i in range(8)]
    assert tgt.tolist() == want and n == sum(1 for x in want if x >= 0) and tok.tolist() == t[40:48].tolist()


def test_raw_dump_and_bad_files(tmp_path):
    raw = tmp_path / "raw.bin"
    np.arange(100, dtype=np.uint16).tofile(raw)
    with pytest.raises(ValueError, match="no shard header"):
        TokenDataset(raw, seq_len=8)
    ds = TokenDataset(raw, seq_len=8, raw_width=2)
    assert ds.window(1)[0].tolist() == list(range(8, 16))
    bad = tmp_path / "bad.b2tk"
    good = open(_shards(tmp_path, sizes=(64,))[0][0], "rb").read()
    bad.write_bytes(good[:60])                                    # header says 64 tokens, the file holds 14
    with pytest.raises(ValueError, match="shorter"):
        TokenDataset(bad, seq_len=8)
    with pytest.raises(ValueError, match="less than one window"):
        TokenDataset(_shards(tmp_path, sizes=(5,))[0], seq_len=8)


@pytest.mark.parametrize("total", [1, 2, 7, 64, 1000, 4097])
def test_permutation_is_a_bijection(total):
    for epoch in (0, 1):
        assert sorted(permute(total, 11, epoch, p) for p in range(total)) == list(range(total))
    if total >= 64:
        assert [permute(total, 11, 0, p) for p in range(total)] != [permute(total, 11, 1, p) for p in range(total)]
        assert [permute(total, 11, 0, p) for p in range(total)] != [permute(total, 12, 0, p) for p in range(total)]


def test_loader_ranks_are_disjoint_and_resume_continues(tmp_path):
    paths, _ = _shards(tmp_path, sizes=(4000, 3000))
    ds = TokenDataset(paths, seq_len=8)
    per_epoch = None
    seen = []
    for rank in range(2):
        ld = BatchLoader(ds, accum=2, micro_batch=3, rank=rank, world=2, seed=5, slots=3, threads=3, pin=False)
        per_epoch = ld.batches_per_epoch
        rows = []
        for _ in range(per_epoch):
            tok, tgt, n, b = ld.next()
            assert tok.shape == (2, 3, 8) and n == 48
            assert torch.equal(tok[..., 1:], tgt[..., :-1])
            rows += [tuple(r) for r in tok.reshape(-1, 8).tolist()]
        seen.append(rows)
        ld.close()
    assert per_epoch == len(ds) // 12
    every = [tuple(ds.window(i)[0].tolist()) for i in range(len(ds))]
    assert len(set(seen[0]) & set(seen[1])) == 0 or len(set(every)) < len(every)
    assert set(seen[0]) | set(seen[1]) <= set(every) and len(seen[0]) + len(seen[1]) == per_epoch * 12
    # one rank x 12 rows sees the same global batches as two ranks x 6 rows
    one = BatchLoader(ds, accum=4, micro_batch=3, seed=5, pin=False)
    b0 = set(tuple(r) for r in one.next()[0].reshape(-1, 8).tolist())
    assert b0 == set(seen[0][:6]) | set(seen[1][:6])
    # resume: a loader started at batch k continues the stream of one that ran from 0
    a = BatchLoader(ds, accum=1, micro_batch=4, seed=9, pin=False)
    stream = [a.next()[0].clone() for _ in range(7)]
    assert a.state() == {"next_batch": 7}
    b = BatchLoader(ds, accum=1, micro_batch=4, seed=9, start_batch=4, pin=False)
    assert all(torch.equal(b.next()[0], stream[4 + i]) for i in range(3))
    # the second epoch is another order of the same windows
    c = BatchLoader(ds, accum=1, micro_batch=4, seed=9, start_batch=a.batches_per_epoch, pin=False)
    assert not torch.equal(c.next()[0], stream[0])


def test_loader_refuses_a_dataset_smaller_than_a_batch(tmp_path):
    paths, _ = _shards(tmp_path, sizes=(100,))
    with pytest.raises(ValueError, match="fewer windows"):
        BatchLoader(TokenDataset(paths, seq_len=8), accum=4, micro_batch=8, pin=False)


def test_native_bpe_matches_the_plain_loop():
    data = (b"the cat sat on the mat, the rat sat on the cat. aaa aaaa banana bandana " * 7) + bytes(range(200, 256))
    want = bpe_train(data, 40)
    bpe = ByteBpe.train(data, 40, pieces="none")
    assert [(a, b) for a, b, _ in want["merges"]] == bpe.merges
    assert bpe.encode(data) == want["tokenIds"]
    assert bpe.decode_bytes(bpe.encode(data)) == data


def test_bpe_with_pieces_and_special_tokens():
    text = "Hello world, it's 2024!  The quick brown fox can't jump over 13 lazy dogs.\n\nnaïve café " * 20
    assert b"".join(split_pieces(text.encode())) == text.encode()
    pieces = split_pieces(b"it's 12 dogs,  two\n")
    assert pieces == [b"it", b"'s", b" 12", b" dogs", b",", b" ", b" two", b"\n"]
    bpe = ByteBpe.train(text.encode(), 60, special=["<|endoftext|>"])
    assert 0 < len(bpe.merges) <= 60 and bpe.vocab_size == 256 + len(bpe.merges) + 1
    ids = bpe.encode(text + "<|endoftext|>" + "fox")
    assert ids.count(bpe.special_ids["<|endoftext|>"]) == 1 and bpe.decode(ids) == text + "<|endoftext|>fox"
    assert len(ids) < len(text.encode()) // 2                      # it compresses its own training text
    assert all(b" " not in bpe.vocab[256 + k][1:] for k in range(len(bpe.merges)))   # no merge crosses a word boundary
    again = ByteBpe.from_json(bpe.to_json())
    assert again.encode("The lazy fox") == bpe.encode("The lazy fox")
    with pytest.raises(ValueError):
        ByteBpe([(300, 1)])


def test_native_bpe_equals_the_plain_loop_on_random_low_entropy_text():
    """Small alphabets make overlapping pairs ("aaaa"), ties and merges of merges common: the incremental trainer and the
    rank-ordered encoder must still agree with the loop that recounts every pair after every merge."""
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=150, deadline=None)
    @given(st.binary(min_size=0, max_size=120).map(lambda b: bytes(97 + (x % 3) for x in b)), st.integers(min_value=0, max_value=25))
    def check(data, merges):
        want = bpe_train(data, merges)
        bpe = ByteBpe.train(data, merges, pieces="none")
        assert bpe.merges == [(a, b) for a, b, _ in want["merges"]]
        assert bpe.encode(data) == want["tokenIds"]
        assert bpe.decode_bytes(bpe.encode(data)) == data

    check()


def test_loader_with_every_slot_and_thread_count_delivers_the_same_stream(tmp_path):
    paths, _ = _shards(tmp_path, sizes=(3000,))
    ds = TokenDataset(paths, seq_len=8)
    ref = None
    for slots, threads in ((2, 1), (2, 4), (3, 2), (5, 3), (8, 8)):
        ld = BatchLoader(ds, accum=1, micro_batch=5, seed=4, slots=slots, threads=threads, pin=False)
        got = [ld.next()[0].clone() for _ in range(40)]
        ld.close()
        ref = ref or got
        assert all(torch.equal(a, b) for a, b in zip(got, ref)), (slots, threads)


def test_loader_ring_protocol_is_checked_on_every_interleaving():
    """The slot ring of the loader as a model: safe and live on every interleaving of 2 slots x 2 workers x 5 batches and of
    3 slots x 3 workers x 5 batches; the two broken variants are caught (out-of-order delivery; the ring stalls)."""
    from openagents_b200.data.loader_model import check_loader_ring
    for slots, workers in ((2, 2), (3, 3), (2, 3)):
        r = check_loader_ring(slots, workers, 5)
        assert r["safety"].ok and r["safety"].states > 100, r["safety"]
        assert r["every_batch_is_delivered"].ok
        bad = r["mutation_worker_ignores_expected_batch"]
        assert not bad.ok and bad.violated in ("invariant delivered_in_order_exactly_once", "invariant one_filler_per_slot") and bad.trace
        assert not r["mutation_release_keeps_expected_batch"].ok
