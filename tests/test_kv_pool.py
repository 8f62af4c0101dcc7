"""Paged KV bookkeeping and prefix sharing (host C++)."""
import pytest

from openagents_b200.models.engine import KVPool


def test_alloc_extend_free():
    p = KVPool(8, 16)
    assert p.free_pages == 8
    assert p.begin(1) == 0
    p.extend(1, 17)
    assert p.length(1) == 17 and len(p.pages(1)) == 2 and p.free_pages == 6
    p.extend(1, 15)
    assert len(p.pages(1)) == 2
    p.extend(1, 1)
    assert len(p.pages(1)) == 3
    with pytest.raises(MemoryError):
        p.extend(1, 16 * 6)
    assert p.length(1) == 33          # a failed extend allocates nothing
    p.truncate(1, 16)
    assert len(p.pages(1)) == 1 and p.free_pages == 7
    p.end(1)
    assert p.free_pages == 8
    with pytest.raises(KeyError):
        p.extend(1, 1)


def test_prefix_sharing():
    p = KVPool(16, 16)
    toks = list(range(40))
    assert p.begin(1, toks) == 0
    p.extend(1, 40)
    p.publish(1, toks)
    pages1 = p.pages(1)
    # same first 32 tokens, different tail: two full pages are shared
    toks2 = toks[:32] + [999] * 10
    cached = p.begin(2, toks2)
    assert cached == 32
    p.extend(2, len(toks2) - cached)
    pages2 = p.pages(2)
    assert pages2[:2] == pages1[:2] and pages2[2] != pages1[2]
    # an identical prompt never reuses its last token's page: one token is always left to compute
    assert p.begin(3, toks[:32]) == 16
    hits, lookups = p.prefix_stats
    assert hits == 3 and lookups >= 3
    p.end(1)
    assert p.pages(2)[:2] == pages1[:2]      # shared pages survive their first owner
    p.end(2)
    p.end(3)
    assert p.free_pages == 16                # every page can be allocated again ...
    assert p.retained_pages == 2             # ... and the two published pages stay findable until their pages are needed
    assert p.begin(4, toks) == 32 and p.retained_pages == 0 and p.free_pages == 14
    p.end(4)


def test_retained_prefix_pages_are_reclaimed_oldest_first_and_never_hit_stale():
    """Pages of a closed conversation keep serving prefix hits; an allocation that finds no free page takes the longest-unused
    retained page, which leaves the index, so a later lookup of that prefix misses instead of reading another sequence's K/V."""
    p = KVPool(8, 16)
    a, b = list(range(100, 148)), list(range(200, 248))          # 48 tokens = 3 pages each
    for sid, toks in ((1, a), (2, b)):
        assert p.begin(sid, toks) == 0
        p.extend(sid, 48)
        p.publish(sid, toks)
        p.end(sid)                                               # a first, then b: a's pages are the oldest
    assert p.retained_pages == 6 and p.free_pages == 8
    assert p.begin(3, None) == 0
    p.extend(3, 16 * 4)                                          # 2 free pages + the 2 oldest retained ones (a's first two)
    assert p.retained_pages == 4 and p.free_pages == 4
    assert p.begin(4, a + [1]) == 0                              # a's chain is broken at its first page: a miss, not stale K/V
    p.end(4)
    assert p.begin(5, b + [1]) == 48 and p.retained_pages == 1   # b is intact; the hit takes its pages out of the retained list
    with pytest.raises(MemoryError):
        p.extend(5, 16 * 3)                                      # 1 retained + 0 free < 2 more pages needed beyond the partial one
    p.extend(5, 16)                                              # one more page: the last retained one (a's third) is reclaimed
    assert p.retained_pages == 0 and p.free_pages == 0
    p.end(3)
    p.end(5)
    assert p.free_pages == 8 and p.retained_pages == 3           # b's published pages are retained again


def test_stage_decode_batch():
    """One native call grows a whole decode batch and fills the launch metadata."""
    import torch
    from openagents_b200.models.engine import KVPool
    pool = KVPool(64)
    for sid, n in ((7, 15), (9, 33)):
        pool.begin(sid)
        pool.extend(sid, n)
    seq = torch.tensor([7, 9], dtype=torch.int64)
    pos, slot, ctx = (torch.zeros(2, dtype=torch.int32) for _ in range(3))
    table = torch.full((2, 8), -1, dtype=torch.int32)
    args = (seq.data_ptr(), 2, 8)
    ptrs = (pos.data_ptr(), slot.data_ptr(), ctx.data_ptr(), table.data_ptr())
    assert pool.stage_decode(*args, True, *ptrs) is True
    assert pos.tolist() == [15, 33] and ctx.tolist() == [16, 34]
    assert table[0].tolist() == pool.pages(7) + [0] * 7 and table[1, :3].tolist() == pool.pages(9)
    assert slot.tolist() == [pool.pages(7)[0] * 16 + 15, pool.pages(9)[2] * 16 + 1]
    assert pool.stage_decode(*args, False, *ptrs) is True          # sequence 7 crossed into a new page
    assert len(pool.pages(7)) == 2 and table[0, :2].tolist() == pool.pages(7) and slot[0].item() == pool.pages(7)[1] * 16
    assert pool.stage_decode(*args, False, *ptrs) is False and pool.length(7) == 18
    import pytest
    with pytest.raises(KeyError):
        pool.stage_decode(torch.tensor([1234], dtype=torch.int64).data_ptr(), 1, 8, True, *ptrs)
    with pytest.raises(ValueError):
        pool.stage_decode(*args[:2], 1, True, *ptrs)


def test_publish_covers_the_whole_sequence_and_hits_compare_tokens():
    """A page is registered under the tokens it really holds: publishing a continued sequence takes the full token
    list, and a lookup whose tokens differ from the registered page's is not a hit."""
    p = KVPool(32, 16)
    turn1 = list(range(100, 140))                  # 40 tokens
    p.begin(1, turn1)
    p.extend(1, 40)
    p.publish(1, turn1)
    gen = list(range(500, 508))                    # 8 generated tokens, then a second turn of 16
    turn2 = list(range(700, 716))
    p.extend(1, 8 + 16)
    p.publish(1, turn1 + gen + turn2)              # 64 tokens: pages 2 and 3 are registered under their true contents
    assert p.begin(2, turn1 + gen + turn2 + [1]) == 64
    assert p.begin(3, turn2 * 4 + [1]) == 0        # the new turn alone is not a prefix of anything cached
    # a list longer than the sequence is cut to what the sequence holds
    p.begin(4)
    p.extend(4, 16)
    p.publish(4, list(range(900, 948)))
    assert p.begin(5, list(range(900, 948)) + [1]) == 16


def test_truncate_unregisters_the_partial_page_and_copies_a_shared_one():
    p = KVPool(32, 16)
    A = list(range(200, 248))                      # three full pages
    p.begin(1, A)
    p.extend(1, 48)
    p.publish(1, A)
    assert p.truncate(1, 20) is None               # sole owner: page 1 stays, leaves the index
    assert len(p.pages(1)) == 2
    assert p.begin(2, A + [1]) == 16               # only page 0 can still be shared
    p.end(2)
    # shared partial page: the truncating sequence gets its own copy, the other keeps the original
    B = list(range(300, 348))
    p.begin(3, B)
    p.extend(3, 48)
    p.publish(3, B)
    assert p.begin(4, B + [7]) == 48
    p.extend(4, 1)
    before = p.pages(3)
    cow = p.truncate(4, 40)
    assert cow is not None and cow[0] == before[2] and cow[1] not in before
    assert p.pages(4)[2] == cow[1] and p.pages(3) == before
    assert p.begin(5, B + [9]) == 48               # sequence 3's pages are still registered and intact
    with pytest.raises(ValueError):
        p.truncate(4, 1000)


def test_stage_decode_is_all_or_nothing():
    import torch
    pool = KVPool(3, 16)
    for sid in (1, 2):
        pool.begin(sid)
        pool.extend(sid, 16)                       # both sit on a page boundary; one page is left
    seq = torch.tensor([1, 2], dtype=torch.int64)
    pos, slot, ctx = (torch.zeros(2, dtype=torch.int32) for _ in range(3))
    table = torch.zeros((2, 4), dtype=torch.int32)
    with pytest.raises(MemoryError):
        pool.stage_decode(seq.data_ptr(), 2, 4, True, pos.data_ptr(), slot.data_ptr(), ctx.data_ptr(), table.data_ptr())
    assert pool.length(1) == 16 and pool.length(2) == 16 and pool.free_pages == 1      # nothing grew


def test_retention_can_be_switched_off(monkeypatch):
    toks = list(range(40))

    def closed_conversation(p):
        p.begin(1, toks)
        p.extend(1, 40)
        p.publish(1, toks)
        p.end(1)
    p = KVPool(16, 16)
    closed_conversation(p)
    assert p.retained_pages == 2
    p.set_retention(False)                       # switching off gives back what was retained
    assert p.retained_pages == 0 and p.free_pages == 16 and p.begin(2, toks) == 0
    p.end(2)
    closed_conversation(p)
    assert p.retained_pages == 0 and p.begin(3, toks) == 0
    monkeypatch.setenv("B200_KV_RETAIN", "0")   # the process-wide default (what bit-exact repeat tests set)
    q = KVPool(16, 16)
    closed_conversation(q)
    assert q.retained_pages == 0 and q.begin(2, toks) == 0
