"""Property test of the page allocator against a shadow model of what the device cache would hold.

Random interleavings of begin (with prefix lookup) / prefill / publish / decode / truncate / end over a small pool and a
three-letter alphabet (so prefixes collide all the time).  The shadow model writes every token a sequence appends into
the page slot the allocator assigned, exactly as the engine's kernels would, and after every operation checks that

* every live sequence still reads its own tokens from its pages (a prefix hit handed out the right K/V, nobody wrote
  into a page someone else still reads, truncate's copy-on-write protected the sharer),
* pages are conserved: free pages + distinct pages held by live sequences = the pool.
"""
import hypothesis.strategies as st
from hypothesis import settings
from hypothesis.stateful import RuleBasedStateMachine, initialize, invariant, precondition, rule

from openagents_b200.models.engine import KVPool

PS, NP = 4, 24
TOK = st.integers(0, 2)


class PoolMachine(RuleBasedStateMachine):
    @initialize()
    def start(self):
        self.pool = KVPool(NP, PS)
        self.content = [[None] * PS for _ in range(NP)]     # what the device cache holds, per page slot
        self.seqs: dict[int, list[int]] = {}                # live sequence -> its tokens (all of them have K/V)
        self.next_id = 1

    # ---- helpers
    def _write(self, sid, start):
        pages = self.pool.pages(sid)
        toks = self.seqs[sid]
        for p in range(start, len(toks)):
            self.content[pages[p // PS]][p % PS] = toks[p]

    def _append(self, sid, new):
        try:
            self.pool.extend(sid, len(new))
        except MemoryError:
            return False
        start = len(self.seqs[sid])
        self.seqs[sid] += new
        self._write(sid, start)
        return True

    # ---- rules
    @rule(tokens=st.lists(TOK, min_size=1, max_size=14), publish=st.booleans())
    def begin(self, tokens, publish):
        sid = self.next_id
        self.next_id += 1
        cached = self.pool.begin(sid, tokens)
        assert cached % PS == 0 and cached < len(tokens)
        pages = self.pool.pages(sid)
        for p in range(cached):                               # a hit must hold exactly these tokens already
            assert self.content[pages[p // PS]][p % PS] == tokens[p], "prefix hit with wrong contents"
        self.seqs[sid] = list(tokens[:cached])
        if not self._append(sid, list(tokens[cached:])):
            self.pool.end(sid)
            del self.seqs[sid]
            return
        if publish:
            self.pool.publish(sid, self.seqs[sid])

    @precondition(lambda self: self.seqs)
    @rule(data=st.data(), tok=TOK, publish=st.booleans())
    def decode(self, data, tok, publish):
        sid = data.draw(st.sampled_from(sorted(self.seqs)))
        if self._append(sid, [tok]) and publish:
            self.pool.publish(sid, self.seqs[sid])

    @precondition(lambda self: self.seqs)
    @rule(data=st.data())
    def truncate(self, data):
        sid = data.draw(st.sampled_from(sorted(self.seqs)))
        n = len(self.seqs[sid])
        new_len = data.draw(st.integers(0, n))
        try:
            cow = self.pool.truncate(sid, new_len)
        except MemoryError:
            return                                            # no page for the private copy: nothing changed
        if cow is not None:
            src, dst = cow
            self.content[dst] = list(self.content[src])       # the engine copies the page's K/V
        self.seqs[sid] = self.seqs[sid][:new_len]
        assert self.pool.length(sid) == new_len

    @precondition(lambda self: self.seqs)
    @rule(data=st.data())
    def end(self, data):
        sid = data.draw(st.sampled_from(sorted(self.seqs)))
        self.pool.end(sid)
        del self.seqs[sid]

    # ---- invariants
    @invariant()
    def sequences_read_their_own_tokens(self):
        if not hasattr(self, "pool"):
            return
        for sid, toks in self.seqs.items():
            assert self.pool.length(sid) == len(toks)
            pages = self.pool.pages(sid)
            assert len(pages) >= (len(toks) + PS - 1) // PS
            for p, t in enumerate(toks):
                assert self.content[pages[p // PS]][p % PS] == t, (sid, p)

    @invariant()
    def pages_are_conserved(self):
        if not hasattr(self, "pool"):
            return
        held = set()
        for sid in self.seqs:
            held.update(self.pool.pages(sid))
        assert self.pool.free_pages + len(held) == NP


PoolMachine.TestCase.settings = settings(max_examples=150, stateful_step_count=40, deadline=None)
TestPool = PoolMachine.TestCase
