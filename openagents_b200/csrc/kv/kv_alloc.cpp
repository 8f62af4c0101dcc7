// Paged KV-cache bookkeeping on the host: a page free-list with reference counts, per-sequence
// page lists, and a prefix index keyed by a hash chain over full pages of token ids so a new
// request can share the pages of an earlier one with the same prefix.  Published pages outlive their
// last holder (retained, oldest reclaimed first when pages run short), so the earlier request may be over.
//
// The reference lists "KV and prefix caches, continuous batching" as model-server infrastructure
// (docs/muse/muse-glimmer.md:113-114) and derives a cache-affinity key from a canonical prompt
// prefix (apps/openagents.com/workers/api/src/inference/prompt-prefix-cache.ts:324); the page
// mechanics here are this framework's own.
#include <cstdint>
#include <cstring>
#include <iterator>
#include <list>
#include <unordered_map>
#include <vector>

namespace {

struct Seq {
  std::vector<int32_t> pages;
  int64_t n_tokens = 0;
  std::vector<uint64_t> chain;  // hash of each full page's prefix chain, parallel to pages
};

struct Pool {
  int32_t n_pages, page_size;
  std::vector<int32_t> free_list;
  std::vector<int32_t> refcnt;
  std::vector<uint64_t> page_hash;     // chain hash a page is registered under (0 = none)
  std::vector<int32_t> page_tokens;    // [n_pages][page_size] token ids of a registered page: a hit must match them,
                                       // so a hash collision or a stale registration can never hand out wrong K/V
  std::unordered_map<uint64_t, int32_t> prefix;  // chain hash -> page
  // Registered pages that no sequence holds any more keep their K/V and their place in the prefix index until the page is
  // needed: a later prompt with the same prefix (the next turn of a closed conversation, the same system prompt an hour
  // later) still hits them.  Oldest first; a hit takes the page out again, an allocation that finds the free list empty takes
  // the oldest one and unregisters it.
  std::list<int32_t> retained;
  std::vector<std::list<int32_t>::iterator> retained_at;
  std::vector<uint8_t> is_retained;
  bool retain = true;                  // off: a page nobody holds leaves the index at once (prefix hits among live sequences only)
  std::unordered_map<int64_t, Seq> seqs;
  uint64_t hits = 0, lookups = 0;
};

uint64_t mix(uint64_t h, uint64_t v) {
  h ^= v + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
  h *= 0xff51afd7ed558ccdull;
  h ^= h >> 33;
  return h;
}

uint64_t page_chain_hash(uint64_t prev, const int32_t* toks, int n) {
  uint64_t h = prev ? prev : 0x243F6A8885A308D3ull;
  for (int i = 0; i < n; i++) h = mix(h, (uint64_t)(uint32_t)toks[i] + 1);
  return h ? h : 1;
}

void unregister_page(Pool* p, int32_t pg) {
  if (p->page_hash[pg]) {
    auto it = p->prefix.find(p->page_hash[pg]);
    if (it != p->prefix.end() && it->second == pg) p->prefix.erase(it);
    p->page_hash[pg] = 0;
  }
}

void release_page(Pool* p, int32_t pg) {
  if (--p->refcnt[pg] == 0) {
    if (p->retain && p->page_hash[pg]) {   // still a valid prefix page: keep it findable until the page is needed
      p->retained.push_back(pg);
      p->retained_at[pg] = std::prev(p->retained.end());
      p->is_retained[pg] = 1;
    } else {
      unregister_page(p, pg);
      p->free_list.push_back(pg);
    }
  }
}

inline int64_t available(const Pool* p) { return (int64_t)p->free_list.size() + (int64_t)p->retained.size(); }

// A page to write into: a free one, else the longest-unused retained prefix page (which leaves the index).  The caller has
// checked available() > 0.
int32_t take_page(Pool* p) {
  int32_t pg;
  if (!p->free_list.empty()) {
    pg = p->free_list.back();
    p->free_list.pop_back();
  } else {
    pg = p->retained.front();
    p->retained.pop_front();
    p->is_retained[pg] = 0;
    unregister_page(p, pg);
  }
  p->refcnt[pg] = 1;
  return pg;
}

// A prefix hit on a page: one more holder; a retained page is in use again.
void share_page(Pool* p, int32_t pg) {
  if (p->is_retained[pg]) {
    p->retained.erase(p->retained_at[pg]);
    p->is_retained[pg] = 0;
  }
  p->refcnt[pg]++;
}

}  // namespace

extern "C" {

void* b200_kv_create(int32_t n_pages, int32_t page_size) {
  Pool* p = new Pool();
  p->n_pages = n_pages;
  p->page_size = page_size;
  p->refcnt.assign(n_pages, 0);
  p->page_hash.assign(n_pages, 0);
  p->page_tokens.assign((size_t)n_pages * (size_t)page_size, -1);
  p->retained_at.assign(n_pages, p->retained.end());
  p->is_retained.assign(n_pages, 0);
  p->free_list.reserve(n_pages);
  for (int32_t i = n_pages - 1; i >= 0; i--) p->free_list.push_back(i);
  return p;
}
void b200_kv_destroy(void* h) { delete (Pool*)h; }
// Pages an allocation can take: free ones plus retained prefix pages (which are given up when needed).
int32_t b200_kv_free_pages(void* h) { return (int32_t)available((Pool*)h); }
int32_t b200_kv_retained_pages(void* h) { return (int32_t)((Pool*)h)->retained.size(); }
// Turn retention of published pages on or off; turning it off gives the pages retained so far back.
void b200_kv_set_retention(void* h, int32_t on) {
  Pool* p = (Pool*)h;
  p->retain = on != 0;
  if (!p->retain) {
    for (int32_t pg : p->retained) {
      p->is_retained[pg] = 0;
      unregister_page(p, pg);
      p->free_list.push_back(pg);
    }
    p->retained.clear();
  }
}
int32_t b200_kv_total_pages(void* h) { return ((Pool*)h)->n_pages; }
uint64_t b200_kv_prefix_hits(void* h) { return ((Pool*)h)->hits; }
uint64_t b200_kv_prefix_lookups(void* h) { return ((Pool*)h)->lookups; }

// Start a sequence.  If `tokens` is given, full pages whose prefix chain is already cached are
// shared; returns the number of tokens covered by shared pages (a multiple of the page size, and
// always less than n_tokens so at least one token is left to compute), or -1 if the id is in use.
int64_t b200_kv_seq_begin(void* h, int64_t seq_id, const int32_t* tokens, int64_t n_tokens) {
  Pool* p = (Pool*)h;
  if (p->seqs.count(seq_id)) return -1;
  Seq& s = p->seqs[seq_id];
  if (!tokens) return 0;
  uint64_t chain = 0;
  int64_t full = (n_tokens - 1) / p->page_size;  // leave the last token uncached
  for (int64_t i = 0; i < full; i++) {
    chain = page_chain_hash(chain, tokens + i * p->page_size, p->page_size);
    p->lookups++;
    auto it = p->prefix.find(chain);
    if (it == p->prefix.end()) break;
    if (std::memcmp(&p->page_tokens[(size_t)it->second * p->page_size], tokens + i * p->page_size,
                    sizeof(int32_t) * (size_t)p->page_size) != 0)
      break;                            // same hash, different tokens: not a hit
    p->hits++;
    share_page(p, it->second);
    s.pages.push_back(it->second);
    s.chain.push_back(chain);
    s.n_tokens += p->page_size;
  }
  return s.n_tokens;
}

// Grow the sequence to hold n_new more tokens.  Returns 0, -1 (unknown sequence) or -2 (out of
// pages; nothing is allocated in that case).
int32_t b200_kv_seq_extend(void* h, int64_t seq_id, int64_t n_new) {
  Pool* p = (Pool*)h;
  auto it = p->seqs.find(seq_id);
  if (it == p->seqs.end()) return -1;
  Seq& s = it->second;
  int64_t need = (s.n_tokens + n_new + p->page_size - 1) / p->page_size - (int64_t)s.pages.size();
  if (need > available(p)) return -2;
  for (int64_t i = 0; i < need; i++) s.pages.push_back(take_page(p));
  s.n_tokens += n_new;
  return 0;
}

// Register the sequence's full pages in the prefix index (call once their K/V are written).
// `tokens` are ALL n_tokens ids the sequence holds so far, from position 0 (for a continued session: the earlier
// turns too, not just the new one); a list longer than the sequence is cut to the sequence's length.
void b200_kv_seq_publish(void* h, int64_t seq_id, const int32_t* tokens, int64_t n_tokens) {
  Pool* p = (Pool*)h;
  auto it = p->seqs.find(seq_id);
  if (it == p->seqs.end()) return;
  Seq& s = it->second;
  if (n_tokens > s.n_tokens) n_tokens = s.n_tokens;
  int64_t full = n_tokens / p->page_size;
  if (full > (int64_t)s.pages.size()) full = (int64_t)s.pages.size();
  uint64_t chain = s.chain.empty() ? 0 : s.chain.back();
  for (int64_t i = (int64_t)s.chain.size(); i < full; i++) {
    chain = page_chain_hash(chain, tokens + i * p->page_size, p->page_size);
    s.chain.push_back(chain);
    int32_t pg = s.pages[i];
    if (!p->prefix.count(chain) && p->page_hash[pg] == 0) {
      p->prefix[chain] = pg;
      p->page_hash[pg] = chain;
      std::memcpy(&p->page_tokens[(size_t)pg * p->page_size], tokens + i * p->page_size, sizeof(int32_t) * (size_t)p->page_size);
    }
  }
}

int64_t b200_kv_seq_len(void* h, int64_t seq_id) {
  Pool* p = (Pool*)h;
  auto it = p->seqs.find(seq_id);
  return it == p->seqs.end() ? -1 : it->second.n_tokens;
}
int32_t b200_kv_seq_n_pages(void* h, int64_t seq_id) {
  Pool* p = (Pool*)h;
  auto it = p->seqs.find(seq_id);
  return it == p->seqs.end() ? -1 : (int32_t)it->second.pages.size();
}
// Copies up to `cap` page ids; returns the number of pages of the sequence.
int32_t b200_kv_seq_pages(void* h, int64_t seq_id, int32_t* out, int32_t cap) {
  Pool* p = (Pool*)h;
  auto it = p->seqs.find(seq_id);
  if (it == p->seqs.end()) return -1;
  const auto& pg = it->second.pages;
  int32_t n = (int32_t)pg.size();
  std::memcpy(out, pg.data(), sizeof(int32_t) * (size_t)(n < cap ? n : cap));
  return n;
}
// One decode step for a whole batch in a single call: every sequence grows by one token and the
// per-sequence launch metadata is written straight into the caller's (pinned) staging arrays:
// pos[b] = position of the new token, slot[b] = its physical cache slot, ctx[b] = new length,
// table[b][0..max_pages) = page list (rows are rewritten only when `full_table` is set or the
// sequence just took a new page).  Returns 0, or -1 unknown sequence / -2 out of pages / -3 sequence
// longer than max_pages pages; on an error NO sequence of the batch has changed (the batch is checked
// before it is grown).  *table_dirty is set when any table row was written.
int32_t b200_kv_stage_decode(void* h, const int64_t* seq_ids, int32_t B, int32_t max_pages, int32_t full_table,
                             int32_t* pos, int32_t* slot, int32_t* ctx, int32_t* table, int32_t* table_dirty) {
  Pool* p = (Pool*)h;
  const int64_t ps = p->page_size;
  int32_t dirty = 0;
  {   // first pass: nothing is changed unless the whole batch can grow
    int64_t need = 0;
    for (int32_t b = 0; b < B; b++) {
      auto it = p->seqs.find(seq_ids[b]);
      if (it == p->seqs.end()) return -1;
      const Seq& s = it->second;
      const int64_t pages_after = (s.n_tokens + 1 + ps - 1) / ps;
      if (pages_after > max_pages || (int64_t)s.pages.size() > max_pages) return -3;
      if (pages_after > (int64_t)s.pages.size()) need++;
    }
    if (need > available(p)) return -2;
  }
  for (int32_t b = 0; b < B; b++) {
    auto it = p->seqs.find(seq_ids[b]);
    if (it == p->seqs.end()) return -1;
    Seq& s = it->second;
    const int64_t p0 = s.n_tokens;
    const bool new_page = (p0 + 1 + ps - 1) / ps > (int64_t)s.pages.size();
    if (new_page) {
      if ((int64_t)s.pages.size() + 1 > max_pages) return -3;
      if (available(p) == 0) return -2;
      s.pages.push_back(take_page(p));
    }
    if ((int64_t)s.pages.size() > max_pages) return -3;
    s.n_tokens = p0 + 1;
    pos[b] = (int32_t)p0;
    slot[b] = (int32_t)(s.pages[p0 / ps] * ps + p0 % ps);
    ctx[b] = (int32_t)(p0 + 1);
    if (full_table || new_page) {
      int32_t* row = table + (size_t)b * max_pages;
      std::memcpy(row, s.pages.data(), sizeof(int32_t) * s.pages.size());
      std::memset(row + s.pages.size(), 0, sizeof(int32_t) * (size_t)(max_pages - (int64_t)s.pages.size()));
      dirty = 1;
    }
  }
  *table_dirty = dirty;
  return 0;
}

// Drop the tokens from position new_len on (a rejected speculative tail, a cancelled turn).  Pages that fall
// away are released.  The page that stays partly filled will be written again from position new_len, so it leaves the
// prefix index, and if another sequence shares it this sequence gets a page of its own: the call then returns 1 with
// *cow_src / *cow_dst set, and the caller must copy the page's K/V (every layer) from src to dst before the next
// write.  Returns 0 when no copy is needed, -1 for a bad sequence or length, -2 when a private page is needed and
// none is free (nothing has changed in that case).
int32_t b200_kv_seq_truncate(void* h, int64_t seq_id, int64_t new_len, int32_t* cow_src, int32_t* cow_dst) {
  Pool* p = (Pool*)h;
  auto it = p->seqs.find(seq_id);
  if (it == p->seqs.end() || new_len < 0 || new_len > it->second.n_tokens) return -1;
  Seq& s = it->second;
  const size_t keep = (size_t)((new_len + p->page_size - 1) / p->page_size);
  const size_t full = (size_t)(new_len / p->page_size);
  const bool partial = keep > full && keep <= s.pages.size();
  int32_t rc = 0;
  if (partial) {
    const int32_t pg = s.pages[full];
    if (p->refcnt[pg] > 1) {
      if (available(p) == 0) return -2;
      const int32_t fresh = take_page(p);
      p->refcnt[pg]--;                  // the other holders keep the original (and its registration)
      s.pages[full] = fresh;
      if (cow_src) *cow_src = pg;
      if (cow_dst) *cow_dst = fresh;
      rc = 1;
    } else {
      unregister_page(p, pg);
    }
  }
  while (s.pages.size() > keep) {
    release_page(p, s.pages.back());
    s.pages.pop_back();
  }
  if (s.chain.size() > full) s.chain.resize(full);
  s.n_tokens = new_len;
  return rc;
}
void b200_kv_seq_end(void* h, int64_t seq_id) {
  Pool* p = (Pool*)h;
  auto it = p->seqs.find(seq_id);
  if (it == p->seqs.end()) return;
  for (int32_t pg : it->second.pages) release_page(p, pg);
  p->seqs.erase(it);
}

}  // extern "C"
