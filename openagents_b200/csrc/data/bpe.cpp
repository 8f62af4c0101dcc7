// Byte-level BPE: trainer and encoder.
//
// Ids 0..255 are the bytes; merge k creates id 256 + k.  The trainer picks the most frequent adjacent pair (ties: the
// pair with the lower first id, then the lower second id), counting every adjacent position of every word times the
// word's count, and replaces its occurrences left to right.  Pair counts are kept incrementally: a merge only recounts
// the words that contain the pair, found through a pair -> words index, and the maximum comes from a heap with lazy
// deletion.  With the whole text as a single word this is exactly the plain loop "count all pairs, merge the best,
// repeat"; with pre-tokenisation the words are the distinct pieces and their multiplicities.
//
// Pre-tokenisation ("pieces"): mode 0 none; mode 1 splits like the GPT-2 pattern restricted to what can be decided per
// byte: contractions ('s 't 're 've 'm 'll 'd), an optional leading space followed by a run of letters (bytes >= 0x80
// count as letters, so UTF-8 sequences stay inside one piece), or of digits, or of other printable bytes; runs of white
// space, where the last space before a non-space starts the next piece.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <queue>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#define B200_API extern "C" __attribute__((visibility("default")))

namespace {

inline bool is_letter(uint8_t c) { return (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z') || c >= 0x80; }
inline bool is_digit(uint8_t c) { return c >= '0' && c <= '9'; }
inline bool is_space(uint8_t c) { return c == ' ' || c == '\t' || c == '\n' || c == '\r' || c == '\v' || c == '\f'; }
inline int cls(uint8_t c) { return is_letter(c) ? 0 : is_digit(c) ? 1 : is_space(c) ? 3 : 2; }

// Appends the end offset of every piece of text[0, n) to ends.
void split_pieces(const uint8_t* t, uint64_t n, int mode, std::vector<uint64_t>& ends) {
  if (mode == 0) {
    if (n) ends.push_back(n);
    return;
  }
  uint64_t i = 0;
  while (i < n) {
    uint64_t j = i;
    if (t[i] == '\'' && i + 1 < n) {                      // contractions
      const uint8_t a = t[i + 1] | 0x20, b = i + 2 < n ? (t[i + 2] | 0x20) : 0;
      if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e') || (a == 'l' && b == 'l')) { ends.push_back(i + 3); i += 3; continue; }
      if (a == 's' || a == 't' || a == 'm' || a == 'd') { ends.push_back(i + 2); i += 2; continue; }
    }
    if (is_space(t[i])) {
      while (j < n && is_space(t[j])) j++;
      if (j < n && j - i > 1 && t[j - 1] == ' ') j--;     // the last space belongs to the next piece
      else if (j < n && j - i == 1 && t[i] == ' ') {      // one space followed by a non-space: it leads that piece
        const int c = cls(t[j]);
        uint64_t k = j;
        while (k < n && cls(t[k]) == c) k++;
        ends.push_back(k);
        i = k;
        continue;
      }
      ends.push_back(j);
      i = j;
      continue;
    }
    const int c = cls(t[i]);
    while (j < n && cls(t[j]) == c) j++;
    ends.push_back(j);
    i = j;
  }
}

using Pair = uint64_t;
inline Pair mk(int32_t a, int32_t b) { return ((uint64_t)(uint32_t)a << 32) | (uint32_t)b; }

struct HeapItem {
  int64_t count;
  Pair pair;
  bool operator<(const HeapItem& o) const {          // max-heap: higher count first, then the LOWER pair
    if (count != o.count) return count < o.count;
    return pair > o.pair;
  }
};

struct Trained {
  std::vector<int32_t> merges;       // a, b per merge
  std::string error;
};

struct Word {
  std::vector<int32_t> ids;
  int64_t count;
};

void train(std::vector<Word>& words, int n_merges, Trained* out) {
  std::unordered_map<Pair, int64_t> cnt;
  std::unordered_map<Pair, std::vector<uint32_t>> where;      // may hold stale or repeated entries; checked on use
  std::priority_queue<HeapItem> heap;
  cnt.reserve(1 << 16);
  for (uint32_t w = 0; w < words.size(); w++) {
    const auto& ids = words[w].ids;
    for (size_t i = 0; i + 1 < ids.size(); i++) {
      const Pair p = mk(ids[i], ids[i + 1]);
      cnt[p] += words[w].count;
      auto& v = where[p];
      if (v.empty() || v.back() != w) v.push_back(w);
    }
  }
  for (auto& kv : cnt) heap.push({kv.second, kv.first});
  std::vector<Pair> touched;
  for (int k = 0; k < n_merges; k++) {
    Pair best = 0;
    bool found = false;
    while (!heap.empty()) {
      const HeapItem top = heap.top();
      auto it = cnt.find(top.pair);
      if (it != cnt.end() && it->second == top.count && top.count > 0) { best = top.pair; found = true; break; }
      heap.pop();
    }
    if (!found) break;
    const int32_t a = (int32_t)(best >> 32), b = (int32_t)(best & 0xffffffffu), nid = 256 + k;
    out->merges.push_back(a);
    out->merges.push_back(b);
    std::vector<uint32_t> ws;
    ws.swap(where[best]);
    std::sort(ws.begin(), ws.end());
    ws.erase(std::unique(ws.begin(), ws.end()), ws.end());
    touched.clear();
    for (uint32_t w : ws) {
      auto& ids = words[w].ids;
      bool has = false;
      for (size_t i = 0; i + 1 < ids.size(); i++)
        if (ids[i] == a && ids[i + 1] == b) { has = true; break; }
      if (!has) continue;
      const int64_t c = words[w].count;
      for (size_t i = 0; i + 1 < ids.size(); i++) {
        const Pair p = mk(ids[i], ids[i + 1]);
        cnt[p] -= c;
        touched.push_back(p);
      }
      size_t o = 0;
      for (size_t i = 0; i < ids.size();) {
        if (i + 1 < ids.size() && ids[i] == a && ids[i + 1] == b) { ids[o++] = nid; i += 2; }
        else ids[o++] = ids[i++];
      }
      ids.resize(o);
      for (size_t i = 0; i + 1 < ids.size(); i++) {
        const Pair p = mk(ids[i], ids[i + 1]);
        cnt[p] += c;
        touched.push_back(p);
        if (ids[i] == nid || ids[i + 1] == nid) {
          auto& v = where[p];
          if (v.empty() || v.back() != w) v.push_back(w);
        }
      }
    }
    cnt.erase(best);
    std::sort(touched.begin(), touched.end());
    touched.erase(std::unique(touched.begin(), touched.end()), touched.end());
    for (Pair p : touched) {
      auto it = cnt.find(p);
      if (it == cnt.end()) continue;
      if (it->second <= 0) cnt.erase(it);
      else heap.push({it->second, p});
    }
  }
}

struct Encoder {
  std::unordered_map<Pair, int32_t> rank;        // pair -> merge index
  std::unordered_map<std::string, std::vector<int32_t>> cache;
};

void encode_piece(Encoder* e, const uint8_t* t, size_t n, std::vector<int32_t>& out) {
  if (n == 1) { out.push_back(t[0]); return; }
  std::string key((const char*)t, n);
  if (n <= 64) {
    auto it = e->cache.find(key);
    if (it != e->cache.end()) { out.insert(out.end(), it->second.begin(), it->second.end()); return; }
  }
  std::vector<int32_t> ids(t, t + n);
  for (;;) {
    int32_t best = INT32_MAX;
    for (size_t i = 0; i + 1 < ids.size(); i++) {
      auto it = e->rank.find(mk(ids[i], ids[i + 1]));
      if (it != e->rank.end() && it->second < best) best = it->second;
    }
    if (best == INT32_MAX) break;
    // merge every occurrence of the lowest-ranked pair, left to right
    Pair bp = 0;
    for (size_t i = 0; i + 1 < ids.size(); i++) {
      auto it = e->rank.find(mk(ids[i], ids[i + 1]));
      if (it != e->rank.end() && it->second == best) { bp = it->first; break; }
    }
    const int32_t a = (int32_t)(bp >> 32), b = (int32_t)(bp & 0xffffffffu), nid = 256 + best;
    size_t o = 0;
    for (size_t i = 0; i < ids.size();) {
      if (i + 1 < ids.size() && ids[i] == a && ids[i + 1] == b) { ids[o++] = nid; i += 2; }
      else ids[o++] = ids[i++];
    }
    ids.resize(o);
  }
  if (n <= 64 && e->cache.size() < (1u << 20)) e->cache.emplace(std::move(key), ids);
  out.insert(out.end(), ids.begin(), ids.end());
}

}  // namespace

// Pieces of text: writes up to cap end offsets, returns how many pieces there are.
B200_API int64_t b200_bpe_split(const uint8_t* text, uint64_t n, int mode, uint64_t* ends, uint64_t cap) {
  std::vector<uint64_t> e;
  split_pieces(text, n, mode, e);
  for (size_t i = 0; i < e.size() && i < cap; i++) ends[i] = e[i];
  return (int64_t)e.size();
}

B200_API void* b200_bpe_train_text(const uint8_t* text, uint64_t n, int n_merges, int mode) {
  auto* out = new Trained();
  if (n_merges < 0 || (mode != 0 && mode != 1)) { out->error = "bad arguments"; return out; }
  std::vector<uint64_t> ends;
  split_pieces(text, n, mode, ends);
  std::unordered_map<std::string, int64_t> uniq;
  uint64_t at = 0;
  for (uint64_t e : ends) {
    uniq[std::string((const char*)text + at, e - at)]++;
    at = e;
  }
  std::vector<std::pair<std::string, int64_t>> sorted(uniq.begin(), uniq.end());
  std::sort(sorted.begin(), sorted.end());           // a fixed word order, whatever the hash function
  std::vector<Word> words;
  words.reserve(sorted.size());
  for (auto& kv : sorted) {
    Word w;
    w.ids.assign((const uint8_t*)kv.first.data(), (const uint8_t*)kv.first.data() + kv.first.size());
    w.count = kv.second;
    words.push_back(std::move(w));
  }
  train(words, n_merges, out);
  return out;
}
B200_API const char* b200_bpe_train_error(void* h) { auto* t = (Trained*)h; return t->error.empty() ? nullptr : t->error.c_str(); }
B200_API int b200_bpe_n_merges(void* h) { return (int)(((Trained*)h)->merges.size() / 2); }
B200_API void b200_bpe_get_merges(void* h, int32_t* out) {
  auto* t = (Trained*)h;
  std::memcpy(out, t->merges.data(), t->merges.size() * sizeof(int32_t));
}
B200_API void b200_bpe_train_free(void* h) { delete (Trained*)h; }

// merges: 2 ids per merge, in training order.  A merge may only name bytes and earlier merges.
B200_API void* b200_bpe_encoder(const int32_t* merges, int n_merges) {
  auto* e = new Encoder();
  for (int k = 0; k < n_merges; k++) {
    const int32_t a = merges[2 * k], b = merges[2 * k + 1];
    if (a < 0 || b < 0 || a >= 256 + k || b >= 256 + k) { delete e; return nullptr; }
    e->rank.emplace(mk(a, b), k);          // the first merge of a pair wins
  }
  return e;
}
// Returns the number of ids; writes at most cap of them.  One encoder must not be used from two threads at once.
B200_API int64_t b200_bpe_encode(void* h, const uint8_t* text, uint64_t n, int mode, int32_t* out, uint64_t cap) {
  auto* e = (Encoder*)h;
  std::vector<uint64_t> ends;
  split_pieces(text, n, mode, ends);
  std::vector<int32_t> ids;
  ids.reserve(n / 3 + 8);
  uint64_t at = 0;
  for (uint64_t end : ends) {
    encode_piece(e, text + at, end - at, ids);
    at = end;
  }
  for (size_t i = 0; i < ids.size() && i < cap; i++) out[i] = ids[i];
  return (int64_t)ids.size();
}
B200_API void b200_bpe_encoder_free(void* h) { delete (Encoder*)h; }
