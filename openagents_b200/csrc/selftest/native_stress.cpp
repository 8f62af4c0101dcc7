// A stress program for the host-side native code, meant to be built with a sanitizer:
//
//   g++ -std=c++17 -O1 -g -fsanitize=thread            native_stress.cpp ../data/*.cpp ../kv/kv_alloc.cpp ../gguf/*.cpp -pthread -fopenmp
//   g++ -std=c++17 -O1 -g -fsanitize=address,undefined native_stress.cpp ../data/*.cpp ../kv/kv_alloc.cpp ../gguf/*.cpp -pthread -fopenmp
//
// Thread sanitizer: the loader's worker threads, its ring of slots and the consumer (data races, lock order).  Address and
// undefined-behaviour sanitizers: the shard reader's bounds, the BPE trainer's and encoder's containers, the KV page pool
// under a random sequence of begin / extend / publish / truncate / end, and the GGUF reader on thousands of damaged files.  The program also checks the results it can check
// (every batch equals the windows the sampler names; an encoded text decodes to itself; the pool returns every page).
// Exit code 0 = all checks passed.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

extern "C" {
void* b200_tokds_open(const char** paths, int n_paths, int seq_len, int raw_width);
const char* b200_tokds_error(void*);
uint64_t b200_tokds_windows(void*);
void b200_tokds_close(void*);
int64_t b200_tokds_read(void*, uint64_t window, int64_t* tok, int64_t* tgt);
uint64_t b200_tokds_permute(uint64_t total, uint64_t seed, uint64_t epoch, uint64_t pos);
int b200_tok_shard_write(const char* path, const void* tokens, uint64_t n, int width, const uint8_t* mask);
void* b200_loader_create(void* ds, int rows, int rank, int world, uint64_t seed, uint64_t start_batch, int shuffle, int threads);
const char* b200_loader_error(void*);
int b200_loader_add_slot(void*, int64_t* tok, int64_t* tgt);
int b200_loader_start(void*);
int b200_loader_next(void*, int* slot, uint64_t* batch, int64_t* valid, int timeout_ms);
int b200_loader_release(void*, int slot);
void b200_loader_destroy(void*);
void* b200_bpe_train_text(const uint8_t* text, uint64_t n, int n_merges, int mode);
int b200_bpe_n_merges(void*);
void b200_bpe_get_merges(void*, int32_t* out);
void b200_bpe_train_free(void*);
void* b200_bpe_encoder(const int32_t* merges, int n_merges);
int64_t b200_bpe_encode(void*, const uint8_t* text, uint64_t n, int mode, int32_t* out, uint64_t cap);
void b200_bpe_encoder_free(void*);
void* b200_gguf_open(const char* path);
const char* b200_gguf_error(void*);
void b200_gguf_close(void*);
const char* b200_gguf_meta_json(void*);
uint64_t b200_gguf_n_tensors(void*);
const char* b200_gguf_tensor_name(void*, uint64_t i);
uint64_t b200_gguf_tensor_nbytes(void*, uint64_t i);
const void* b200_gguf_tensor_data(void*, uint64_t i);
void* b200_gguf_writer_new(const char* path, uint32_t alignment);
void b200_gguf_writer_kv_u32(void*, const char* key, uint32_t v);
void b200_gguf_writer_kv_str(void*, const char* key, const char* v, uint64_t n);
void b200_gguf_writer_kv_str_array(void*, const char* key, const char* blob, const uint64_t* lens, uint64_t n);
int b200_gguf_writer_tensor(void*, const char* name, uint32_t type, uint32_t ndim, const uint64_t* dims, const void* data);
int b200_gguf_writer_finish(void*);
void b200_gguf_writer_free(void*);
void* b200_kv_create(int32_t n_pages, int32_t page_size);
void b200_kv_destroy(void*);
int32_t b200_kv_free_pages(void*);
int32_t b200_kv_retained_pages(void*);
int32_t b200_kv_seq_pages(void*, int64_t, int32_t*, int32_t);
int32_t b200_kv_total_pages(void*);
int64_t b200_kv_seq_begin(void*, int64_t seq_id, const int32_t* tokens, int64_t n_tokens);
int32_t b200_kv_seq_extend(void*, int64_t seq_id, int64_t n_new);
void b200_kv_seq_publish(void*, int64_t seq_id, const int32_t* tokens, int64_t n_tokens);
int64_t b200_kv_seq_len(void*, int64_t seq_id);
int32_t b200_kv_seq_truncate(void*, int64_t seq_id, int64_t new_len, int32_t* cow_src, int32_t* cow_dst);
void b200_kv_seq_end(void*, int64_t seq_id);
}

static int failures = 0;
#define CHECK(cond)                                                       \
  do {                                                                    \
    if (!(cond)) {                                                        \
      std::fprintf(stderr, "check failed at line %d: %s\n", __LINE__, #cond); \
      failures++;                                                         \
    }                                                                     \
  } while (0)

static uint64_t rng_state = 0x243F6A8885A308D3ull;
static uint64_t rnd() {
  rng_state ^= rng_state << 13;
  rng_state ^= rng_state >> 7;
  rng_state ^= rng_state << 17;
  return rng_state;
}

static void loader_stress(const std::string& dir) {
  const int T = 16;
  std::vector<uint16_t> a(5000), b(3111);
  for (auto& x : a) x = (uint16_t)(rnd() % 50000);
  for (auto& x : b) x = (uint16_t)(rnd() % 50000);
  std::vector<uint8_t> mask(b.size());
  for (auto& m : mask) m = (uint8_t)(rnd() & 1);
  const std::string pa = dir + "/a.b2tk", pb = dir + "/b.b2tk";
  CHECK(b200_tok_shard_write(pa.c_str(), a.data(), a.size(), 2, nullptr) == 0);
  CHECK(b200_tok_shard_write(pb.c_str(), b.data(), b.size(), 2, mask.data()) == 0);
  const char* paths[2] = {pa.c_str(), pb.c_str()};
  void* ds = b200_tokds_open(paths, 2, T, 0);
  CHECK(b200_tokds_error(ds) == nullptr);
  const uint64_t windows = b200_tokds_windows(ds);
  CHECK(windows == (a.size() - 1) / T + (b.size() - 1) / T);
  for (int round = 0; round < 3; round++) {
    const int rows = 6, world = 2, rank = round % 2, slots = 2 + round * 2, threads = 1 + round * 3;
    const uint64_t seed = 77 + round, start = round * 5;
    void* L = b200_loader_create(ds, rows, rank, world, seed, start, 1, threads);
    CHECK(b200_loader_error(L) == nullptr);
    std::vector<std::vector<int64_t>> tok(slots, std::vector<int64_t>(rows * T)), tgt(slots, std::vector<int64_t>(rows * T));
    for (int s = 0; s < slots; s++) CHECK(b200_loader_add_slot(L, tok[s].data(), tgt[s].data()) == s);
    CHECK(b200_loader_start(L) == 0);
    const uint64_t usable = windows - windows % (uint64_t)(rows * world);
    std::vector<int64_t> wt(T), wg(T);
    const int batches = round == 2 ? 7 : 200;          // the last round destroys the loader while its workers are busy
    for (int i = 0; i < batches; i++) {
      int slot = -1;
      uint64_t batch = 0;
      int64_t valid = 0;
      CHECK(b200_loader_next(L, &slot, &batch, &valid, 20000) == 0);
      CHECK(batch == start + (uint64_t)i);
      int64_t want_valid = 0;
      for (int r = 0; r < rows; r++) {
        const uint64_t P = batch * (uint64_t)(world * rows) + (uint64_t)r * world + rank;
        const uint64_t w = b200_tokds_permute(windows, seed, P / usable, P % usable);
        want_valid += b200_tokds_read(ds, w, wt.data(), wg.data());
        CHECK(std::memcmp(wt.data(), tok[slot].data() + (size_t)r * T, T * sizeof(int64_t)) == 0);
        CHECK(std::memcmp(wg.data(), tgt[slot].data() + (size_t)r * T, T * sizeof(int64_t)) == 0);
      }
      CHECK(valid == want_valid);
      CHECK(b200_loader_release(L, slot) == 0);
      CHECK(b200_loader_release(L, slot) == -1);         // a slot is released once
    }
    b200_loader_destroy(L);
  }
  b200_tokds_close(ds);
}

static void bpe_stress() {
  std::string text;
  const char* words[] = {"the", "cat", "sat", "on", "a", "mat", "aaaa", "banana", "it's", "2024", "na\xc3\xafve", "  ", "\n"};
  for (int i = 0; i < 4000; i++) {
    text += words[rnd() % 13];
    text += (rnd() % 5 == 0) ? ", " : " ";
  }
  for (int mode = 0; mode < 2; mode++) {
    void* tr = b200_bpe_train_text((const uint8_t*)text.data(), text.size(), 200, mode);
    const int n = b200_bpe_n_merges(tr);
    CHECK(n > 10 && n <= 200);
    std::vector<int32_t> merges((size_t)n * 2);
    b200_bpe_get_merges(tr, merges.data());
    b200_bpe_train_free(tr);
    void* enc = b200_bpe_encoder(merges.data(), n);
    CHECK(enc != nullptr);
    std::vector<int32_t> ids(text.size());
    const int64_t k = b200_bpe_encode(enc, (const uint8_t*)text.data(), text.size(), mode, ids.data(), ids.size());
    CHECK(k > 0 && (size_t)k < text.size() / 2);
    std::vector<std::string> vocab(256 + n);
    for (int i = 0; i < 256; i++) vocab[i] = std::string(1, (char)i);
    for (int i = 0; i < n; i++) vocab[256 + i] = vocab[merges[2 * i]] + vocab[merges[2 * i + 1]];
    std::string back;
    for (int64_t i = 0; i < k; i++) back += vocab[ids[i]];
    CHECK(back == text);
    b200_bpe_encoder_free(enc);
  }
  int32_t bad[2] = {300, 1};
  CHECK(b200_bpe_encoder(bad, 1) == nullptr);
}

static void kv_stress() {
  const int page = 16;
  void* p = b200_kv_create(64, page);
  const int32_t total = b200_kv_free_pages(p);
  std::vector<int64_t> live;
  std::vector<std::vector<int32_t>> toks(32);
  for (int step = 0; step < 20000; step++) {
    const int op = (int)(rnd() % 5);
    if (op == 0 && live.size() < 12) {
      const int64_t id = 1 + (int64_t)(rnd() % 31);
      bool used = false;
      for (int64_t l : live) used |= l == id;
      if (used) continue;
      auto& t = toks[id];
      t.resize(1 + rnd() % 70);
      for (auto& x : t) x = (int32_t)(rnd() % 4);          // a tiny alphabet: prefix hits are common
      const int64_t cached = b200_kv_seq_begin(p, id, t.data(), (int64_t)t.size());
      if (cached < 0) continue;                              // out of pages: nothing was opened
      CHECK(cached <= (int64_t)t.size() && cached % page == 0);
      if (b200_kv_seq_extend(p, id, (int64_t)t.size() - cached) < 0) { b200_kv_seq_end(p, id); continue; }
      live.push_back(id);
    } else if (!live.empty()) {
      const size_t at = rnd() % live.size();
      const int64_t id = live[at];
      if (op == 1) {
        b200_kv_seq_publish(p, id, toks[id].data(), (int64_t)toks[id].size());
      } else if (op == 2) {
        const int64_t len = b200_kv_seq_len(p, id);
        CHECK(len == (int64_t)toks[id].size());
        const int64_t nl = (int64_t)(rnd() % (uint64_t)(len + 1));
        int32_t src = -1, dst = -1;
        const int32_t rc = b200_kv_seq_truncate(p, id, nl, &src, &dst);
        if (rc >= 0) toks[id].resize((size_t)nl);
        CHECK(rc != 1 || (src >= 0 && dst >= 0 && src != dst));
      } else if (op == 3) {
        const int64_t add = 1 + (int64_t)(rnd() % 20);
        if (b200_kv_seq_extend(p, id, add) >= 0)
          for (int64_t i = 0; i < add; i++) toks[id].push_back((int32_t)(rnd() % 4));
      } else {
        b200_kv_seq_end(p, id);
        live.erase(live.begin() + (long)at);
      }
    }
    CHECK(b200_kv_free_pages(p) >= 0 && b200_kv_free_pages(p) <= total);
    if (step % 50 == 0) {
      // every page is either held by a live sequence (shared pages once) or can be allocated (free, or a retained prefix page):
      // nothing leaks, and nothing that a sequence holds is also on offer
      std::vector<uint8_t> held((size_t)total, 0);
      int32_t n_held = 0, buf[64];
      for (int64_t id : live) {
        const int32_t n = b200_kv_seq_pages(p, id, buf, 64);
        CHECK(n >= 0 && n <= 64);
        for (int32_t i = 0; i < n; i++) {
          CHECK(buf[i] >= 0 && buf[i] < total);
          if (!held[(size_t)buf[i]]) { held[(size_t)buf[i]] = 1; n_held++; }
        }
      }
      CHECK(n_held + b200_kv_free_pages(p) == total);
      CHECK(b200_kv_retained_pages(p) >= 0 && b200_kv_retained_pages(p) <= b200_kv_free_pages(p));
    }
  }
  for (int64_t id : live) b200_kv_seq_end(p, id);
  CHECK(b200_kv_free_pages(p) == total);                    // published pages are cached, not leaked: ending every sequence frees them
  b200_kv_destroy(p);
}

// A valid file, then thousands of damaged copies (flipped bytes, overwritten 64-bit counts, cut tails): the reader must either
// refuse with an error or hand out tensors that lie inside the mapping; every byte it hands out is read here so that the
// address sanitizer sees an out-of-range pointer.
static void gguf_fuzz(const std::string& dir) {
  const std::string good = dir + "/good.gguf", bad = dir + "/bad.gguf";
  std::vector<float> w0(64 * 8), w1(32);
  for (auto& x : w0) x = (float)(rnd() % 100) / 10.f;
  for (auto& x : w1) x = 1.f;
  void* w = b200_gguf_writer_new(good.c_str(), 32);
  b200_gguf_writer_kv_str(w, "general.architecture", "llama", 5);
  b200_gguf_writer_kv_u32(w, "llama.block_count", 2);
  const char blob[] = "abcde";
  const uint64_t lens[3] = {1, 2, 2};
  b200_gguf_writer_kv_str_array(w, "tokenizer.ggml.tokens", blob, lens, 3);
  const uint64_t d0[2] = {64, 8}, d1[1] = {32};
  CHECK(b200_gguf_writer_tensor(w, "blk.0.w", 0, 2, d0, w0.data()) == 0);        // type 0: F32
  CHECK(b200_gguf_writer_tensor(w, "norm", 0, 1, d1, w1.data()) == 0);
  CHECK(b200_gguf_writer_finish(w) == 0);
  b200_gguf_writer_free(w);
  std::vector<uint8_t> bytes;
  {
    FILE* f = std::fopen(good.c_str(), "rb");
    CHECK(f != nullptr);
    uint8_t buf[4096];
    size_t n;
    while (f && (n = std::fread(buf, 1, sizeof buf, f)) > 0) bytes.insert(bytes.end(), buf, buf + n);
    if (f) std::fclose(f);
  }
  CHECK(bytes.size() > 64 * 8 * 4);
  int opened = 0, refused = 0;
  for (int iter = 0; iter < 3000; iter++) {
    std::vector<uint8_t> m = bytes;
    const int kind = (int)(rnd() % 4);
    const size_t header = m.size() - (64 * 8 + 32) * 4;          // most damage goes where the structure is
    if (kind == 0) {
      for (int k = 0; k < 1 + (int)(rnd() % 4); k++) m[rnd() % header] ^= (uint8_t)(1u << (rnd() % 8));
    } else if (kind == 1) {
      const size_t at = rnd() % (header - 8);
      const uint64_t v = (rnd() % 3 == 0) ? ~0ull : (rnd() % 3 == 0 ? (1ull << 62) : rnd());
      std::memcpy(m.data() + at, &v, 8);
    } else if (kind == 2) {
      m.resize(rnd() % m.size());
    } else {
      const size_t at = rnd() % header;
      m[at] = (uint8_t)rnd();
      m.resize(header + rnd() % (m.size() - header));
    }
    FILE* f = std::fopen(bad.c_str(), "wb");
    if (!f) continue;
    if (!m.empty()) std::fwrite(m.data(), 1, m.size(), f);
    std::fclose(f);
    void* r = b200_gguf_open(bad.c_str());
    if (b200_gguf_error(r) != nullptr) {
      refused++;
    } else {
      opened++;
      volatile uint64_t sink = std::strlen(b200_gguf_meta_json(r));
      const uint64_t nt = b200_gguf_n_tensors(r);
      CHECK(nt < 1000);
      for (uint64_t i = 0; i < nt; i++) {
        sink += std::strlen(b200_gguf_tensor_name(r, i));
        const uint8_t* p = (const uint8_t*)b200_gguf_tensor_data(r, i);
        const uint64_t nb = b200_gguf_tensor_nbytes(r, i);
        for (uint64_t k = 0; k < nb; k += 61) sink += p[k];
        if (nb) sink += p[nb - 1];
      }
      (void)sink;
    }
    b200_gguf_close(r);
  }
  CHECK(refused > 100 && opened > 10);                          // both outcomes were exercised
}

int main(int argc, char** argv) {
  if (argc < 2) {
    std::fprintf(stderr, "usage: native_stress <scratch directory>\n");
    return 2;
  }
  loader_stress(argv[1]);
  bpe_stress();
  kv_stress();
  gguf_fuzz(argv[1]);
  std::printf("native stress: %d failed checks\n", failures);
  return failures ? 1 : 0;
}
