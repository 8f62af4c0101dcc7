// Token shards, a deterministic shuffled sampler and a prefetching batch loader for training.
//
// A shard file is a 32-byte header followed by the token ids (little endian, 2 or 4 bytes each) and, optionally, one
// byte per token saying whether that token is a training target (instruction tuning masks the prompt tokens):
//
//   offset 0   char[4]  "B2TK"
//          4   u32      version (1)
//          8   u32      bytes per token (2 or 4)
//         12   u32      flags (bit 0: a target mask follows the tokens)
//         16   u64      number of tokens
//         24   u64      reserved (0)
//
// A file without the header can be opened as a raw dump of 2- or 4-byte ids (the layout several public GPT-2 data
// preparations write).  A data set is a list of shards cut into windows of seq_len + 1 tokens with stride seq_len: the
// first seq_len tokens are the inputs, the last seq_len the targets.  The order of windows in epoch e is a keyed
// permutation (a 4-round Feistel network on the next power of four, cycle-walked into range), so the sampler has no
// state beyond a batch counter: resuming a run needs that one integer, and every rank computes its own rows of batch b
// without talking to the others.
//
// The loader fills caller-provided buffers (pinned host memory, so that the copy to the GPU is asynchronous) from worker
// threads and hands them over in batch order.
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#define B200_API extern "C" __attribute__((visibility("default")))

namespace {

struct Shard {
  int fd = -1;
  void* map = nullptr;
  size_t size = 0;
  const uint8_t* tokens = nullptr;
  const uint8_t* mask = nullptr;
  uint64_t n = 0;
  int width = 2;
  uint64_t windows = 0;
};

struct Dataset {
  std::vector<Shard> shards;
  std::vector<uint64_t> first;      // first[i] = number of windows before shard i
  uint64_t windows = 0, tokens = 0;
  int T = 0;
  std::string error;
  ~Dataset() {
    for (auto& s : shards) {
      if (s.map) munmap(s.map, s.size);
      if (s.fd >= 0) close(s.fd);
    }
  }
};

inline uint64_t mix64(uint64_t x) {      // splitmix64 finaliser
  x += 0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  return x ^ (x >> 31);
}

// A bijection of [0, total): Feistel network on 2*half bits, repeated until the value falls inside the range.
uint64_t permute(uint64_t total, uint64_t seed, uint64_t epoch, uint64_t pos) {
  if (total <= 1) return 0;
  int bits = 1;
  while (bits < 64 && (1ull << bits) < total) bits++;
  const int half = (bits + 1) / 2;
  const uint64_t hm = (1ull << half) - 1;
  const uint64_t key = mix64(seed ^ mix64(epoch + 0x51ED27ull));
  uint64_t x = pos;
  do {
    uint64_t l = x >> half, r = x & hm;
    for (int round = 0; round < 4; round++) {
      const uint64_t f = mix64(r ^ key ^ ((uint64_t)round << 56)) & hm;
      const uint64_t nl = r, nr = l ^ f;
      l = nl;
      r = nr;
    }
    x = (l << half) | r;
  } while (x >= total);       // the walk stays inside the orbit of pos, which contains a value < total (pos itself)
  return x;
}

bool open_shard(Dataset* d, const char* path, int raw_width) {
  Shard s;
  s.fd = open(path, O_RDONLY);
  if (s.fd < 0) { d->error = std::string("cannot open ") + path; return false; }
  struct stat st;
  if (fstat(s.fd, &st) != 0 || st.st_size <= 0) { close(s.fd); d->error = std::string("empty or unreadable: ") + path; return false; }
  s.size = (size_t)st.st_size;
  s.map = mmap(nullptr, s.size, PROT_READ, MAP_PRIVATE, s.fd, 0);
  if (s.map == MAP_FAILED) { close(s.fd); d->error = std::string("mmap failed: ") + path; return false; }
  const uint8_t* p = (const uint8_t*)s.map;
  bool ok = true;
  if (s.size >= 32 && std::memcmp(p, "B2TK", 4) == 0) {
    uint32_t ver, width, flags;
    uint64_t n;
    std::memcpy(&ver, p + 4, 4);
    std::memcpy(&width, p + 8, 4);
    std::memcpy(&flags, p + 12, 4);
    std::memcpy(&n, p + 16, 8);
    if (ver != 1 || (width != 2 && width != 4)) { d->error = std::string("unsupported shard header: ") + path; ok = false; }
    const uint64_t room = s.size - 32;
    if (ok && (n > room / width || ((flags & 1) && n > room - n * width))) { d->error = std::string("shard shorter than its header says: ") + path; ok = false; }
    if (ok) {
      s.width = (int)width;
      s.n = n;
      s.tokens = p + 32;
      s.mask = (flags & 1) ? p + 32 + n * width : nullptr;
    }
  } else if (raw_width == 2 || raw_width == 4) {
    s.width = raw_width;
    s.n = s.size / raw_width;
    s.tokens = p;
  } else {
    d->error = std::string("no shard header (open it as a raw dump by naming the id width): ") + path;
    ok = false;
  }
  if (!ok) { munmap(s.map, s.size); close(s.fd); return false; }
  s.windows = s.n > 0 ? (s.n - 1) / (uint64_t)d->T : 0;
  d->first.push_back(d->windows);
  d->windows += s.windows;
  d->tokens += s.n;
  d->shards.push_back(s);
  return true;
}

// Copies window w into tok / tgt (seq_len ids each).  Returns the number of unmasked targets, -1 when out of range.
int64_t read_window(const Dataset* d, uint64_t w, int64_t* tok, int64_t* tgt) {
  if (w >= d->windows) return -1;
  size_t lo = 0, hi = d->shards.size();
  while (hi - lo > 1) {
    const size_t mid = (lo + hi) / 2;
    if (d->first[mid] <= w) lo = mid; else hi = mid;
  }
  const Shard& s = d->shards[lo];
  const uint64_t at = (w - d->first[lo]) * (uint64_t)d->T;
  const int T = d->T;
  int64_t valid = 0;
  if (s.width == 2) {
    const uint16_t* t = (const uint16_t*)s.tokens + at;
    for (int i = 0; i < T; i++) { tok[i] = t[i]; tgt[i] = t[i + 1]; }
  } else {
    const uint32_t* t = (const uint32_t*)s.tokens + at;
    for (int i = 0; i < T; i++) { tok[i] = t[i]; tgt[i] = t[i + 1]; }
  }
  if (s.mask) {
    const uint8_t* m = s.mask + at + 1;
    for (int i = 0; i < T; i++) {
      if (m[i]) valid++; else tgt[i] = -1;
    }
  } else {
    valid = T;
  }
  return valid;
}

enum SlotState { FREE = 0, FILLING = 1, READY = 2, HELD = 3 };

struct Slot {
  int64_t *tok = nullptr, *tgt = nullptr;
  int state = FREE;
  uint64_t expect = 0;       // the batch this slot takes next
  int64_t valid = 0;
};

struct Loader {
  const Dataset* ds = nullptr;
  int rows = 0, rank = 0, world = 1, shuffle = 1, nthreads = 1;
  uint64_t seed = 0, start = 0, usable = 0;
  std::vector<Slot> slots;
  std::vector<std::thread> workers;
  std::mutex mu;
  std::condition_variable cv;
  uint64_t next_fill = 0, next_take = 0;
  bool stop = false, started = false;
  std::string error;
};

void fill(Loader* L, Slot& s, uint64_t b) {
  const Dataset* d = L->ds;
  const int T = d->T;
  int64_t valid = 0;
  for (int i = 0; i < L->rows; i++) {
    const uint64_t P = b * ((uint64_t)L->world * L->rows) + (uint64_t)i * L->world + L->rank;
    const uint64_t epoch = P / L->usable, idx = P % L->usable;
    const uint64_t w = L->shuffle ? permute(d->windows, L->seed, epoch, idx) : idx;
    valid += read_window(d, w, s.tok + (size_t)i * T, s.tgt + (size_t)i * T);
  }
  s.valid = valid;
}

void worker(Loader* L) {
  for (;;) {
    uint64_t b;
    Slot* s;
    {
      std::unique_lock<std::mutex> lk(L->mu);
      b = L->next_fill++;
      s = &L->slots[(b - L->start) % L->slots.size()];
      L->cv.wait(lk, [&] { return L->stop || (s->state == FREE && s->expect == b); });
      if (L->stop) return;
      s->state = FILLING;
    }
    fill(L, *s, b);
    {
      std::lock_guard<std::mutex> lk(L->mu);
      s->state = READY;
    }
    L->cv.notify_all();
  }
}

}  // namespace

B200_API void* b200_tokds_open(const char** paths, int n_paths, int seq_len, int raw_width) {
  auto* d = new Dataset();
  d->T = seq_len;
  if (seq_len <= 0 || n_paths <= 0) { d->error = "seq_len and the number of shards must be positive"; return d; }
  for (int i = 0; i < n_paths; i++)
    if (!open_shard(d, paths[i], raw_width)) break;
  if (d->error.empty() && d->windows == 0) d->error = "the shards hold less than one window of seq_len + 1 tokens";
  return d;
}
B200_API const char* b200_tokds_error(void* h) { auto* d = (Dataset*)h; return d->error.empty() ? nullptr : d->error.c_str(); }
B200_API uint64_t b200_tokds_windows(void* h) { return ((Dataset*)h)->windows; }
B200_API uint64_t b200_tokds_tokens(void* h) { return ((Dataset*)h)->tokens; }
B200_API void b200_tokds_close(void* h) { delete (Dataset*)h; }
B200_API int64_t b200_tokds_read(void* h, uint64_t window, int64_t* tok, int64_t* tgt) { return read_window((Dataset*)h, window, tok, tgt); }
B200_API uint64_t b200_tokds_permute(uint64_t total, uint64_t seed, uint64_t epoch, uint64_t pos) {
  return pos < total ? permute(total, seed, epoch, pos) : UINT64_MAX;
}

B200_API int b200_tok_shard_write(const char* path, const void* tokens, uint64_t n, int width, const uint8_t* mask) {
  if (width != 2 && width != 4) return -2;
  FILE* f = std::fopen(path, "wb");
  if (!f) return -1;
  uint8_t hdr[32] = {0};
  std::memcpy(hdr, "B2TK", 4);
  const uint32_t ver = 1, w = (uint32_t)width, flags = mask ? 1u : 0u;
  std::memcpy(hdr + 4, &ver, 4);
  std::memcpy(hdr + 8, &w, 4);
  std::memcpy(hdr + 12, &flags, 4);
  std::memcpy(hdr + 16, &n, 8);
  bool ok = std::fwrite(hdr, 1, 32, f) == 32;
  ok = ok && (n == 0 || std::fwrite(tokens, (size_t)width, n, f) == n);
  if (mask) ok = ok && (n == 0 || std::fwrite(mask, 1, n, f) == n);
  ok = (std::fclose(f) == 0) && ok;
  return ok ? 0 : -3;
}

B200_API void* b200_loader_create(void* ds, int rows, int rank, int world, uint64_t seed, uint64_t start_batch, int shuffle, int threads) {
  auto* L = new Loader();
  L->ds = (const Dataset*)ds;
  L->rows = rows; L->rank = rank; L->world = world; L->seed = seed; L->start = start_batch; L->shuffle = shuffle;
  L->nthreads = threads < 1 ? 1 : (threads > 16 ? 16 : threads);
  if (!ds || rows <= 0 || world <= 0 || rank < 0 || rank >= world) { L->error = "bad loader arguments"; return L; }
  const uint64_t per = (uint64_t)rows * world;
  L->usable = L->ds->windows - L->ds->windows % per;
  if (L->usable == 0) L->error = "the data set holds fewer windows than one batch over all ranks";
  L->next_fill = L->next_take = start_batch;
  return L;
}
B200_API const char* b200_loader_error(void* h) { auto* L = (Loader*)h; return L->error.empty() ? nullptr : L->error.c_str(); }
B200_API uint64_t b200_loader_batches_per_epoch(void* h) { auto* L = (Loader*)h; return L->usable / ((uint64_t)L->rows * L->world); }
B200_API int b200_loader_add_slot(void* h, int64_t* tok, int64_t* tgt) {
  auto* L = (Loader*)h;
  if (L->started || !tok || !tgt) return -1;
  Slot s;
  s.tok = tok; s.tgt = tgt;
  s.expect = L->start + L->slots.size();
  L->slots.push_back(s);
  return (int)L->slots.size() - 1;
}
B200_API int b200_loader_start(void* h) {
  auto* L = (Loader*)h;
  if (L->started || !L->error.empty() || L->slots.empty()) return -1;
  L->started = true;
  const int n = L->nthreads < (int)L->slots.size() ? L->nthreads : (int)L->slots.size();   // a worker without a slot would only wait
  for (int i = 0; i < n; i++) L->workers.emplace_back(worker, L);
  return 0;
}
// 0: *slot holds batch *batch (with *valid unmasked targets); 1: nothing ready within timeout_ms; -1: not started.
B200_API int b200_loader_next(void* h, int* slot, uint64_t* batch, int64_t* valid, int timeout_ms) {
  auto* L = (Loader*)h;
  if (!L->started) return -1;
  std::unique_lock<std::mutex> lk(L->mu);
  const uint64_t b = L->next_take;
  Slot& s = L->slots[(b - L->start) % L->slots.size()];
  const bool got = L->cv.wait_for(lk, std::chrono::milliseconds(timeout_ms), [&] { return s.state == READY && s.expect == b; });
  if (!got) return 1;
  s.state = HELD;
  L->next_take++;
  *slot = (int)((b - L->start) % L->slots.size());
  *batch = b;
  *valid = s.valid;
  return 0;
}
B200_API int b200_loader_release(void* h, int slot) {
  auto* L = (Loader*)h;
  {
    std::lock_guard<std::mutex> lk(L->mu);
    if (slot < 0 || slot >= (int)L->slots.size() || L->slots[slot].state != HELD) return -1;
    L->slots[slot].state = FREE;
    L->slots[slot].expect += L->slots.size();
  }
  L->cv.notify_all();
  return 0;
}
B200_API void b200_loader_destroy(void* h) {
  auto* L = (Loader*)h;
  {
    std::lock_guard<std::mutex> lk(L->mu);
    L->stop = true;
  }
  L->cv.notify_all();
  for (auto& t : L->workers) t.join();
  delete L;
}
