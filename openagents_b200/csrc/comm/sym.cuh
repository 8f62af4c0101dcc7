// Device-side view of the symmetric heap: every rank maps every peer's heap (NVLink peer memory)
// and, where NVSwitch multicast is available, one multicast address that reaches all replicas.
// Kernels move data with plain peer loads/stores or `multimem.*` and synchronise through flag
// words in a control block at the start of each heap.  Every wait is bounded; on expiry the
// waiting thread records a status code in the control block and returns.
//
// The reference has no collective layer in-tree (its gradient averaging is a host-side mean:
// apps/openagents.com/workers/api/src/cs336-a1-real-gradient-workload.ts:872-891); the semantics
// kept here are the ones it names for the upstream collectives: a failed collective is reported,
// never left hanging (apps/openagents.com/workers/api/src/training-standby-dispatch.ts:6-12).
#pragma once
#include "../kernels/common.cuh"

namespace b200 {

constexpr int kMaxRanks = 8;
constexpr int kSymChannels = 32;
constexpr size_t kSymControlBytes = 4096;

struct SymControl {               // first kSymControlBytes of every heap
  uint32_t flag[kSymChannels];    // arrival counters, written by peers
  int epoch[kSymChannels];        // barriers completed on the channel (local)
  int ticket[kSymChannels];       // CTAs of the current launch that have finished (local)
  int status;                     // last error (B200Status), 0 if none
  int timeouts;                   // number of waits that ran out
  uint32_t merge_seq;             // arg-max merges this rank has issued so far (local)
  uint32_t row_seq[64];           // per row of the slot all-reduce: all-reduces this rank has done on that row (local)
  uint32_t row_flag[64];          // per row: pushes that have landed here, one per rank and all-reduce (written by peers)
};
constexpr int kSymSlotRows = 64;

struct SymTable {
  int world, rank, use_mc;
  unsigned long long wait_ns;     // bound of a peer wait
  char* base[kMaxRanks];          // heap of each rank as mapped into this process
  char* mc_base;                  // multicast mapping of the heap (null without NVLS)
};

__device__ __forceinline__ SymControl* sym_ctl(const SymTable& T, int r) { return (SymControl*)T.base[r]; }

__device__ __forceinline__ unsigned long long sym_now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// ---- element-wise pushes ------------------------------------------------------------------
// Add `v` into the fp32 word at byte offset `off` of every rank's heap.
__device__ __forceinline__ void sym_red_all_f32(const SymTable& T, size_t off, float v) {
  if (T.use_mc) {
    asm volatile("multimem.red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(T.mc_base + off), "f"(v) : "memory");
  } else {
    for (int p = 0; p < T.world; p++)
      asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(T.base[p] + off), "f"(v) : "memory");
  }
}
__device__ __forceinline__ void sym_red_all_f32x4(const SymTable& T, size_t off, float4 v) {
  if (T.use_mc) {
    asm volatile("multimem.red.relaxed.sys.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(T.mc_base + off), "f"(v.x),
                 "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
  } else {
    for (int p = 0; p < T.world; p++)
      asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(T.base[p] + off), "f"(v.x), "f"(v.y),
                   "f"(v.z), "f"(v.w) : "memory");
  }
}
// Add into one rank's heap only (reduce-scatter towards the owner).
__device__ __forceinline__ void sym_red_to_f32x4(const SymTable& T, int dst, size_t off, float4 v) {
  asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(T.base[dst] + off), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ void sym_red_to_f32(const SymTable& T, int dst, size_t off, float v) {
  asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(T.base[dst] + off), "f"(v) : "memory");
}
// Store one fp32 at `off` of every rank's heap.
__device__ __forceinline__ void sym_st_all_f32(const SymTable& T, size_t off, float v) {
  if (T.use_mc) {
    asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(T.mc_base + off), "f"(v) : "memory");
  } else {
    for (int p = 0; p < T.world; p++)
      asm volatile("st.relaxed.sys.global.f32 [%0], %1;" ::"l"(T.base[p] + off), "f"(v) : "memory");
  }
}
// Store 16 bytes at `off` of every rank's heap (all-gather push).
__device__ __forceinline__ void sym_st_all_v4(const SymTable& T, size_t off, uint4 v) {
  if (T.use_mc) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(T.mc_base + off),
                 "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
                 "f"(__uint_as_float(v.w)) : "memory");
  } else {
    for (int p = 0; p < T.world; p++)
      asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(T.base[p] + off), "r"(v.x), "r"(v.y),
                   "r"(v.z), "r"(v.w) : "memory");
  }
}
// Sum of the fp32x4 at `off` over all ranks (pull).
__device__ __forceinline__ float4 sym_ld_reduce_f32x4(const SymTable& T, size_t off) {
  float4 r;
  if (T.use_mc) {
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(r.x), "=f"(r.y), "=f"(r.z), "=f"(r.w) : "l"(T.mc_base + off) : "memory");
  } else {
    r = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < T.world; p++) {
      float4 v;
      asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                   : "l"(T.base[p] + off) : "memory");
      r.x += v.x; r.y += v.y; r.z += v.z; r.w += v.w;
    }
  }
  return r;
}
// Sum over ranks of eight bf16 values (16 bytes) accumulated in fp32.
__device__ __forceinline__ void sym_ld_reduce_bf16x8(const SymTable& T, size_t off, float (&out)[8]) {
  if (T.use_mc) {
    uint32_t a, b, c, d;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "l"(T.mc_base + off) : "memory");
    const uint32_t w[4] = {a, b, c, d};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const float2 f = __bfloat1622float2(*(const __nv_bfloat162*)&w[i]);
      out[2 * i] = f.x;
      out[2 * i + 1] = f.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; i++) out[i] = 0.f;
    for (int p = 0; p < T.world; p++) {
      uint4 v;
      asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                   : "l"(T.base[p] + off) : "memory");
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const float2 f = __bfloat1622float2(*(const __nv_bfloat162*)&w[i]);
        out[2 * i] += f.x;
        out[2 * i + 1] += f.y;
      }
    }
  }
}

// ---- synchronisation ----------------------------------------------------------------------
// One thread: announce this rank on `ch` to every rank, then wait until every rank has announced
// the same round.  Everything this rank wrote before (by any of its threads that synchronised with
// the caller) is visible to peers that pass the barrier.  Returns false if the wait ran out.
__device__ __forceinline__ bool sym_barrier_thread(const SymTable& T, int ch) {
  SymControl* me = sym_ctl(T, T.rank);
  const int e = me->epoch[ch];
  const uint32_t target = (uint32_t)T.world * (uint32_t)(e + 1);
  __threadfence_system();
  if (T.use_mc) {
    asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(T.mc_base + offsetof(SymControl, flag) + 4 * ch),
                 "r"(1u) : "memory");
  } else {
    for (int p = 0; p < T.world; p++)
      asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(&sym_ctl(T, p)->flag[ch]), "r"(1u) : "memory");
  }
  const unsigned long long t0 = sym_now_ns();
  bool ok = true;
  for (uint32_t spin = 0;; ++spin) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(&me->flag[ch]) : "memory");
    if ((int32_t)(v - target) >= 0) break;
    if ((spin & 63u) == 63u && sym_now_ns() - t0 > T.wait_ns) {
      ok = false;
      break;
    }
  }
  me->epoch[ch] = e + 1;   // advance even on failure so later rounds stay aligned with the peers
  if (!ok) {
    me->status = (int)B200_ERR_TIMEOUT_PEER;
    atomicAdd(&me->timeouts, 1);
  }
  __threadfence_system();
  return ok;
}

// ---- "ready" handshake ---------------------------------------------------------------------
// A kernel that adds into a tensor of every rank (a fused all-reduce) may only start adding once every
// rank has finished reading that tensor's previous contents.  Instead of a stand-alone barrier
// launch between reader and writer, the READER signals when it is done (sym_signal_ready, no wait) and
// the WRITER checks the signals just before its first remote add (sym_wait_ready), by which time they
// have normally long arrived.  One signal per rank per phase; the writer's last CTA closes the phase
// (see sym_kernel_end_barrier).  Channel kSymReadyCh of the control block is reserved for this.
constexpr int kSymReadyCh = 4;

// Call from every thread of every CTA at the end of the reading kernel.
__device__ __forceinline__ void sym_signal_ready(const SymTable& T, int n_ctas) {
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    SymControl* me = sym_ctl(T, T.rank);
    const int done = atomicAdd(&me->ticket[kSymReadyCh], 1);
    if (done == n_ctas - 1) {
      me->ticket[kSymReadyCh] = 0;
      __threadfence_system();
      if (T.use_mc) {
        asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(T.mc_base + offsetof(SymControl, flag) + 4 * kSymReadyCh),
                     "r"(1u) : "memory");
      } else {
        for (int p = 0; p < T.world; p++)
          asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(&sym_ctl(T, p)->flag[kSymReadyCh]), "r"(1u) : "memory");
      }
    }
  }
}

// One thread: wait until every rank has signalled the current phase.  Returns false (and records the
// time-out) if the wait ran out; the caller goes on either way, as after a timed-out barrier.
__device__ __forceinline__ bool sym_wait_ready(const SymTable& T) {
  SymControl* me = sym_ctl(T, T.rank);
  const int e = *(volatile int*)&me->epoch[kSymReadyCh];
  const uint32_t target = (uint32_t)T.world * (uint32_t)(e + 1);
  const unsigned long long t0 = sym_now_ns();
  for (uint32_t spin = 0;; ++spin) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(&me->flag[kSymReadyCh]) : "memory");
    if ((int32_t)(v - target) >= 0) return true;
    if ((spin & 63u) == 63u && sym_now_ns() - t0 > T.wait_ns) {
      me->status = (int)B200_ERR_TIMEOUT_PEER;
      atomicAdd(&me->timeouts, 1);
      return false;
    }
  }
}

// ---- all-gather by push, consumed tile by tile --------------------------------------------------
// Rank r writes its rows of a row-sharded tensor into every rank's full copy (sym_st_all_v4) and then
// bumps counter kSymAgCh0 + r on every rank (sym_signal_rows, called by every thread of every CTA of
// the pushing kernel).  A consumer that needs rows owned by rank r waits until that counter has
// reached the number of all-gathers issued so far (`epoch`, counted by the host, the same on all
// ranks), so it can start on the rows that are already there while the others are still in flight.
constexpr int kSymAgCh0 = 8;   // channels 8 .. 8 + kMaxRanks - 1

__device__ __forceinline__ void sym_signal_rows(const SymTable& T, int n_ctas) {
  // The CTA barrier orders every thread's pushes before thread 0's system-scope fence and release below
  // (release is cumulative), so the threads need no system fence of their own, which would cost each of
  // them a round trip to the peers.
  __syncthreads();
  if (threadIdx.x == 0) {
    SymControl* me = sym_ctl(T, T.rank);
    const int done = atomicAdd(&me->ticket[kSymAgCh0], 1);
    if (done == n_ctas - 1) {
      me->ticket[kSymAgCh0] = 0;
      __threadfence_system();
      const size_t off = offsetof(SymControl, flag) + 4 * (kSymAgCh0 + T.rank);
      if (T.use_mc) {
        asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(T.mc_base + off), "r"(1u) : "memory");
      } else {
        for (int p = 0; p < T.world; p++)
          asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(T.base[p] + off), "r"(1u) : "memory");
      }
    }
  }
}

// One thread: wait until rank `owner` has pushed its rows of all-gather number `epoch`.  Returns false
// (and records the time-out) if the wait ran out.
__device__ __forceinline__ bool sym_wait_rows(const SymTable& T, int owner, uint32_t epoch) {
  SymControl* me = sym_ctl(T, T.rank);
  const unsigned long long t0 = sym_now_ns();
  for (uint32_t spin = 0;; ++spin) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(&me->flag[kSymAgCh0 + owner]) : "memory");
    if ((int32_t)(v - epoch) >= 0) return true;
    if ((spin & 63u) == 63u && sym_now_ns() - t0 > T.wait_ns) {
      me->status = (int)B200_ERR_TIMEOUT_PEER;
      atomicAdd(&me->timeouts, 1);
      return false;
    }
  }
}

// ---- one-shot all-reduce through per-rank slots -------------------------------------------------
// Decode-time row-parallel projections (a few tokens to a batch of 64) leave their partial result in LOCAL memory,
// at full single-GPU speed; the kernel that needs the sum (the RMSNorm that follows) is the all-reduce: its CTA for
// row t pushes this rank's partial row into slot (parity, rank, t) of a [2][world][rows][d] fp32 tensor on every rank
// (multimem.st / peer stores, 16 bytes per lane), raises row_flag[t] everywhere with one system-scope release,
// waits until the world has done the same, and adds the slots up in rank order, so every replica computes
// bit-identical sums.  There is no barrier, no cross-CTA ticket and no "ready" handshake: rows are independent, the
// sequence number of a row lives in device memory (so the scheme replays unchanged inside a CUDA graph), slot parity
// alternates with it, and a rank can only write parity p of a row again after it has consumed the all-reduce in
// between, to which every peer contributed after it had finished reading parity p.
constexpr int kSymMergeCh0 = 24;   // flag channels 24 .. 24 + kMaxRanks - 1: arg-max merge

// Thread 0 of the CTA that owns row t, after a CTA barrier that follows the CTA's pushes: publish them.
__device__ __forceinline__ void sym_row_signal(const SymTable& T, int t) {
  const size_t off = offsetof(SymControl, row_flag) + 4 * (size_t)t;
  if (T.use_mc) {
    asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(T.mc_base + off), "r"(1u) : "memory");
  } else {
    for (int p = 0; p < T.world; p++)
      asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(T.base[p] + off), "r"(1u) : "memory");
  }
}
// One thread: wait until every rank's push number `seq` of row t has landed here.  Returns false (and records the
// time-out) if the wait ran out.
__device__ __forceinline__ bool sym_row_wait(const SymTable& T, int t, uint32_t seq) {
  SymControl* me = sym_ctl(T, T.rank);
  const uint32_t target = (uint32_t)T.world * seq;
  const unsigned long long t0 = sym_now_ns();
  for (uint32_t spin = 0;; ++spin) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(&me->row_flag[t]) : "memory");
    if ((int32_t)(v - target) >= 0) return true;
    if ((spin & 63u) == 63u && sym_now_ns() - t0 > T.wait_ns) {
      me->status = (int)B200_ERR_TIMEOUT_PEER;
      atomicAdd(&me->timeouts, 1);
      return false;
    }
  }
}
// One thread: wait until flag `ch` of this rank has reached `seq`.  Returns false (and records the
// time-out) if the wait ran out.
__device__ __forceinline__ bool sym_wait_flag(const SymTable& T, int ch, uint32_t seq) {
  SymControl* me = sym_ctl(T, T.rank);
  const unsigned long long t0 = sym_now_ns();
  for (uint32_t spin = 0;; ++spin) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(&me->flag[ch]) : "memory");
    if ((int32_t)(v - seq) >= 0) return true;
    if ((spin & 63u) == 63u && sym_now_ns() - t0 > T.wait_ns) {
      me->status = (int)B200_ERR_TIMEOUT_PEER;
      atomicAdd(&me->timeouts, 1);
      return false;
    }
  }
}

// Call from every thread of every CTA at the end of a kernel that pushed data to peers: the CTA that
// finishes last runs the cross-rank barrier, so when the kernel completes, every rank's pushes have
// landed everywhere.  No CTA waits for another CTA.  `close_ready_phase`: this kernel consumed one
// phase of the ready handshake (every CTA has read the phase number by now).
__device__ __forceinline__ void sym_kernel_end_barrier(const SymTable& T, int ch, int n_ctas, bool close_ready_phase = false) {
  __shared__ int s_is_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    SymControl* me = sym_ctl(T, T.rank);
    const int done = atomicAdd(&me->ticket[ch], 1);
    s_is_last = (done == n_ctas - 1);
    if (s_is_last) {
      me->ticket[ch] = 0;
      if (close_ready_phase) me->epoch[kSymReadyCh] += 1;
      __threadfence();
      sym_barrier_thread(T, ch);
    }
  }
  __syncthreads();
}

}  // namespace b200
