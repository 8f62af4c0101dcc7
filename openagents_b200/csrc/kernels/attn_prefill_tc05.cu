// Causal grouped-query flash attention for prefill on the 5th-generation tensor cores (head dim 128).
//
// One CTA = 128 query rows of one head.  Roles: warps 0 and 10 are the TMA producers (a ring of K / V
// blocks of 64 keys gathered page by page from the paged fp16 cache), warps 1 and 11 issue the two
// kinds of tcgen05.mma, warps 2..9 do the online softmax: two warps per 32 query rows (the two share a tensor-memory lane
// quarter), one taking keys 0..63 of a block and output columns 0..63, the other the rest; they swap
// their partial row maxima through shared memory once per block.  Two warps per scheduler is what
// hides the latencies of tensor-memory loads, exponentials and barriers.  Per key block j:
//   S_j = Q K_j^T        tcgen05.mma 128 x 128 x 128 into one of two S accumulators in tensor memory
//   softmax              S_j -> registers (tcgen05.ld), mask, running max / sum, P_j (fp16 pairs) -> tensor
//                        memory over the S columns it came from, where the next MMA reads it as its A operand
//   O += P_j V_j         tcgen05.mma 128 x 128 x 128 accumulating in ONE O tile that stays in tensor memory
//                        for the whole row block, V taken as it lies in the cache ([key][dim], i.e. the
//                        MN-major form of the B operand)
// The exponent offset of a row (its running maximum) is only moved when the maximum has grown by more
// than 8 (a factor 256, well inside fp16 for P and fp32 for O and the row sum); then the row's owner
// thread rescales the O row in tensor memory (tcgen05.ld / st) between two PV products.  After the
// first key blocks of a causal row that is rare, so the steady state has no O traffic at all.
// Sliding windows, learned sink logits and a context that is longer than the chunk (chunked prefill,
// prefix reuse) are handled by the mask and the block range.  Math as in the reference's attention
// (apps/openagents.com/workers/api/src/cs336-a1-real-gradient-workload.ts:478-518: max-subtract,
// exp, normalise).  Every wait is bounded; a wait that runs out sets the status word and the CTA
// leaves through the common exit, which frees its tensor memory.
#include "tc05.cuh"

using namespace b200;
using namespace b200::tc;

namespace {

constexpr int QB = 128, KB = 128, HD = 128, KV_STAGES = 3;
constexpr int K_BYTES = KB * HD * 2;            // 16 KB: two halves of [64 keys][64 dims]
constexpr uint32_t TMEM_COLS = 512;             // S: 2 x 128 (P is written over the S columns it came from), O: 128, Q: 64
constexpr float kRescaleStep = 8.f;             // log2 units
constexpr float kLog2e = 1.4426950408889634f;

struct PrefillArgs {
  const int* page_table;   // [n_seqs][max_pages]
  const int* q_start;      // [n_seqs]
  const int* q_len;        // [n_seqs]
  const int* ctx_len;      // [n_seqs]
  const float* sinks;      // [Hq] or null
  __nv_bfloat16* out;      // [T_total][Hq * HD]
  int* status;
  const __half* q;         // [T_total][Hq * HD], rotated and scaled
  int max_pages, Hq, Hkv, window, T_total;
};

// fp16 x fp16 -> fp32 instruction descriptor; b_mn: the B operand is MN-major.
__host__ __device__ constexpr uint32_t idesc_f16(int M, int N, bool b_mn) {
  return (1u << 4) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// D (tensor memory) (+)= A (tensor memory: lane = row, 32-bit column j = elements 2j, 2j + 1 of the K slice) x B (shared
// memory descriptor).  An A operand in shared memory costs a 128-row x 32-byte read per instruction whatever N
// is, which is what bounds MMAs with a narrow N; from tensor memory it does not.
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__global__ void __launch_bounds__(384, 1) attn_prefill_tc05_kernel(                                                                    const __grid_constant__ CUtensorMap tmK,
                                                                    const __grid_constant__ CUtensorMap tmV,
                                                                    const PrefillArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sKV = smem;                                    // KV_STAGES x (K, V)
  uint64_t* bars = (uint64_t*)(sKV + KV_STAGES * 2 * K_BYTES);
  uint64_t* q_full = bars;                                // [1]
  uint64_t* kv_full = bars + 1;                           // [KV_STAGES]
  uint64_t* kv_empty = kv_full + KV_STAGES;               // [KV_STAGES]
  uint64_t* s_full = kv_empty + KV_STAGES;                // [2]
  uint64_t* s_empty = s_full + 2;                         // [2]
  uint64_t* p_full = s_empty + 2;                         // [2]
  uint64_t* pv_done = p_full + 2;                         // [2]: PV product of the blocks that used P buffer b
  uint64_t* x_full = pv_done + 2;                          // [4 quarters][2]: both warps of a pair have posted their half
  uint32_t* tmem_holder = (uint32_t*)(x_full + 8);
  volatile int* abort_flag = (volatile int*)(tmem_holder + 1);
  float* xch = (float*)(bars + 32);                       // [2 (block parity)][2 (half)][128 rows] partial row maxima / sums

  const int seq = blockIdx.z, h = blockIdx.y, qb = gridDim.x - 1 - blockIdx.x;   // longest (latest) query blocks first
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(q_full), 4);
    for (int s = 0; s < KV_STAGES; s++) {
      mbar_init(smem_u32(kv_full + s), 1);
      mbar_init(smem_u32(kv_empty + s), 1);
    }
    for (int s = 0; s < 2; s++) {
      mbar_init(smem_u32(s_full + s), 1);
      mbar_init(smem_u32(s_empty + s), 8);
      mbar_init(smem_u32(p_full + s), 8);
    }
    mbar_init(smem_u32(pv_done), 1);
    mbar_init(smem_u32(pv_done + 1), 1);
    for (int s = 0; s < 8; s++) mbar_init(smem_u32(x_full + s), 2);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  pdl_trigger();
  pdl_wait();

  const int qlen = a.q_len[seq];
  const int q0 = qb * QB;
  const bool live = q0 < qlen;            // a dead CTA still goes through the common exit (it holds tensor memory)
  const int ctx = a.ctx_len[seq], qs = a.q_start[seq];
  const int kh = h / (a.Hq / a.Hkv);
  const int pos0 = ctx - qlen + q0;       // absolute position of this CTA's first query row
  const int k_hi = min(ctx, pos0 + QB);   // keys [k_lo, k_hi) can matter to some row
  const int k_lo = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
  const int jb0 = k_lo / KB, jb1 = live ? (k_hi + KB - 1) / KB : jb0;   // key blocks [jb0, jb1)
  const int nb = jb1 - jb0;
  const uint32_t S_T = tmem_base, O_T = tmem_base + 256;   // S buffers at +0, +128; O at +256
  const uint32_t Q_T = tmem_base + 384;                    // Q (fp16 pairs, 64 columns)
  // P_j (fp16 pairs) overwrites S_j: the warp that owns keys [64 h, 64 h + 64) of a block writes columns [64 h, 64 h + 32)

  // Four single-thread roles, each in a warp of its own, because what a thread can issue is the bound here:
  // about 55 cycles per tcgen05.mma and 100-200 per TMA load, barrier wait, fence or commit.
  //   warp 0: K loads (and the byte count of the whole stage)      warp 10: V loads
  //   warp 1: S_j = Q K_j^T                                         warp 11: O += P_j V_j, releases the stage
  if (warp == 0 || warp == 10) {
    if (lane == 0 && nb > 0) {
      const bool is_k = warp == 0;
      const int* pt = a.page_table + (size_t)seq * a.max_pages;
      for (int j = 0; j < nb; j++) {
        const int s = j % KV_STAGES;
        const uint32_t ph = (j / KV_STAGES) & 1;
        if (!mbar_wait(smem_u32(kv_empty + s), ph ^ 1, abort_flag)) break;
        const uint32_t bar = smem_u32(kv_full + s);
        // the barrier holds one pending arrival until this arrive.expect_tx, so V bytes that land first cannot
        // complete the phase early
        if (is_k) mbar_expect_tx(bar, 2 * K_BYTES);
        uint8_t* dst = sKV + (size_t)s * 2 * K_BYTES + (is_k ? 0 : K_BYTES);
        const CUtensorMap* tm = is_k ? &tmK : &tmV;
#pragma unroll
        for (int p = 0; p < KB / 16; p++) {
          const int pi = (jb0 + j) * (KB / 16) + p;
          const int page = (pi * 16 < ctx) ? pt[pi] : 0;          // pages past the context are masked anyway
          const int row = (page * a.Hkv + kh) * 16;
#pragma unroll
          for (int hf = 0; hf < 2; hf++) tma_load_2d(smem_u32(dst + hf * (K_BYTES / 2) + p * 2048), tm, bar, hf * 64, row);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && nb > 0) {
      constexpr uint32_t idesc_s = idesc_f16(QB, KB, false);
      bool ok = mbar_wait(smem_u32(q_full), 0, abort_flag);
      for (int j = 0; j < nb && ok; j++) {
        const int s = j % KV_STAGES, b = j & 1;
        if (!mbar_wait(smem_u32(kv_full + s), (j / KV_STAGES) & 1, abort_flag)) break;
        if (!mbar_wait(smem_u32(s_empty + b), ((j >> 1) & 1) ^ 1, abort_flag)) break;
        if (j >= 2 && !mbar_wait(smem_u32(pv_done + b), ((j - 2) >> 1) & 1, abort_flag)) break;   // P_{j-2} sits in S buffer b
        tc_fence_after();
        const uint32_t ka = smem_u32(sKV + (size_t)s * 2 * K_BYTES);
#pragma unroll
        for (int kk = 0; kk < HD / 16; kk++)
          umma_ts(S_T + b * KB, Q_T + 8 * kk, smem_desc_sw128(ka + (kk >> 2) * (K_BYTES / 2)) + 2 * (kk & 3), idesc_s,
                  kk != 0 ? 1u : 0u);
        umma_commit(smem_u32(s_full + b));
      }
    }
  } else if (warp == 11) {
    if (lane == 0 && nb > 0) {
      constexpr uint32_t idesc_o = idesc_f16(QB, HD, true);
      for (int j = 0; j < nb; j++) {
        const int s = j % KV_STAGES, b = j & 1;
        if (!mbar_wait(smem_u32(kv_full + s), (j / KV_STAGES) & 1, abort_flag)) break;       // V_j has landed
        if (!mbar_wait(smem_u32(p_full + b), (j >> 1) & 1, abort_flag)) break;                // P_j written, O rows rescaled if needed
        tc_fence_after();
        const uint32_t va = smem_u32(sKV + (size_t)s * 2 * K_BYTES + K_BYTES);
#pragma unroll
        for (int kk = 0; kk < KB / 16; kk++)
          umma_ts(O_T, S_T + b * KB + (kk >> 2) * 64 + 8 * (kk & 3), smem_desc_sw128_mn(va + kk * 2048, K_BYTES / 2), idesc_o,
                  (j != 0 || kk != 0) ? 1u : 0u);
        // a commit covers this thread's MMAs only; S_j is known to be done because the softmax of block j needed it
        umma_commit(smem_u32(pv_done + b));
        umma_commit(smem_u32(kv_empty + s));
      }
    }
  } else if (warp < 10 && nb > 0) {
    const int q = warp & 3;                      // tensor-memory lane quarter this warp may read
    const int hsel = (warp - 2) >> 2;            // 0: keys 0..31 of a block, output columns 0..63; 1: the other half
    const int row = q * 32 + lane;               // query row of this thread (shared with the partner warp's same lane)
    const int qpos = pos0 + row;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    constexpr int HK = KB / 2, HO = HD / 2;
    float m_used = -INFINITY, l = 0.f;     // exponent offset of this row (log2 units) and this warp's part of the row sum
    bool ok = true;
    // post this warp's half and wait (bounded, like every wait here) for the partner's; use number `u` of buffer `bb`
    if (hsel == 0) {
      // This row of Q (fp16, already rotated and scaled) goes to tensor memory once: column j = dims 2j, 2j + 1.
      const bool in = qs + q0 + row < a.T_total;
      const uint4* qrow = (const uint4*)(a.q + ((size_t)(qs + q0 + (in ? row : 0)) * a.Hq + h) * HD);
#pragma unroll
      for (int c = 0; c < 2; c++) {
        uint32_t r[32];
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const uint4 v = in ? qrow[c * 8 + i] : make_uint4(0u, 0u, 0u, 0u);
          r[4 * i] = v.x; r[4 * i + 1] = v.y; r[4 * i + 2] = v.z; r[4 * i + 3] = v.w;
        }
        tmem_st32(Q_T + lane_addr + c * 32, r);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(q_full));
    }
    auto pair_sync = [&](int bb, int u) -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(x_full + q * 2 + bb));
      bool k = mbar_wait(smem_u32(x_full + q * 2 + bb), (uint32_t)u & 1, abort_flag);
      return __all_sync(0xffffffffu, k && !*abort_flag);
    };

    for (int j = 0; j < nb; j++) {
      const int b = j & 1;
      ok = mbar_wait(smem_u32(s_full + b), (j >> 1) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok && !*abort_flag);
      if (!ok) break;
      tc_fence_after();
      float sv[HK];
      {
        uint32_t r[32];
#pragma unroll
        for (int c = 0; c < HK / 32; c++) {
          tmem_ld32(S_T + b * KB + lane_addr + hsel * HK + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i++) sv[c * 32 + i] = __uint_as_float(r[i]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(s_empty + b));
      // mask, maximum of this half, swap with the partner warp
      const int kb0 = (jb0 + j) * KB;
      const bool edge = kb0 + KB - 1 > pos0 || kb0 + KB > ctx || (a.window > 0 && kb0 < pos0 + QB - a.window);
      if (edge) {
#pragma unroll
        for (int i = 0; i < HK; i++) {
          const int kp = kb0 + hsel * HK + i;
          if (kp > qpos || kp >= ctx || (a.window > 0 && kp <= qpos - a.window)) sv[i] = -INFINITY;
        }
      }
      float mx0 = fmaxf(sv[0], sv[1]), mx1 = fmaxf(sv[2], sv[3]);
#pragma unroll
      for (int i = 4; i < HK; i += 4) {
        mx0 = max3(mx0, sv[i], sv[i + 1]);
        mx1 = max3(mx1, sv[i + 2], sv[i + 3]);
      }
      float* xb = xch + b * 256;
      xb[hsel * 128 + row] = fmaxf(mx0, mx1);
      ok = pair_sync(b, j >> 1);
      if (!ok) break;
      const float bmax = fmaxf(fmaxf(mx0, mx1), xb[(hsel ^ 1) * 128 + row]) * kLog2e;
      // move the exponent offset only when it is far behind (or not set yet); both warps of a pair decide alike
      const bool unset = m_used == -INFINITY;
      const bool behind = bmax > m_used + kRescaleStep;          // false while bmax is -inf
      if (j > 0 && __any_sync(0xffffffffu, behind && !unset)) {
        const float m_new = fmaxf(m_used, bmax);
        const float scale = (m_new == -INFINITY) ? 1.f : ex2_approx(m_used - m_new);
        ok = mbar_wait(smem_u32(pv_done + ((j - 1) & 1)), ((j - 1) >> 1) & 1, abort_flag);       // PV_{j-1} has finished
        ok = __all_sync(0xffffffffu, ok && !*abort_flag);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < HO / 32; c++) {
          uint32_t r[32];
          tmem_ld32(O_T + lane_addr + hsel * HO + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i++) r[i] = __float_as_uint(__uint_as_float(r[i]) * scale);
          tmem_st32(O_T + lane_addr + hsel * HO + c * 32, r);
        }
        tmem_st_wait();
        tc_fence_before();
        l *= scale;
        m_used = m_new;
      } else if (unset) {
        m_used = bmax;                             // nothing accumulated yet under the old offset (O row and l are zero)
      }
      const float off = (m_used == -INFINITY) ? 0.f : m_used;
      float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
      // P row (fp16 pairs) straight into tensor memory, where the PV product reads it as its A operand:
      // this warp's 64 keys become 32 columns at the start of its own half of S buffer b
      uint32_t pw[HK / 2];
#pragma unroll
      for (int i = 0; i < HK / 2; i++) {
        const float p0 = ex2_approx(fmaf(sv[2 * i], kLog2e, -off)), p1 = ex2_approx(fmaf(sv[2 * i + 1], kLog2e, -off));
        if (i & 1) { sum2 += p0; sum3 += p1; } else { sum0 += p0; sum1 += p1; }
        const __half2 hh = __floats2half2_rn(p0, p1);
        pw[i] = *(const uint32_t*)&hh;
      }
      // (S buffer b is free for P_j: S_j was only issued once PV_{j-2}, the last reader of these columns, had finished)
      tmem_st32(S_T + b * KB + lane_addr + hsel * HK, pw);
      tmem_st_wait();
      l += (sum0 + sum1) + (sum2 + sum3);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(p_full + b));
    }
    if (ok) {
      ok = mbar_wait(smem_u32(pv_done + ((nb - 1) & 1)), ((nb - 1) >> 1) & 1, abort_flag);          // last PV product
      ok = __all_sync(0xffffffffu, ok && !*abort_flag);
    }
    // row sum = both halves (the partner is at the same point: every exit above is taken by whole CTAs' worth of
    // warps only through the abort flag, in which case nothing is written)
    if (__all_sync(0xffffffffu, ok)) {
      float* xl = xch + (nb & 1) * 256;            // the buffer the last block did not use
      xl[hsel * 128 + row] = l;
      ok = pair_sync(nb & 1, nb >> 1);
      l += xl[(hsel ^ 1) * 128 + row];
      tc_fence_after();
      if (a.sinks) l += (m_used == -INFINITY) ? 1.f : ex2_approx(a.sinks[h] * kLog2e - m_used);
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const bool wr = ok && row < qlen - q0;
      __nv_bfloat16* dst = a.out + (size_t)(qs + q0 + row) * a.Hq * HD + (size_t)h * HD + hsel * HO;
#pragma unroll
      for (int c = 0; c < HO / 32; c++) {
        uint32_t r[32];
        tmem_ld32(O_T + lane_addr + hsel * HO + c * 32, r);
        tmem_ld_wait();
        if (wr) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 v;
            __nv_bfloat162* p = (__nv_bfloat162*)&v;
#pragma unroll
            for (int k = 0; k < 4; k++)
              p[k] = __floats2bfloat162_rn(__uint_as_float(r[i + 2 * k]) * inv, __uint_as_float(r[i + 2 * k + 1]) * inv);
            *(uint4*)(dst + c * 32 + i) = v;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
  if (threadIdx.x == 0 && *abort_flag && a.status) atomicExch(a.status, (int)B200_ERR_TIMEOUT_MMA);
}

}  // namespace

// q fp16 [T_total][Hq * 128] (rotated, pre-scaled by 1/sqrt(128)); kc / vc fp16 [n_pages][Hkv][16][128];
// out bf16 [T_total][Hq * 128].  Sequences as in b200_attn_prefill; max_q = longest chunk.
B200_API int b200_attn_prefill_tc05(const void* q, const void* kc, const void* vc, const int* page_table, int max_pages,
                                    int n_pages, const int* q_start, const int* q_len, const int* ctx_len, int n_seqs,
                                    int max_q, int T_total, int Hq, int Hkv, int window, const float* sinks, void* out,
                                    int* status, cudaStream_t st) {
  if (Hq % Hkv || n_seqs < 1 || max_q < 1 || !page_table) return B200_ERR_BAD_ARG;
  CUtensorMap tk, tv;
  int rc;
  const uint64_t rows = (uint64_t)n_pages * Hkv * 16;
  rc = make_tmap_2d(&tk, kc, 2, rows, HD, (uint64_t)HD * 2, 16, 64, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tv, vc, 2, rows, HD, (uint64_t)HD * 2, 16, 64, true);
  if (rc) return rc;
  PrefillArgs a;
  a.q = (const __half*)q; a.T_total = T_total;
  a.page_table = page_table; a.q_start = q_start; a.q_len = q_len; a.ctx_len = ctx_len; a.sinks = sinks;
  a.out = (__nv_bfloat16*)out; a.status = status; a.max_pages = max_pages; a.Hq = Hq; a.Hkv = Hkv; a.window = window;
  constexpr size_t smem = 1024 + KV_STAGES * 2 * K_BYTES + 32 * 8 + 2 * 2 * 128 * 4;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  dim3 grid((max_q + QB - 1) / QB, Hq, n_seqs);
  return launch_pdl(attn_prefill_tc05_kernel, grid, dim3(384), smem, st, tk, tv, a);
}
