// Quantized-weight GEMM for decode batches (up to 64 tokens per tile) on tcgen05 with the
// dequantization inside the pipeline:
//     Y[t][n] (+)= sum_k X[t][k] * W[n][k],   W in Q4_K-R or Q6_K-R (row-major packed), X bf16.
// The packed weights are read from HBM exactly once, in their 4.5- or 6.6-bit form; nothing keeps a
// bf16 copy of them.
//
// The weight tile is the MMA's M operand (128 weight rows), the tokens are its N operand (64), so a
// decode batch fills the 128-lane accumulator without padding.  A persistent CTA (one per SM) walks
// work items (128-row tile, K split) with a ring of stages of one superblock (256 of K) each:
//   warp 0      one thread: TMA loads of the raw packed superblocks (128 rows x 144 / 208 bytes)
//   warp 1      one thread: tcgen05.mma, TS form: the expanded weights are the A operand in TENSOR
//               MEMORY, the activations the B operand in shared memory; owns the allocation
//   warp 2      one thread: TMA loads of the activation tiles (from L2; they are a few hundred KB)
//   warps 4-11  expansion: a thread owns one weight row (= one tensor-memory lane) and two 64-wide K
//               blocks of every stage: one mask puts two adjacent 4-bit values into the mantissas of
//               a bf16 pair, one subtraction and one fma apply the sub-block scale and offset, and
//               tcgen05.st writes the 64 values where the MMA reads them, with no shared-memory round
//               trip, no swizzle arithmetic and no proxy fence.  The same warps run the epilogue of
//               item i after they have expanded the first stage of item i + 1 (two accumulators).
// Each scheduler of the SM hosts one single-thread role warp and two expansion warps: the role threads run
// dependent instruction chains and fall behind when they have to share their scheduler with more busy warps
// (measured: with sixteen expansion warps the MMA thread needed 1400 cycles to issue a stage's sixteen MMAs),
// which is also why the issuing loop below works on precomputed descriptor words.
// Stages hand over through mbarriers; every wait is bounded and reports through `status`.
//
// Epilogues: plain store (fp32 and/or bf16), accumulation with vector `red` (K may be split; under tensor
// parallelism the row-parallel projections accumulate this rank's partial result that way and the RMSNorm
// that follows all-reduces it) and SwiGLU over interleaved (gate, up) rows.
//
// GEMM-shaped reference math: apps/openagents.com/workers/api/src/cs336-a2-benchmark-workload.ts:251-292;
// the quantized formats are the ones the reference serves (docs/muse/muse-glimmer.md:112).
#include "tc05.cuh"

using namespace b200;
using namespace b200::tc;

enum { QW_Q4KR = 0, QW_Q6KR = 1 };
enum { QEPI_STORE = 0, QEPI_ADD = 1, QEPI_SWIGLU = 2 };

struct QGemmArgs {
  const __half* w2;      // Q6_K-R: fp16 d per (row, superblock); unused for Q4_K-R
  float* out_f32;        // [T][ldo] (STORE / ADD), or null
  __nv_bfloat16* out_bf16;   // [T][ldo] (STORE) or [T][ldo] with N / 2 live columns (SWIGLU), or null
  const float* bias;     // [N] in the row order of W, or null (applied by K split 0)
  int ldo, T, N, K;
  int epi;
  int splits, sb_per_split, n_items;
  int* status;
};

__device__ __forceinline__ uint32_t bf162_as_u32(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __nv_bfloat162 u32_as_bf162(uint32_t v) { return *reinterpret_cast<__nv_bfloat162*>(&v); }

__device__ __forceinline__ uint32_t pack2(float lo, float hi) { return bf162_as_u32(__floats2bfloat162_rn(lo, hi)); }

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
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// D (tensor memory) (+)= A (tensor memory: lane = row, 32-bit column j = elements 2j, 2j + 1 of the K slice)
// x B (shared-memory descriptor).
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Q4_K-R: one 32-element sub-block (4 words, word w = elements 8w .. 8w + 7, element i at bit
// 4 (i / 2) + 16 (i % 2)) -> 16 words of bf16 pairs.  The nibble sits in the mantissa of bf16 16.0 (one shift and
// one lop3 for two weights); (16 + q) - 24 = q - 8 is exact, and value = a * (q - 8) + c with c = 8 a - min keeps
// the constant small (the sub-block's range is roughly centred on it), so rounding a and c to bf16 costs no more
// than rounding the weight itself does.
__device__ __forceinline__ void expand_q4k(__nv_bfloat162 A2, __nv_bfloat162 C2, const uint4 q, uint32_t* out) {
  const __nv_bfloat162 off = __halves2bfloat162(__float2bfloat16(24.f), __float2bfloat16(24.f));
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const uint32_t v = w[i];
    const uint32_t t0 = ((v << 3) & 0x00780078u) | 0x41804180u;
    const uint32_t t1 = ((v >> 1) & 0x00780078u) | 0x41804180u;
    const uint32_t t2 = ((v >> 5) & 0x00780078u) | 0x41804180u;
    const uint32_t t3 = ((v >> 9) & 0x00780078u) | 0x41804180u;
    out[4 * i + 0] = bf162_as_u32(__hfma2(__hsub2(u32_as_bf162(t0), off), A2, C2));
    out[4 * i + 1] = bf162_as_u32(__hfma2(__hsub2(u32_as_bf162(t1), off), A2, C2));
    out[4 * i + 2] = bf162_as_u32(__hfma2(__hsub2(u32_as_bf162(t2), off), A2, C2));
    out[4 * i + 3] = bf162_as_u32(__hfma2(__hsub2(u32_as_bf162(t3), off), A2, C2));
  }
}

// Q6_K-R: 6-bit value = nibble | two high bits; (64 + q) - 96 = q - 32 is exact in bf16.  `ss` holds
// the two bf16 scales of the sub-block (first and second 16 elements).
__device__ __forceinline__ void expand_q6k(const uint4 lo, const uint2 tw, uint32_t ss, uint32_t* out) {
  const __nv_bfloat162 sv = u32_as_bf162(ss);
  const __nv_bfloat162 off = __halves2bfloat162(__float2bfloat16(96.f), __float2bfloat16(96.f));
  const uint32_t w[4] = {lo.x, lo.y, lo.z, lo.w};
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const uint32_t v = w[i];
    const uint32_t T = (i < 2 ? tw.x : tw.y) >> (4 * (i & 1));
    const __nv_bfloat162 S2 = i < 2 ? __halves2bfloat162(sv.x, sv.x) : __halves2bfloat162(sv.y, sv.y);
    const uint32_t q0 = (v & 0x000F000Fu) | ((T & 0x00030003u) << 4);
    const uint32_t q1 = ((v >> 4) & 0x000F000Fu) | (((T >> 2) & 0x00030003u) << 4);
    const uint32_t q2 = ((v >> 8) & 0x000F000Fu) | (((T >> 8) & 0x00030003u) << 4);
    const uint32_t q3 = ((v >> 12) & 0x000F000Fu) | (((T >> 10) & 0x00030003u) << 4);
    out[4 * i + 0] = bf162_as_u32(__hmul2(__hsub2(u32_as_bf162((q0 << 1) | 0x42804280u), off), S2));
    out[4 * i + 1] = bf162_as_u32(__hmul2(__hsub2(u32_as_bf162((q1 << 1) | 0x42804280u), off), S2));
    out[4 * i + 2] = bf162_as_u32(__hmul2(__hsub2(u32_as_bf162((q2 << 1) | 0x42804280u), off), S2));
    out[4 * i + 3] = bf162_as_u32(__hmul2(__hsub2(u32_as_bf162((q3 << 1) | 0x42804280u), off), S2));
  }
}

constexpr int QBM = 128, QBN = 64, QSB = 256;      // weight rows per tile, tokens per tile, K per stage
constexpr int kRoleWarps = 4;                      // raw loads, MMA, activation loads, one idle (keeps warp % 4 = lane quarter)
constexpr int kDqWarps = 8;                        // expansion warps: lane quarter = warp & 3, K half = (warp - 4) >> 2
constexpr int kQThreads = 32 * (kRoleWarps + kDqWarps);
constexpr int kXStage = 4 * QBN * 64 * 2;          // four 64-wide K blocks of activations: 32 KB
constexpr int kAS = 3;                             // operand stages in tensor memory (and activation stages in shared memory)
// Every CTA walks the K range of its item from a different starting superblock (rotated by the CTA index): at any
// moment the SMs then read different slices of the activations, instead of all of them pulling the same few L2 lines.
__device__ __forceinline__ int rot_sb(int sb0, int sb1, int i) { const int n = sb1 - sb0; return sb0 + (i + (int)blockIdx.x) % n; }

// Build with -DQGEMM_STAMPS to have CTA 0's MMA thread add up, over all launches: [0] cycles spent waiting for operands,
// [1] cycles spent issuing, [2] cycles from an item's first stage to the retirement of its last, [3] stages counted in [2].
// `b200_qgemm_stamps(out, reset)` copies the four counters out.  Not compiled by default.
#ifdef QGEMM_STAMPS
__device__ long long g_qgemm_stamps[4];
#define QSTAMP_T0() long long _qs = clock64()
#define QSTAMP_ADD(i) do { const long long _qn = clock64(); if (blockIdx.x == 0) g_qgemm_stamps[i] += _qn - _qs; _qs = _qn; } while (0)
#else
#define QSTAMP_T0() do { } while (0)
#define QSTAMP_ADD(i) do { } while (0)
#endif

template <int WT> struct QTraits { static constexpr int RAWB = WT == QW_Q4KR ? 144 : 208; static constexpr int RS = WT == QW_Q4KR ? 6 : 4; };

// tcgen05.mma (TS form) with the shared-memory descriptor given as its two 32-bit halves: the issuing thread adds
// block offsets to the low word only (the 14-bit address field cannot carry out of it), one instruction per MMA.
__device__ __forceinline__ void umma_ts_lohi(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 bd;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 bd, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], bd, %4, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <int WT>
__global__ void __launch_bounds__(kQThreads, 1) qgemm_kernel(const __grid_constant__ CUtensorMap tmW,
                                                             const __grid_constant__ CUtensorMap tmX, const QGemmArgs a) {
  constexpr int RAWB = QTraits<WT>::RAWB, RS = QTraits<WT>::RS;
  constexpr int RAW_BYTES = QBM * RAWB;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sX = smem;                               // kAS stages of activations, 128-byte swizzle
  uint8_t* sR = sX + kAS * kXStage;                 // RS raw packed stages
  uint64_t* bars = (uint64_t*)(sR + RS * RAW_BYTES);
  uint64_t* raw_full = bars;             // [RS]  TMA bytes landed
  uint64_t* raw_empty = raw_full + RS;   // [RS]  every expansion warp has read the stage
  uint64_t* x_full = raw_empty + RS;     // [kAS]
  uint64_t* a_full = x_full + kAS;       // [kAS] every expansion warp has written its part of the operand
  uint64_t* done = a_full + kAS;         // [kAS] the stage's MMAs have finished: its activation and operand slots are free
  uint64_t* tfull = done + kAS;          // [2]   accumulator complete
  uint64_t* tempty = tfull + 2;          // [2]   accumulator read back by every epilogue warp
  uint32_t* tmem_holder = (uint32_t*)(tempty + 2);
  volatile int* abort_flag = (volatile int*)(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nsb_total = a.K / QSB;

  if (threadIdx.x == 0) {
    for (int s = 0; s < RS; s++) {
      mbar_init(smem_u32(raw_full + s), 1);
      mbar_init(smem_u32(raw_empty + s), kDqWarps);
    }
    for (int s = 0; s < kAS; s++) {
      mbar_init(smem_u32(x_full + s), 1);
      mbar_init(smem_u32(a_full + s), kDqWarps);
      mbar_init(smem_u32(done + s), 1);
    }
    for (int s = 0; s < 2; s++) {
      mbar_init(smem_u32(tfull + s), 1);
      mbar_init(smem_u32(tempty + s), kDqWarps);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  // tensor-memory columns: accumulators at +0 and +64, operand stages at +128, +256 and +384 (128 columns = 256 of K each)
  pdl_trigger();

  if (warp == 0) {
    // The weights are not written by any kernel: this thread does not wait for the kernel before this one, so the
    // first stages stream in while that kernel is still finishing.
    if (lane == 0) {
      uint32_t g = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < a.n_items && ok; item += gridDim.x) {
        const int tile = item / a.splits, sp = item - tile * a.splits;
        const int sb0 = sp * a.sb_per_split, sb1 = min(nsb_total, sb0 + a.sb_per_split);
        for (int sb = sb0; sb < sb1; sb++, g++) {
          const uint32_t s = g % RS;
          if (!mbar_wait(smem_u32(raw_empty + s), ((g / RS) & 1) ^ 1, abort_flag)) { ok = false; break; }
          mbar_expect_tx(smem_u32(raw_full + s), RAW_BYTES);
          tma_load_2d(smem_u32(sR + s * RAW_BYTES), &tmW, smem_u32(raw_full + s), rot_sb(sb0, sb1, sb - sb0) * RAWB, tile * QBM);
        }
      }
    }
  } else if (warp == 2) {
    if (lane == 0) {
      pdl_wait();
      uint32_t g = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < a.n_items && ok; item += gridDim.x) {
        const int tile = item / a.splits, sp = item - tile * a.splits;
        const int sb0 = sp * a.sb_per_split, sb1 = min(nsb_total, sb0 + a.sb_per_split);
        for (int sb = sb0; sb < sb1; sb++, g++) {
          const uint32_t s = g % kAS;
          if (!mbar_wait(smem_u32(done + s), ((g / kAS) & 1) ^ 1, abort_flag)) { ok = false; break; }
          mbar_expect_tx(smem_u32(x_full + s), kXStage);
          const int k0 = rot_sb(sb0, sb1, sb - sb0) * QSB;
          const uint32_t dst = smem_u32(sX + s * kXStage), bar = smem_u32(x_full + s);
#pragma unroll
          for (int u = 0; u < 4; u++) tma_load_2d(dst + u * (QBN * 128), &tmX, bar, k0 + u * 64, 0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_bf16(QBM, QBN);
      const uint64_t bd0 = smem_desc_sw128(smem_u32(sX));
      const uint32_t b_hi = (uint32_t)(bd0 >> 32), b_lo0 = (uint32_t)bd0;
      uint32_t g = 0, tcount = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < a.n_items && ok; item += gridDim.x, tcount++) {
        const int tile = item / a.splits, sp = item - tile * a.splits;
        const int n_st = min(nsb_total, (sp + 1) * a.sb_per_split) - sp * a.sb_per_split;
        (void)tile;
        const uint32_t acc = tcount & 1;
        if (!mbar_wait(smem_u32(tempty + acc), ((tcount >> 1) & 1) ^ 1, abort_flag)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * QBN;
#ifdef QGEMM_STAMPS
        const long long item_t0 = clock64();
#endif
        for (int i = 0; i < n_st; i++, g++) {
          const uint32_t s = g % kAS, ph = (g / kAS) & 1;
          QSTAMP_T0();
          if (!mbar_wait(smem_u32(a_full + s), ph, abort_flag) || !mbar_wait(smem_u32(x_full + s), ph, abort_flag)) { ok = false; break; }
          QSTAMP_ADD(0);                  // cycles this thread waited for the stage's operands
          tc_fence_after();
          const uint32_t a_tmem = tmem_base + 128 + s * 128;
          const uint32_t b_lo = b_lo0 + s * (kXStage >> 4);
          umma_ts_lohi(d_tmem, a_tmem, b_lo, b_hi, idesc, i != 0 ? 1u : 0u);
#pragma unroll
          for (int m = 1; m < 16; m++)     // K block m / 4 (8 KB apart in shared memory, 32 columns apart in tensor memory), K step m % 4
            umma_ts_lohi(d_tmem, a_tmem + (m >> 2) * 32 + (m & 3) * 8, b_lo + (m >> 2) * ((QBN * 128) >> 4) + (m & 3) * 2, b_hi, idesc, 1u);
          umma_commit(smem_u32(done + s));
          QSTAMP_ADD(1);                  // cycles to issue the stage's 16 MMAs and the commit
#ifdef QGEMM_STAMPS
          // retire time of a stage: with the operands of the NEXT stage already there (wait above near zero), the gap
          // between two stages' `done` barriers is what the tensor core needed for 16 MMAs
          if (blockIdx.x == 0 && i + 1 == n_st) {
            mbar_wait(smem_u32(done + s), ph, abort_flag);
            g_qgemm_stamps[2] += clock64() - item_t0;
            g_qgemm_stamps[3] += n_st;
          }
#endif
        }
        umma_commit(smem_u32(tfull + acc));      // released even after a failed wait; the flag says why
      }
    }
  } else if (warp >= kRoleWarps) {
    // ---- expansion + epilogue warps
    const int dw = warp - kRoleWarps, q = warp & 3, khalf = dw >> 2;      // lane quarter; K blocks 2 khalf, 2 khalf + 1 of a stage
    const int row = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    uint32_t g = 0, ecount = 0;
    bool ok = true;
    bool waited = false;

    // epilogue of the item with accumulator number `ec`: this warp takes its lane quarter and 32 of the 64 token columns
    auto epilogue = [&](int item, uint32_t ec) {
      const int tile = item / a.splits, sp = item - tile * a.splits;
      const uint32_t acc = ec & 1;
      bool tok = mbar_wait(smem_u32(tfull + acc), (ec >> 1) & 1, abort_flag);
      tok = __all_sync(0xffffffffu, tok && !*abort_flag);
      if (!tok) { ok = false; return; }
      tc_fence_after();
      if (!waited) {                      // first global write of this thread: the kernel before this one must be complete
        pdl_wait();
        waited = true;
      }
      const int n = tile * QBM + row;
      const int t0 = khalf * 32;
      uint32_t v[32];
      tmem_ld32(tmem_base + lane_addr + acc * QBN + (uint32_t)t0, v);
      tmem_ld_wait();
      const bool live = n < a.N;
      if (a.epi == QEPI_SWIGLU) {
        // rows are (gate_i, up_i) pairs in adjacent lanes; the even lane finishes the even tokens, the odd lane the odd ones
        const float b = (a.bias && live) ? a.bias[n] : 0.f;
        const bool odd = lane & 1;
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const float va = __uint_as_float(v[j]) + b, vb = __uint_as_float(v[j + 1]) + b;
          const float pa = __shfl_xor_sync(0xffffffffu, va, 1), pb = __shfl_xor_sync(0xffffffffu, vb, 1);
          const float gate = odd ? pb : va, up = odd ? vb : pa;
          const int t = t0 + j + (odd ? 1 : 0);
          if (live && t < a.T) a.out_bf16[(size_t)t * a.ldo + (n >> 1)] = __float2bfloat16(silu(gate) * up);
        }
      } else {
        // Transpose 4 x 4 patches inside each lane quad (four shuffles per four tokens): a lane then holds, for ONE token,
        // four consecutive output columns, so that a warp instruction moves four rows of 128 contiguous bytes: vector
        // stores, vector reductions into L2, full packets over NVLink.
        float b = 0.f;
        if (a.bias && live && sp == 0) b = a.bias[n];
        const int lq = lane & 3, nq = tile * QBM + q * 32 + (lane & ~3);      // first of this lane's four columns
        const bool quad_live = nq + 3 < a.N && (a.ldo & 3) == 0;
#pragma unroll
        for (int k4 = 0; k4 < 8; k4++) {
          float c[4] = {__uint_as_float(v[4 * k4]) + b, __uint_as_float(v[4 * k4 + 1]) + b, __uint_as_float(v[4 * k4 + 2]) + b,
                        __uint_as_float(v[4 * k4 + 3]) + b};
          float x0 = (lq & 1) ? c[0] : c[1];
          x0 = __shfl_xor_sync(0xffffffffu, x0, 1);
          if (lq & 1) c[0] = x0; else c[1] = x0;
          float x1 = (lq & 1) ? c[2] : c[3];
          x1 = __shfl_xor_sync(0xffffffffu, x1, 1);
          if (lq & 1) c[2] = x1; else c[3] = x1;
          float x2 = (lq & 2) ? c[0] : c[2];
          x2 = __shfl_xor_sync(0xffffffffu, x2, 2);
          if (lq & 2) c[0] = x2; else c[2] = x2;
          float x3 = (lq & 2) ? c[1] : c[3];
          x3 = __shfl_xor_sync(0xffffffffu, x3, 2);
          if (lq & 2) c[1] = x3; else c[3] = x3;
          const int t = t0 + 4 * k4 + lq;          // c[0..3] = columns nq .. nq + 3 of token t
          if (t >= a.T) continue;
          const size_t idx = (size_t)t * a.ldo + nq;
          if (quad_live) {
            const float4 o = make_float4(c[0], c[1], c[2], c[3]);
            if (a.epi == QEPI_ADD) {
              asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(a.out_f32 + idx), "f"(o.x), "f"(o.y), "f"(o.z), "f"(o.w) : "memory");
            } else {
              if (a.out_f32) *(float4*)(a.out_f32 + idx) = o;
              if (a.out_bf16) *(uint2*)(a.out_bf16 + idx) = make_uint2(pack2(o.x, o.y), pack2(o.z, o.w));
            }
          } else {
#pragma unroll
            for (int e = 0; e < 4; e++) {
              if (nq + e >= a.N) break;
              if (a.epi == QEPI_ADD) {
                asm volatile("red.relaxed.gpu.global.add.f32 [%0], %1;" ::"l"(a.out_f32 + idx + e), "f"(c[e]) : "memory");
              } else {
                if (a.out_f32) a.out_f32[idx + e] = c[e];
                if (a.out_bf16) a.out_bf16[idx + e] = __float2bfloat16(c[e]);
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(tempty + acc));
    };

    int pending = -1;
    for (int item = blockIdx.x; item < a.n_items && ok; item += gridDim.x) {
      const int tile = item / a.splits, sp = item - tile * a.splits;
      const int sb0 = sp * a.sb_per_split, sb1 = min(nsb_total, sb0 + a.sb_per_split);
      const int n = tile * QBM + row;
      [[maybe_unused]] float d6 = 0.f;
      if constexpr (WT == QW_Q6KR) d6 = (n < a.N) ? __half2float(a.w2[(size_t)n * nsb_total + rot_sb(sb0, sb1, 0)]) : 0.f;
      for (int sb = sb0; sb < sb1 && ok; sb++, g++) {
        [[maybe_unused]] float d6_next = 0.f;
        if constexpr (WT == QW_Q6KR) {      // the next stage's d, fetched a stage ahead so that its latency is hidden
          if (n < a.N && sb + 1 < sb1) d6_next = __half2float(a.w2[(size_t)n * nsb_total + rot_sb(sb0, sb1, sb + 1 - sb0)]);
        }
        const uint32_t rs = g % RS, s = g % kAS;
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(raw_full + rs), (g / RS) & 1, abort_flag));
        if (!ok) break;
        const uint8_t* rowp = sR + rs * RAW_BYTES + row * RAWB;
        [[maybe_unused]] uint4 hdr;
        [[maybe_unused]] float d4 = 0.f, dmin4 = 0.f;
        if constexpr (WT == QW_Q4KR) {
          hdr = *(const uint4*)rowp;
          const __half2 dd = *reinterpret_cast<const __half2*>(&hdr.x);
          d4 = __low2float(dd);
          dmin4 = __high2float(dd);
        }
#pragma unroll
        for (int u = 0; u < 2; u++) {
          const int kbu = 2 * khalf + u;               // K block of the stage
          uint32_t r[32];
          if constexpr (WT == QW_Q4KR) {
            // sub-blocks 2 kbu and 2 kbu + 1: their 6-bit scale and min, byte-parallel
            uint32_t S, Mn;
            if (kbu < 2) {
              S = hdr.y & 0x3F3F3F3Fu;
              Mn = hdr.z & 0x3F3F3F3Fu;
            } else {
              S = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
              Mn = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
            }
#pragma unroll
            for (int h = 0; h < 2; h++) {
              const int j = 2 * kbu + h, sh = 8 * (j & 3);
              const float av = d4 * (float)((S >> sh) & 0xFFu);
              const __nv_bfloat16 ab = __float2bfloat16(av);
              const __nv_bfloat16 cb = __float2bfloat16(8.f * __bfloat162float(ab) - dmin4 * (float)((Mn >> sh) & 0xFFu));
              expand_q4k(__halves2bfloat162(ab, ab), __halves2bfloat162(cb, cb), *(const uint4*)(rowp + 16 + j * 16), r + 16 * h);
            }
          } else {
#pragma unroll
            for (int h = 0; h < 2; h++) {
              const int j = 2 * kbu + h;
              const uint32_t scw = *(const uint16_t*)(rowp + 192 + 2 * j);
              const __nv_bfloat162 ss = __floats2bfloat162_rn(d6 * (float)(int8_t)(scw & 0xFF), d6 * (float)(int8_t)(scw >> 8));
              expand_q6k(*(const uint4*)(rowp + j * 16), *(const uint2*)(rowp + 128 + j * 8), bf162_as_u32(ss), r + 16 * h);
            }
          }
          if (u == 0) {      // the first values are in registers: only now does this warp need the operand slot
            ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(done + s), ((g / kAS) & 1) ^ 1, abort_flag));
            if (!ok) break;
            tc_fence_after();
          } else {           // everything this warp needs from the raw stage has been read
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(raw_empty + rs));
            tmem_st_wait();  // the first store must have left the registers it reads: they are reused
          }
          tmem_st32(tmem_base + lane_addr + 128 + s * 128 + kbu * 32, r);
        }
        if (!ok) break;
        if constexpr (WT == QW_Q6KR) d6 = d6_next;
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(a_full + s));
        if (pending >= 0) {     // the MMA thread has a stage of the new item queued: finish the old item now
          epilogue(pending, ecount++);
          pending = -1;
        }
      }
      pending = item;
    }
    if (pending >= 0 && ok) epilogue(pending, ecount++);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
  if (threadIdx.x == 0 && *abort_flag && a.status) atomicExch(a.status, (int)B200_ERR_TIMEOUT_MMA);
}

static int q_sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

template <int WT>
static int launch_q(const void* w, const void* x, int ldx, QGemmArgs a, cudaStream_t st) {
  constexpr int RAWB = QTraits<WT>::RAWB, RS = QTraits<WT>::RS;
  constexpr size_t smem = 1024 + kAS * (size_t)kXStage + (size_t)RS * QBM * RAWB + (2 * RS + 3 * kAS + 4) * 8 + 16;
  static_assert(smem <= 227 * 1024, "shared memory budget");
  auto kern = qgemm_kernel<WT>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int nsb = a.K / QSB;
  CUtensorMap tw, tx;
  // packed rows as bytes: [N][nsb * RAWB], one box = 128 rows of one superblock; rows past N read as zeros (scale 0)
  int rc = make_tmap_2d(&tw, w, 1, (uint64_t)a.N, (uint64_t)nsb * RAWB, (uint64_t)nsb * RAWB, QBM, RAWB, false);
  if (rc) return rc;
  rc = make_tmap_2d(&tx, x, 2, (uint64_t)a.T, (uint64_t)a.K, (uint64_t)ldx * 2, QBN, 64, true);
  if (rc) return rc;
  const int grid = a.n_items < q_sm_count() ? a.n_items : q_sm_count();
  return launch_pdl(kern, dim3(grid), dim3(kQThreads), smem, st, tw, tx, a);
}

// wt: QW_Q4KR / QW_Q6KR; `w` the row-major packed plane the mat-vec kernels read as well ([N][K / 256][144 or 208
// bytes]), `w2` the fp16 d plane of Q6_K-R.  x: bf16 [T][ldx].  Any T: tokens are taken 64 at a time.
//   QEPI_STORE  out_f32 and/or out_bf16 [T][ldo] = result (+ bias)
//   QEPI_ADD    out_f32 [T][ldo] += result (+ bias); split_k > 1 allowed (0 = choose)
//   QEPI_SWIGLU rows of W are (gate_0, up_0, gate_1, ...); out_bf16 [T][ldo] gets silu(gate) * up, N / 2 columns
B200_API int b200_qgemm(int wt, const void* w, const void* w2, int N, int K, const void* x, int ldx, int T, float* out_f32,
                        void* out_bf16, int ldo, const float* bias, int epi, int split_k, int* status, cudaStream_t st) {
  if (K % QSB || (ldx % 8) || T < 1 || N < 1 || ((uintptr_t)w & 15) || ((uintptr_t)x & 15)) return B200_ERR_BAD_ARG;
  if (wt != QW_Q4KR && wt != QW_Q6KR) return B200_ERR_BAD_ARG;
  if (wt == QW_Q6KR && !w2) return B200_ERR_BAD_ARG;
  if (epi == QEPI_SWIGLU ? (!out_bf16 || (N & 1)) : epi == QEPI_ADD ? !out_f32 : (epi != QEPI_STORE || (!out_f32 && !out_bf16)))
    return B200_ERR_BAD_ARG;
  QGemmArgs a = {};
  a.w2 = (const __half*)w2; a.bias = bias; a.ldo = ldo; a.N = N; a.K = K; a.epi = epi; a.status = status;
  const int nsb = K / QSB, tiles = (N + QBM - 1) / QBM;
  int splits = 1;
  if (epi == QEPI_ADD) {
    if (split_k > 0) splits = split_k;
    else if (tiles < q_sm_count()) {
      splits = q_sm_count() / tiles;                 // fill the GPU once ...
      while (splits > 1 && nsb / splits < 2) splits--;  // ... with at least two stages per item
    }
    if (splits > nsb) splits = nsb;
  } else if (split_k > 1) {
    return B200_ERR_BAD_ARG;
  }
  a.sb_per_split = (nsb + splits - 1) / splits;
  a.splits = (nsb + a.sb_per_split - 1) / a.sb_per_split;     // no empty split
  a.n_items = tiles * a.splits;
  for (int t0 = 0; t0 < T; t0 += QBN) {
    a.T = T - t0 < QBN ? T - t0 : QBN;
    a.out_f32 = out_f32 ? out_f32 + (size_t)t0 * ldo : nullptr;
    a.out_bf16 = out_bf16 ? (__nv_bfloat16*)out_bf16 + (size_t)t0 * ldo : nullptr;
    const void* xs = (const __nv_bfloat16*)x + (size_t)t0 * ldx;
    const int rc = wt == QW_Q4KR ? launch_q<QW_Q4KR>(w, xs, ldx, a, st) : launch_q<QW_Q6KR>(w, xs, ldx, a, st);
    if (rc) return rc;
  }
  return 0;
}

#ifdef QGEMM_STAMPS
B200_API int b200_qgemm_stamps(long long* out, int reset) {
  int rc = (int)cudaMemcpyFromSymbol(out, g_qgemm_stamps, sizeof(long long) * 4);
  if (rc == 0 && reset) {
    const long long z[4] = {0, 0, 0, 0};
    rc = (int)cudaMemcpyToSymbol(g_qgemm_stamps, z, sizeof(z));
  }
  return rc;
}
#endif
