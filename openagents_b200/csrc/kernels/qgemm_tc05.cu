// Quantized-weight GEMM on tcgen05 with the dequantization inside the pipeline:
//     Y[t][n] (+)= sum_k X[t][k] * W[n][k],   W in Q4_K-R or Q6_K-R, X bf16
// used for decode batches above the mat-vec range and for prefill.  The packed weights are read
// from HBM exactly once, in their 4.5- or 6.5-bit form.
//
// The weight tile is the MMA's M operand (128 weight rows), the tokens are its N operand (BN), so a
// 64-token decode batch still fills the 128-lane tensor-memory accumulator.  Roles in a CTA:
//   warp 0      one thread: TMA loads of raw packed weight tiles (128 rows x one superblock)
//   warp 1      one thread: tcgen05.mma issue; the warp owns the tensor-memory allocation
//   warps 2-17  expand raw tiles into 128x64 bf16 operand tiles in the 128-byte-swizzled layout the MMA
//               reads: a pair of warps owns one slot of an 8-slot operand ring and every eighth K
//               block (one mask yields two adjacent bf16 mantissas, one fma applies the scale and
//               offset precomputed at load); warps 2-9 then run the epilogue
//   warp 18     one thread: TMA loads of the activation tiles
// Rings hand over through mbarriers; every wait is bounded and reports through `status`.
// Split-K (grid.z) adds partial tiles into fp32 output with `red.global.add`.
//
// GEMM-shaped reference math: cs336-a2-benchmark-workload.ts:251-292.
#include "tc05.cuh"

using namespace b200;
using namespace b200::tc;

enum { QW_Q4KR = 0, QW_Q6KR = 1 };
enum { QEPI_STORE = 0, QEPI_ADD = 1 };

struct QGemmArgs {
  const uint8_t* w;      // tile-major packed weights: [N/128][K/256][128 rows][RAW bytes]
  const __half* w2;      // unused (scales live in the tile-major rows)
  float* y;              // [T][ldy] fp32
  const float* bias;     // [N] or null (applied by split 0)
  int ldy, T, N, K;
  int epi;
  int sb_per_split;      // superblocks per grid.z slice
  int* status;
  long long* dbg;        // optional [grid][8] cycle counters (profiling builds of the caller only)
};

template <int WT>
struct QTraits {
  static constexpr int RAW = WT == QW_Q4KR ? 160 : 224;   // bytes per row per superblock (tile-major form)
};

__device__ __forceinline__ uint32_t bf162_as_u32(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __nv_bfloat162 u32_as_bf162(uint32_t v) { return *reinterpret_cast<__nv_bfloat162*>(&v); }

// Expand 32 elements (one sub-block: 4 words) into four 16-byte chunks of bf16.
// Q4_K: value = a * (16 + q) + c; the nibble sits in the mantissa of bf16 16.0.  `ac` = (a, c).
__device__ __forceinline__ void expand_q4k(uint32_t ac, const uint4 q, uint4 (&out)[4]) {
  const __nv_bfloat162 acv = u32_as_bf162(ac);
  const __nv_bfloat162 A2 = __halves2bfloat162(acv.x, acv.x), C2 = __halves2bfloat162(acv.y, acv.y);
  const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const uint32_t v = w[i];
    const uint32_t t0 = ((v << 3) & 0x00780078u) | 0x41804180u;
    const uint32_t t1 = ((v >> 1) & 0x00780078u) | 0x41804180u;
    const uint32_t t2 = ((v >> 5) & 0x00780078u) | 0x41804180u;
    const uint32_t t3 = ((v >> 9) & 0x00780078u) | 0x41804180u;
    out[i].x = bf162_as_u32(__hfma2(u32_as_bf162(t0), A2, C2));
    out[i].y = bf162_as_u32(__hfma2(u32_as_bf162(t1), A2, C2));
    out[i].z = bf162_as_u32(__hfma2(u32_as_bf162(t2), A2, C2));
    out[i].w = bf162_as_u32(__hfma2(u32_as_bf162(t3), A2, C2));
  }
}

// Q6_K: 6-bit value = nibble | two high bits; (64 + q) - 96 = q - 32 is exact in bf16.  `ss` holds
// the two bf16 scales of the sub-block (first and second 16 elements).
__device__ __forceinline__ void expand_q6k(const uint4 lo, const uint2 tw, uint32_t ss, uint4 (&out)[4]) {
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
    out[i].x = bf162_as_u32(__hmul2(__hsub2(u32_as_bf162((q0 << 1) | 0x42804280u), off), S2));
    out[i].y = bf162_as_u32(__hmul2(__hsub2(u32_as_bf162((q1 << 1) | 0x42804280u), off), S2));
    out[i].z = bf162_as_u32(__hmul2(__hsub2(u32_as_bf162((q2 << 1) | 0x42804280u), off), S2));
    out[i].w = bf162_as_u32(__hmul2(__hsub2(u32_as_bf162((q3 << 1) | 0x42804280u), off), S2));
  }
}

constexpr int QBM = 128, QBK = 64;

template <int WT, int BN, int RS, int AS, int XS>
__global__ void __launch_bounds__(608) qgemm_kernel(const __grid_constant__ CUtensorMap tmX, const QGemmArgs a) {
  constexpr int RAW = QTraits<WT>::RAW;
  constexpr int RAW_BYTES = QBM * RAW, A_BYTES = QBM * QBK * 2, X_BYTES = BN * QBK * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;                               // AS x 16 KB, swizzled operand tiles
  uint8_t* sX = sA + AS * A_BYTES;                  // XS x BN*128 B, swizzled activation tiles
  uint8_t* sR = sX + XS * X_BYTES;                  // RS raw packed tiles
  uint64_t* bars = (uint64_t*)(sR + ((RS * RAW_BYTES + 127) & ~127));
  uint64_t* raw_full = bars;
  uint64_t* raw_empty = raw_full + RS;
  uint64_t* a_full = raw_empty + RS;
  uint64_t* a_empty = a_full + AS;
  uint64_t* x_full = a_empty + AS;
  uint64_t* x_empty = x_full + XS;
  uint64_t* tfull = x_empty + XS;
  uint32_t* tmem_holder = (uint32_t*)(tfull + 1);
  volatile int* abort_flag = (volatile int*)(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.x * BN, n0 = blockIdx.y * QBM;
  long long* dbg = a.dbg ? a.dbg + ((size_t)(blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 8 : nullptr;
  const long long t_start = clock64();
#define DBG_WAIT(slot_, expr_) do { long long _c = clock64(); expr_; if (dbg && lane == 0) atomicAdd((unsigned long long*)&dbg[slot_], (unsigned long long)(clock64() - _c)); } while (0)
  const int nsb_total = a.K / 256;
  const int sb0 = blockIdx.z * a.sb_per_split;
  const int sb1 = min(nsb_total, sb0 + a.sb_per_split);
  const int nsb = max(0, sb1 - sb0);
  const int KB = nsb * 4;

  if (threadIdx.x == 0) {
    for (int s = 0; s < RS; s++) {
      mbar_init(smem_u32(raw_full + s), 1);
      mbar_init(smem_u32(raw_empty + s), 8);  // 4 K blocks x 2 warps
    }
    for (int s = 0; s < AS; s++) {
      mbar_init(smem_u32(a_full + s), 2);
      mbar_init(smem_u32(a_empty + s), 1);
    }
    for (int s = 0; s < XS; s++) {
      mbar_init(smem_u32(x_full + s), 1);
      mbar_init(smem_u32(x_empty + s), 1);
    }
    mbar_init(smem_u32(tfull), 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    if (lane == 0) {   // raw packed weight tiles, one superblock of 128 rows per stage
      for (int i = 0; i < nsb; i++) {
        const int s = i % RS;
        bool okw; DBG_WAIT(0, okw = mbar_wait(smem_u32(raw_empty + s), ((i / RS) & 1) ^ 1, abort_flag));
        if (!okw) break;
        mbar_expect_tx(smem_u32(raw_full + s), RAW_BYTES);
        // tile-major weights: the 128 rows of one superblock are one contiguous block
        const uint8_t* src = a.w + ((size_t)blockIdx.y * nsb_total + sb0 + i) * RAW_BYTES;
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(smem_u32(sR + s * RAW_BYTES)), "l"(src), "r"((uint32_t)RAW_BYTES), "r"(smem_u32(raw_full + s))
                     : "memory");
      }
    }
  } else if (warp == 2 + 2 * AS) {
    if (lane == 0) {   // activation tiles, one 64-wide K block per stage
      for (int kb = 0; kb < KB; kb++) {
        const int s = kb % XS;
        bool okw; DBG_WAIT(1, okw = mbar_wait(smem_u32(x_empty + s), ((kb / XS) & 1) ^ 1, abort_flag));
        if (!okw) break;
        mbar_expect_tx(smem_u32(x_full + s), X_BYTES);
        tma_load_2d(smem_u32(sX + s * X_BYTES), &tmX, smem_u32(x_full + s), sb0 * 256 + kb * QBK, t0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_bf16(QBM, BN);
      for (int kb = 0; kb < KB; kb++) {
        const int sa = kb % AS, sx = kb % XS;
        bool ok1, ok2;
        DBG_WAIT(2, ok1 = mbar_wait(smem_u32(a_full + sa), (kb / AS) & 1, abort_flag));
        DBG_WAIT(3, ok2 = mbar_wait(smem_u32(x_full + sx), (kb / XS) & 1, abort_flag));
        if (!ok1 || !ok2) break;
        tc_fence_after();
        const uint64_t ad = smem_desc_sw128(smem_u32(sA + sa * A_BYTES));
        const uint64_t bd = smem_desc_sw128(smem_u32(sX + sx * X_BYTES));
#pragma unroll
        for (int k = 0; k < QBK / 16; k++) umma_bf16(tmem_base, ad + 2 * k, bd + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
        umma_commit(smem_u32(a_empty + sa));
        umma_commit(smem_u32(x_empty + sx));
      }
      umma_commit(smem_u32(tfull));
    }
  } else {
    // ---- expansion: sixteen warps; warps 2k and 2k+1 own operand slot k and the K blocks kb = k,
    // k + 8, ..., each expanding 64 of the tile's 128 rows (a lane takes rows lane and lane + 32 of
    // its half).  Eight K blocks are in flight and no two slots share a barrier.
    const int dw = warp - 2, slot = dw >> 1, hh = dw & 1;
    bool ok = true;
    for (int kb = slot; kb < KB && ok; kb += AS) {
      const int i = kb >> 2, g = kb & 3, rs = i % RS;
      if (dw == 0) { DBG_WAIT(4, ok = mbar_wait(smem_u32(raw_full + rs), (i / RS) & 1, abort_flag)); }
      else ok = mbar_wait(smem_u32(raw_full + rs), (i / RS) & 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (dw == 0) { DBG_WAIT(5, ok = mbar_wait(smem_u32(a_empty + slot), ((kb / AS) & 1) ^ 1, abort_flag)); }
      else ok = mbar_wait(smem_u32(a_empty + slot), ((kb / AS) & 1) ^ 1, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const long long t_exp = clock64();
      uint8_t* tile = sA + slot * A_BYTES;
#pragma unroll
      for (int rr = 0; rr < 2; rr++) {
        const int r = 64 * hh + lane + 32 * rr;
        const uint8_t* rowp = sR + rs * RAW_BYTES + r * RAW;
        uint8_t* dst = tile + r * 128;
#pragma unroll
        for (int h = 0; h < 2; h++) {
          const int j = 2 * g + h;
          uint4 out[4];
          if constexpr (WT == QW_Q4KR) {
            expand_q4k(*(const uint32_t*)(rowp + 4 * j), *(const uint4*)(rowp + 32 + j * 16), out);
          } else {
            expand_q6k(*(const uint4*)(rowp + 32 + j * 16), *(const uint2*)(rowp + 160 + j * 8),
                       *(const uint32_t*)(rowp + 4 * j), out);
          }
#pragma unroll
          for (int c = 0; c < 4; c++) *(uint4*)(dst + (((4 * h + c) ^ (r & 7)) << 4)) = out[c];
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (dbg && dw == 0 && lane == 0) atomicAdd((unsigned long long*)&dbg[6], (unsigned long long)(clock64() - t_exp));
      if (lane == 0) {
        mbar_arrive(smem_u32(a_full + slot));
        mbar_arrive(smem_u32(raw_empty + rs));     // this warp is done with its part of the raw tile
      }
    }
    // ---- epilogue: lane quarter = warp % 4, column half = (warp - 2) / 4
    bool tok = mbar_wait(smem_u32(tfull), 0, abort_flag);
    tok = __all_sync(0xffffffffu, tok && ok && !*abort_flag);
    if (tok && nsb > 0 && dw < 8) {
      tc_fence_after();
      const int q = warp & 3, ch = dw >> 2;
      const int n = n0 + q * 32 + lane;
      const float bias = (a.bias && blockIdx.z == 0 && n < a.N) ? a.bias[n] : 0.f;
#pragma unroll 1
      for (int c = ch * (BN / 64); c < (ch + 1) * (BN / 64); c++) {
        uint32_t v[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 32), v);
        tmem_ld_wait();
        if (n < a.N) {
#pragma unroll
          for (int e = 0; e < 32; e++) {
            const int t = t0 + c * 32 + e;
            if (t < a.T) {
              float* p = a.y + (size_t)t * a.ldy + n;
              const float val = __uint_as_float(v[e]) + bias;
              if (a.epi == QEPI_ADD) atomicAdd(p, val);
              else *p = val;
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, BN);
  if (threadIdx.x == 0 && *abort_flag && a.status) atomicExch(a.status, (int)B200_ERR_TIMEOUT_MMA);
  if (dbg && threadIdx.x == 0) dbg[7] = clock64() - t_start;
#undef DBG_WAIT
}

template <int WT, int BN, int RS, int AS, int XS>
static int launch_q(const void* w, const void* w2, const void* x, int ldx, QGemmArgs a, int split_k, cudaStream_t st) {
  constexpr int RAW = QTraits<WT>::RAW;
  constexpr size_t smem = 1024 + (size_t)AS * QBM * QBK * 2 + (size_t)XS * BN * QBK * 2 + (((size_t)RS * QBM * RAW + 127) & ~127) +
                          (2 * RS + 2 * AS + 2 * XS + 1) * 8 + 16;
  static_assert(AS == 4 || AS == 8, "two expansion warps per operand slot");
  static_assert(smem <= 227 * 1024, "shared memory budget");
  auto kern = qgemm_kernel<WT, BN, RS, AS, XS>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  CUtensorMap tx;
  a.w = (const uint8_t*)w;
  int rc = make_tmap_2d(&tx, x, 2, (uint64_t)a.T, (uint64_t)a.K, (uint64_t)ldx * 2, BN, QBK, true);
  if (rc) return rc;
  a.w2 = (const __half*)w2;
  const int nsb = a.K / 256;
  a.sb_per_split = (nsb + split_k - 1) / split_k;
  dim3 grid((a.T + BN - 1) / BN, (a.N + QBM - 1) / QBM, (nsb + a.sb_per_split - 1) / a.sb_per_split);
  kern<<<grid, 32 * (3 + 2 * AS), smem, st>>>(tx, a);
  return (int)cudaGetLastError();
}

// wt: QW_Q4KR / QW_Q6KR; `w` (and `w2`) in the tile-major form: rows padded to a multiple of 128 and
// stored [N/128][K/256][128][bytes], so the 128 rows a CTA needs for one superblock are one
// contiguous block (row-major packed weights make that a 144-byte gather per row, which wastes most
// of every DRAM page).  x: bf16 [T][ldx].  y: fp32 [T][ldy].  split_k > 1 requires epi = QEPI_ADD
// (y then already holds the residual, or zeros).  split_k = 0 chooses a split that fills the GPU.
B200_API int b200_qgemm(int wt, const void* w, const void* w2, int N, int K, const void* x, int ldx, int T, float* y,
                        int ldy, const float* bias, int epi, int split_k, int* status, long long* dbg, cudaStream_t st) {
  if (K % 256 || (ldx % 8) || T < 1 || N < 1) return B200_ERR_BAD_ARG;
  QGemmArgs a;
  a.w = nullptr; a.w2 = nullptr; a.y = y; a.bias = bias; a.ldy = ldy; a.T = T; a.N = N; a.K = K; a.epi = epi; a.sb_per_split = 0;
  a.status = status;
  a.dbg = dbg;
  const int bn = T <= 64 ? 64 : 128;
  if (split_k == 0) {
    const int tiles = ((T + bn - 1) / bn) * ((N + QBM - 1) / QBM);
    split_k = 1;
    if (epi == QEPI_ADD)
      while (tiles * split_k < 120 && split_k * 2 <= K / 256 && split_k < 8) split_k *= 2;
  }
  if (split_k > 1 && epi != QEPI_ADD) return B200_ERR_BAD_ARG;
  if (wt == QW_Q4KR) {
    if (bn == 64) return launch_q<QW_Q4KR, 64, 3, 4, 12>(w, w2, x, ldx, a, split_k, st);
    return launch_q<QW_Q4KR, 128, 3, 8, 2>(w, w2, x, ldx, a, split_k, st);
  }
  if (wt == QW_Q6KR) {
    if (bn == 64) return launch_q<QW_Q6KR, 64, 2, 4, 12>(w, w2, x, ldx, a, split_k, st);
    return launch_q<QW_Q6KR, 128, 2, 8, 2>(w, w2, x, ldx, a, split_k, st);
  }
  return B200_ERR_BAD_ARG;
}
