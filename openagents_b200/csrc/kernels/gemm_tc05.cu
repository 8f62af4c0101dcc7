// bf16 GEMM on the 5th-generation tensor cores: D[M][N] = A[M][K] * B[N][K]^T (+ epilogue).
//
// One CTA computes a 128 x BN output tile.  Warp 0 feeds shared memory with TMA tile loads
// (128-byte swizzle), one elected thread of warp 1 issues tcgen05.mma with the accumulator in
// tensor memory, and warps 2..5 read the accumulator back with tcgen05.ld and run the epilogue
// (bias, GELU, residual, fp32 or bf16 store).  Stages hand over through mbarriers; every wait is
// bounded and a timeout is reported through the status word instead of hanging.
//
// Both operands are K-major ("TN"), which is the natural layout of y = x W^T with W stored
// [out][in]; the GEMM-shaped reference case is cs336-a2-benchmark-workload.ts:251-292.
#include "tc05.cuh"
#include "../comm/sym.cuh"

using namespace b200;
using namespace b200::tc;

namespace b200 {

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
        qr == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

int make_tmap_2d(CUtensorMap* map, const void* base, int elem_bytes, uint64_t rows, uint64_t cols,
                 uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols, bool swizzle128) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return -1;
  if (((uintptr_t)base & 15) || (row_stride_bytes & 15)) return -2;
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                             : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

}  // namespace b200

// ACT_SWIGLU_PAIR: B rows are interleaved (gate_0, up_0, gate_1, ...); the epilogue writes
// silu(gate) * up as bf16, N / 2 values per row of out_bf16 (row stride ldc), nothing else.
enum { ACT_NONE = 0, ACT_GELU = 1, ACT_SWIGLU_PAIR = 2 };

struct GemmEpi {
  float* out_f32;            // either or both outputs
  __nv_bfloat16* out_bf16;
  const float* bias;         // [N] or null
  const float* resid_f32;    // [M][ldc] or null, added after the activation
  const __nv_bfloat16* resid_bf16;
  int ldc;
  int act;
  int accumulate;            // out_f32 += value
  // Split-K (small M): each split adds its partial product into out_f32 with a vector `red`, so
  // out_f32 must already hold the residual (or zeros); bias comes from split 0 only.
  int splitk_red;
  // Swapped operands (few tokens): the kernel computes W X^T, so an accumulator row is an output
  // COLUMN; the epilogue then writes out[col][row] and takes the bias by row.
  int transposed;
  // Grouped GEMM (mixture-of-experts): rows of A and of the output come in groups of `group_rows`
  // (one expert each, a multiple of 128); group g multiplies B rows [g * group_n, (g + 1) * group_n)
  // and only its first group_counts[g] rows are live (tiles beyond them are skipped).
  //   moe_mode 1: columns are (gate, up) pairs; writes silu(gate) * up to out_bf16[m][n / 2]
  //   moe_mode 2: combine: row m is token meta[2m+1] of rank meta[2m]; adds gate_w[m] * value into
  //               that rank's fp32 tensor at heap offset sym_off ([token][ldc]); ends with a barrier
  int group_rows;
  int group_n;
  const int* group_counts;
  int moe_mode;
  const int* meta;
  const float* gate_w;
  int wait_ready;            // fused all-reduce: check the peers' "finished reading" signals before the first add
  // Fused collective epilogue (tensor-parallel row-parallel GEMMs): instead of storing, add the tile
  // into an fp32 tensor [*, ldc] at byte offset sym_off of the symmetric heap.
  //   SYM_ALLREDUCE : into every rank's replica (multimem.red through the switch where available)
  //   SYM_RSCATTER  : row m goes to rank m / rows_per_rank, local row m % rows_per_rank
  //   SYM_RSCATTER_ROWS : row m goes to rank m / rows_per_rank, same row m (the owner keeps its rows in
  //                   place in a full-size tensor: the sequence-sharded residual stream of prefill)
  // The kernel then ends with a cross-rank barrier.
  int sym_mode;
  int rows_per_rank;
  size_t sym_off;
  // All-gather fused into the A operand (sequence-sharded prefill): rows of A are pushed into this
  // rank's memory by their owners (rank m / ag_rows_per_rank, see rmsnorm_allgather_kernel); the
  // producer warp waits for the owner's counter to reach ag_epoch before it loads a tile, and the walk
  // over m tiles starts at this rank's own rows, which need no transfer.  0 = off.
  int ag_rows_per_rank;
  uint32_t ag_epoch;
  SymTable sym;
};
enum { SYM_NONE = 0, SYM_ALLREDUCE = 1, SYM_RSCATTER = 2, SYM_RSCATTER_ROWS = 3 };
__device__ __forceinline__ int rs_row(const GemmEpi& e, int m) { return e.sym_mode == SYM_RSCATTER ? m % e.rows_per_rank : m; }

constexpr int BM = 128, BK = 64;
constexpr int kMaxLiveTiles = 2048;   // grouped mode: 128-row tiles with live rows, listed in shared memory

// Accumulating epilogues (fused collectives, split K) go through shared memory so that one warp
// instruction adds 4 rows x 128 contiguous bytes instead of 32 rows x 16 bytes: reductions that
// cross NVLink are sent as full packets, and local ones touch whole sectors.  `stage` is this warp's
// 32 x 32 fp32 patch; lane = accumulator row on the way in, (row group, float4 column) on the way out.
__device__ __forceinline__ void epilogue_chunk_red(const GemmEpi& e, float* stage, int m_warp0, int n0, int M, int N,
                                                   const uint32_t (&r)[32], bool first_split) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int c4 = 0; c4 < 8; c4++)
    *(float4*)(stage + lane * 32 + ((c4 ^ (lane & 7)) << 2)) =
        make_float4(__uint_as_float(r[4 * c4]), __uint_as_float(r[4 * c4 + 1]), __uint_as_float(r[4 * c4 + 2]),
                    __uint_as_float(r[4 * c4 + 3]));
  __syncwarp();
  const int c4 = lane & 7, n = n0 + c4 * 4;
  if (n < N) {
    const bool sym = e.sym_mode != SYM_NONE;
    float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
    if (e.bias && first_split && (!sym || e.sym.rank == 0)) b = *(const float4*)(e.bias + n);
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const int row = (lane >> 3) + 4 * i, m = m_warp0 + row;
      if (m >= M) break;
      float4 o = *(const float4*)(stage + row * 32 + ((c4 ^ (row & 7)) << 2));
      o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w;
      if (!sym) {
        asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(e.out_f32 + (size_t)m * e.ldc + n),
                     "f"(o.x), "f"(o.y), "f"(o.z), "f"(o.w) : "memory");
      } else if (e.sym_mode == SYM_ALLREDUCE) {
        sym_red_all_f32x4(e.sym, e.sym_off + ((size_t)m * e.ldc + n) * 4, o);
      } else {
        sym_red_to_f32x4(e.sym, m / e.rows_per_rank, e.sym_off + ((size_t)rs_row(e, m) * e.ldc + n) * 4, o);
      }
    }
  }
  __syncwarp();
}

// moe_mode 1: 32 accumulator columns are 16 (gate, up) pairs of one row.
__device__ __forceinline__ void epilogue_row_swiglu(const GemmEpi& e, int m, int n0, const uint32_t (&r)[32]) {
  uint4 o[2];
  __nv_bfloat162* p = (__nv_bfloat162*)o;
#pragma unroll
  for (int j = 0; j < 8; j++) {
    const float g0 = __uint_as_float(r[4 * j]), u0 = __uint_as_float(r[4 * j + 1]);
    const float g1 = __uint_as_float(r[4 * j + 2]), u1 = __uint_as_float(r[4 * j + 3]);
    p[j] = __floats2bfloat162_rn(silu(g0) * u0, silu(g1) * u1);
  }
  uint4* dst = (uint4*)(e.out_bf16 + (size_t)m * e.ldc + (n0 >> 1));
  dst[0] = o[0];
  dst[1] = o[1];
}

// moe_mode 2: like epilogue_chunk_red, but every row has its own destination (rank, token) and weight.
__device__ __forceinline__ void epilogue_chunk_combine(const GemmEpi& e, float* stage, int m_warp0, int live_end,
                                                       int n0, int N, const uint32_t (&r)[32]) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int c4 = 0; c4 < 8; c4++)
    *(float4*)(stage + lane * 32 + ((c4 ^ (lane & 7)) << 2)) =
        make_float4(__uint_as_float(r[4 * c4]), __uint_as_float(r[4 * c4 + 1]), __uint_as_float(r[4 * c4 + 2]),
                    __uint_as_float(r[4 * c4 + 3]));
  __syncwarp();
  const int c4 = lane & 7, n = n0 + c4 * 4;
  if (n < N) {
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const int row = (lane >> 3) + 4 * i, m = m_warp0 + row;
      if (m >= live_end) break;
      const int dst = e.meta[2 * m], tok = e.meta[2 * m + 1];
      const float w = e.gate_w[m];
      float4 o = *(const float4*)(stage + row * 32 + ((c4 ^ (row & 7)) << 2));
      o.x *= w; o.y *= w; o.z *= w; o.w *= w;
      sym_red_to_f32x4(e.sym, dst, e.sym_off + ((size_t)tok * e.ldc + n) * 4, o);
    }
  }
  __syncwarp();
}

// Transposed epilogue: this thread holds, for output column `n` (a weight row), the values of the 32
// output rows t0..t0+31 (tokens).  Consecutive lanes hold consecutive columns, so each of the 32
// stores of a warp covers 128 contiguous bytes.
__device__ __forceinline__ void epilogue_col(const GemmEpi& e, int n, int t0, int n_cols, int n_rows,
                                             const uint32_t (&r)[32], bool first_split) {
  if (n >= n_cols) return;
  const bool sym = e.sym_mode != SYM_NONE;
  const float b = (e.bias && first_split && (!sym || e.sym.rank == 0)) ? e.bias[n] : 0.f;
  // fully unrolled with a predicate per row: an index that is not a compile-time constant would put r[] on the stack
#pragma unroll
  for (int j = 0; j < 32; j++) {
    const int t = t0 + j;
    if (t >= n_rows) continue;
    float x = __uint_as_float(r[j]) + b;
    if (sym) {
      const int owner = e.sym_mode != SYM_ALLREDUCE ? t / e.rows_per_rank : 0;
      const int lrow = rs_row(e, t);
      const size_t off = e.sym_off + ((size_t)lrow * e.ldc + n) * 4;
      if (e.sym_mode == SYM_ALLREDUCE) sym_red_all_f32(e.sym, off, x);
      else sym_red_to_f32(e.sym, owner, off, x);
      continue;
    }
    const size_t idx = (size_t)t * e.ldc + n;
    if (e.splitk_red) {
      asm volatile("red.relaxed.gpu.global.add.f32 [%0], %1;" ::"l"(e.out_f32 + idx), "f"(x) : "memory");
      continue;
    }
    if (e.act == ACT_GELU) x = gelu_tanh(x);
    if (e.resid_f32) x += e.resid_f32[idx];
    if (e.resid_bf16) x += __bfloat162float(e.resid_bf16[idx]);
    if (e.out_f32) e.out_f32[idx] = e.accumulate ? e.out_f32[idx] + x : x;
    if (e.out_bf16) e.out_bf16[idx] = __float2bfloat16(x);
  }
}

__device__ __forceinline__ void epilogue_row(const GemmEpi& e, int m, int n0, int M, int N, const uint32_t (&r)[32],
                                             bool first_split, const float* bias_s = nullptr) {
  if (e.transposed) {
    epilogue_col(e, m, n0, M, N, r, first_split);
    return;
  }
  if (m >= M) return;
  const size_t base = (size_t)m * e.ldc + n0;
  float v[32];
#pragma unroll
  for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]);
  const bool full = n0 + 32 <= N;
  if (e.splitk_red && e.sym_mode == SYM_NONE) {
    const bool add_bias = e.bias && first_split;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      if (n0 + j >= N) continue;
      float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
      if (add_bias) {
        const float4 b = *(const float4*)(e.bias + n0 + j);
        o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w;
      }
      asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(e.out_f32 + base + j), "f"(o.x),
                   "f"(o.y), "f"(o.z), "f"(o.w) : "memory");
    }
    return;
  }
  if (e.sym_mode != SYM_NONE) {
    const bool add_bias = e.bias && e.sym.rank == 0 && first_split;
    const int owner = e.sym_mode != SYM_ALLREDUCE ? m / e.rows_per_rank : 0;
    const int lrow = rs_row(e, m);
    const size_t off = e.sym_off + ((size_t)lrow * e.ldc + n0) * 4;
    if (full) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        if (add_bias) {
          const float4 b = *(const float4*)(e.bias + n0 + j);
          o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w;
        }
        if (e.sym_mode == SYM_ALLREDUCE) sym_red_all_f32x4(e.sym, off + j * 4, o);
        else sym_red_to_f32x4(e.sym, owner, off + j * 4, o);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; j++) {
        if (n0 + j >= N) continue;
        const float x = v[j] + (add_bias ? e.bias[n0 + j] : 0.f);
        if (e.sym_mode == SYM_ALLREDUCE) sym_red_all_f32(e.sym, off + j * 4, x);
        else sym_red_to_f32(e.sym, owner, off + j * 4, x);
      }
    }
    return;
  }
  if (full) {
    if (e.bias) {      // bias_s: this chunk's 32 values staged in shared memory by the warp (broadcast reads)
      const float* bp = bias_s ? bias_s : e.bias + n0;
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const float4 b = *(const float4*)(bp + j);
        v[j] += b.x; v[j + 1] += b.y; v[j + 2] += b.z; v[j + 3] += b.w;
      }
    }
    if (e.act == ACT_GELU) {
#pragma unroll
      for (int j = 0; j < 32; j++) v[j] = gelu_tanh(v[j]);
    }
    if (e.resid_f32) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const float4 b = *(const float4*)(e.resid_f32 + base + j);
        v[j] += b.x; v[j + 1] += b.y; v[j + 2] += b.z; v[j + 3] += b.w;
      }
    }
    if (e.resid_bf16) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        const uint4 b = *(const uint4*)(e.resid_bf16 + base + j);
        const __nv_bfloat162* p = (const __nv_bfloat162*)&b;
#pragma unroll
        for (int q = 0; q < 4; q++) {
          const float2 f = __bfloat1622float2(p[q]);
          v[j + 2 * q] += f.x;
          v[j + 2 * q + 1] += f.y;
        }
      }
    }
    if (e.out_f32) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        if (e.accumulate) {
          const float4 p = *(const float4*)(e.out_f32 + base + j);
          o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w;
        }
        *(float4*)(e.out_f32 + base + j) = o;
      }
    }
    if (e.out_bf16) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        uint4 o;
        __nv_bfloat162* p = (__nv_bfloat162*)&o;
#pragma unroll
        for (int q = 0; q < 4; q++) p[q] = __floats2bfloat162_rn(v[j + 2 * q], v[j + 2 * q + 1]);
        *(uint4*)(e.out_bf16 + base + j) = o;
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; j++) {
      if (n0 + j >= N) continue;
      float x = v[j];
      if (e.bias) x += e.bias[n0 + j];
      if (e.act == ACT_GELU) x = gelu_tanh(x);
      if (e.resid_f32) x += e.resid_f32[base + j];
      if (e.resid_bf16) x += __bfloat162float(e.resid_bf16[base + j]);
      if (e.out_f32) e.out_f32[base + j] = e.accumulate ? e.out_f32[base + j] + x : x;
      if (e.out_bf16) e.out_bf16[base + j] = __float2bfloat16(x);
    }
  }
}

// Persistent kernel: each CTA walks output tiles (m fastest) with a shared-memory ring that keeps
// running across tiles and two accumulator stages in tensor memory, so the epilogue of one tile
// overlaps the main loop of the next.
// AROWS = 64 (at most 64 rows of A in all): the TMA box of A is 64 rows and a stage keeps only those
// 8 KB; the MMA still reads a 128-row operand, whose upper half is whatever follows in shared memory
// (the next stage); rows are independent and rows >= M are never written, so that is harmless, and the
// 8 KB saved per stage buy more stages, i.e. more weight bytes in flight per SM, which is what bounds a
// GEMM with few rows (bytes in flight = bandwidth x latency).
// KSUB = 2 (with AROWS = 64): a stage holds two 64-wide K blocks of each operand behind one barrier.  The thread
// that issues the MMAs spends about 540 cycles per K block on a narrow tile (measured with clock64 stamps: some 55
// per tcgen05.mma, the rest on the barrier wait, the fence and the commit), more than the tensor core needs for
// four narrow MMAs (220 cycles at N = 64), and the producer thread 420; fewer, larger stages halve that overhead.
// MN = true: both operands are given MN-major (A as [K][M], B as [K][N], row-major): the form of dW = dy^T x, where dy
// and x are read as they lie in memory instead of through transposed copies.  A stage then holds, per operand,
// 64-column blocks of [64 k rows][128 bytes] (one TMA box each), which the MMA reads through MN-major descriptors.
template <int BN, int STAGES, int AROWS, int KSUB, bool MN = false>
__global__ void __launch_bounds__(192) gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA,
                                                         const __grid_constant__ CUtensorMap tmB,
                                                         const GemmEpi epi, int M, int N, int K, int splits,
                                                         int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  constexpr int A_SUB = AROWS * BK * 2, B_SUB = BN * BK * 2;      // one 64-wide K block of each operand
  constexpr int A_BYTES = KSUB * A_SUB, B_BYTES = KSUB * B_SUB, BKS = BK * KSUB;
  uint8_t* sA = smem;
  uint8_t* sB = smem + STAGES * A_BYTES;
  uint64_t* bars = (uint64_t*)(sB + STAGES * B_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* tfull = bars + 2 * STAGES;       // [2]
  uint64_t* tempty = bars + 2 * STAGES + 2;  // [2]
  uint32_t* tmem_holder = (uint32_t*)(bars + 2 * STAGES + 4);
  volatile int* abort_flag = (volatile int*)(tmem_holder + 1);
  float* stage_all = (float*)(bars + 2 * STAGES + 6);   // 4 epilogue warps x 32 x 32 fp32, 16-byte aligned
  int* live_m = (int*)(stage_all + 4 * 1024);            // grouped mode: first row of every live 128-row tile
  __shared__ int s_n_live;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KB = (K + BKS - 1) / BKS;               // K in stage units
  int tiles_m = (M + BM - 1) / BM;
  const int tiles_n = (N + BN - 1) / BN;
  int n_tiles = tiles_m * tiles_n * splits;   // work items: (output tile, K split), split fastest
  const int kps = (KB + splits - 1) / splits;
  // fused all-gather: start the walk over m tiles at this rank's own rows
  const int m_rot = epi.ag_rows_per_rank ? ((epi.sym.rank * epi.ag_rows_per_rank) / BM) % tiles_m : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) {
      mbar_init(smem_u32(full + s), 1);
      mbar_init(smem_u32(empty + s), 1);
    }
    for (int s = 0; s < 2; s++) {
      mbar_init(smem_u32(tfull + s), 1);
      mbar_init(smem_u32(tempty + s), 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_holder), 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  // Set-up above touches only this CTA's shared and tensor memory; the operands come from earlier kernels.
  pdl_trigger();
  pdl_wait();

  if (epi.group_rows) {
    // Only the tiles that hold live rows are work items: list them once (the counts are final now).
    if (threadIdx.x == 0) {
      int n = 0;
      const int groups = M / epi.group_rows;
      for (int g = 0; g < groups; g++) {
        const int cnt = min(epi.group_counts[g], epi.group_rows);
        for (int r = 0; r < cnt && n < kMaxLiveTiles; r += BM) live_m[n++] = g * epi.group_rows + r;
      }
      s_n_live = n;
    }
    __syncthreads();
    tiles_m = s_n_live;
    n_tiles = tiles_m * tiles_n;
  }

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0, ag_seen = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_tiles && ok; item += gridDim.x) {
        const int tile = item / splits, sp = item - tile * splits;
        // Dense: m fastest (B tile shared by the CTAs of a wave).  Grouped: n fastest, so that the CTAs of a wave
        // sweep the few row tiles of ONE expert across all its columns: that expert's weights and rows are
        // read from HBM once and stay in L2, instead of every expert's rows being re-read for each column tile.
        const int m0 = epi.group_rows ? live_m[tile / tiles_n] : ((tile % tiles_m + m_rot) % tiles_m) * BM;
        const int n0 = epi.group_rows ? (tile % tiles_n) * BN : (tile / tiles_m) * BN;
        if (epi.ag_rows_per_rank) {       // rows of this tile come from their owners' all-gather pushes
          const int o0 = m0 / epi.ag_rows_per_rank, o1 = min(m0 + BM - 1, M - 1) / epi.ag_rows_per_rank;
          for (int o = o0; o <= o1 && ok; o++) {
            if (ag_seen & (1u << o)) continue;
            if (!sym_wait_rows(epi.sym, o, epi.ag_epoch)) {
              *abort_flag = 1;
              ok = false;
            }
            ag_seen |= 1u << o;
          }
          if (!ok) break;
          asm volatile("fence.proxy.async.global;" ::: "memory");   // peers' stores -> this CTA's TMA reads
        }
        int b_row = n0;
        if (epi.group_rows) b_row += (m0 / epi.group_rows) * epi.group_n;
        const int kb0 = sp * kps, kb1 = min(KB, kb0 + kps);
        for (int kb = kb0; kb < kb1; kb++, it++) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(smem_u32(empty + s), ph ^ 1, abort_flag)) { ok = false; break; }
          mbar_expect_tx(smem_u32(full + s), A_BYTES + B_BYTES);
          if constexpr (MN) {                   // coordinates are (mn, k): 64-column blocks of 64 k rows
#pragma unroll
            for (int hb = 0; hb < BM / 64; hb++)
              tma_load_2d(smem_u32(sA + s * A_BYTES + hb * 8192), &tmA, smem_u32(full + s), m0 + hb * 64, kb * BK);
#pragma unroll
            for (int hb = 0; hb < BN / 64; hb++)
              tma_load_2d(smem_u32(sB + s * B_BYTES + hb * 8192), &tmB, smem_u32(full + s), b_row + hb * 64, kb * BK);
          } else {
#pragma unroll
            for (int u = 0; u < KSUB; u++) {      // a block past the end of K is filled with zeros by the TMA unit
              tma_load_2d(smem_u32(sA + s * A_BYTES + u * A_SUB), &tmA, smem_u32(full + s), kb * BKS + u * BK, m0);
              tma_load_2d(smem_u32(sB + s * B_BYTES + u * B_SUB), &tmB, smem_u32(full + s), kb * BKS + u * BK, b_row);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_bf16(BM, BN) | (MN ? ((1u << 15) | (1u << 16)) : 0u);   // bits 15 / 16: A / B MN-major
      uint32_t it = 0, tcount = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_tiles && ok; item += gridDim.x) {
        const int tile = item / splits, sp = item - tile * splits;
        const int kb0 = sp * kps, kb1 = min(KB, kb0 + kps);
        const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
        tcount++;
        if (!mbar_wait(smem_u32(tempty + acc), aph ^ 1, abort_flag)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; kb++, it++) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(smem_u32(full + s), ph, abort_flag)) { ok = false; break; }
          tc_fence_after();
          if constexpr (MN) {
            // 64-column blocks 8192 bytes apart, 8-row groups along K 1024 bytes apart; a K step of 16 rows is 2048 bytes on
            const uint64_t ad = smem_desc_sw128_mn(smem_u32(sA + s * A_BYTES), 8192);
            const uint64_t bd = smem_desc_sw128_mn(smem_u32(sB + s * B_BYTES), 8192);
#pragma unroll
            for (int k = 0; k < BK / 16; k++)
              umma_bf16(d_tmem, ad + 128 * k, bd + 128 * k, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
          } else {
#pragma unroll
            for (int u = 0; u < KSUB; u++) {
              const uint64_t ad = smem_desc_sw128(smem_u32(sA + s * A_BYTES + u * A_SUB));
              const uint64_t bd = smem_desc_sw128(smem_u32(sB + s * B_BYTES + u * B_SUB));
#pragma unroll
              for (int k = 0; k < BK / 16; k++)
                umma_bf16(d_tmem, ad + 2 * k, bd + 2 * k, idesc, (kb != kb0 || u != 0 || k != 0) ? 1u : 0u);
            }
          }
          umma_commit(smem_u32(empty + s));
        }
        umma_commit(smem_u32(tfull + acc));   // released even after a failed wait; the flag says why
      }
    }
  } else {
    const int q = warp & 3;
    float* stage = stage_all + q * 1024;
    const bool red_path = !epi.transposed && (epi.sym_mode != SYM_NONE || epi.splitk_red);
    bool ready_checked = !(epi.sym_mode != SYM_NONE && epi.wait_ready);
    uint32_t tcount = 0;
    for (int item = blockIdx.x; item < n_tiles; item += gridDim.x) {
      const int tile = item / splits, sp = item - tile * splits;
      const int m0 = epi.group_rows ? live_m[tile / tiles_n] : ((tile % tiles_m + m_rot) % tiles_m) * BM;
      const int n0 = epi.group_rows ? (tile % tiles_n) * BN : (tile / tiles_m) * BN;
      int live_end = M;                       // rows below this index are written
      if (epi.group_rows) {
        const int g = m0 / epi.group_rows;
        live_end = g * epi.group_rows + min(epi.group_counts[g], epi.group_rows);
      }
      const uint32_t acc = tcount & 1, aph = (tcount >> 1) & 1;
      tcount++;
      bool ok = mbar_wait(smem_u32(tfull + acc), aph, abort_flag);
      ok = __all_sync(0xffffffffu, ok && !*abort_flag);  // tcgen05.ld needs the whole warp
      if (!ok) break;
      tc_fence_after();
      if (!ready_checked) {          // once per warp, before its first remote add
        if (lane == 0) sym_wait_ready(epi.sym);
        __syncwarp();
        ready_checked = true;
      }
      const int m = m0 + q * 32 + lane;
      const bool plain = !(epi.moe_mode == 2 || epi.moe_mode == 1 || epi.act == ACT_SWIGLU_PAIR || red_path || epi.transposed);
      const bool stage_bias = plain && epi.bias != nullptr;
      if (stage_bias) {              // the tile's bias values, once per tile, into this warp's staging area
        __syncwarp();
#pragma unroll
        for (int j = 0; j < BN / 32; j++) {
          const int n = n0 + j * 32 + lane;
          stage[j * 32 + lane] = n < N ? epi.bias[n] : 0.f;
        }
        __syncwarp();
      }
      auto process = [&](int c, const uint32_t (&r)[32]) {
        if (n0 + c * 32 >= N) return;
        if (epi.moe_mode == 2) epilogue_chunk_combine(epi, stage, m0 + q * 32, live_end, n0 + c * 32, N, r);
        else if (epi.moe_mode == 1 || epi.act == ACT_SWIGLU_PAIR) { if (m < live_end) epilogue_row_swiglu(epi, m, n0 + c * 32, r); }
        else if (red_path) epilogue_chunk_red(epi, stage, m0 + q * 32, n0 + c * 32, live_end, N, r, sp == 0);
        else epilogue_row(epi, m, n0 + c * 32, live_end, N, r, sp == 0, stage_bias ? stage + c * 32 : nullptr);
      };
      // two register buffers: the tensor-memory load of the next 32 columns is in flight while this chunk is finished
      const uint32_t t_addr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
      uint32_t ra[32], rb[32];
      tmem_ld32(t_addr, ra);
#pragma unroll 1
      for (int c = 0; c < BN / 32; c += 2) {
        tmem_ld_wait();
        tmem_ld32(t_addr + (uint32_t)((c + 1) * 32), rb);
        process(c, ra);
        tmem_ld_wait();
        if (c + 2 < BN / 32) tmem_ld32(t_addr + (uint32_t)((c + 2) * 32), ra);
        process(c + 1, rb);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(tempty + acc));
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 2 * BN);
  if (threadIdx.x == 0 && *abort_flag && status) atomicExch(status, (int)B200_ERR_TIMEOUT_MMA);
  if (epi.sym_mode != SYM_NONE) sym_kernel_end_barrier(epi.sym, 0, gridDim.x, epi.wait_ready != 0);
}

static int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

static bool gemm_deep_enabled() {      // B200_GEMM_DEEP=0: measurement aid, the 128-row box for every M
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("B200_GEMM_DEEP");
    on = (e && e[0] == '0') ? 0 : 1;
  }
  return on == 1;
}

template <int BN, int STAGES, int AROWS = 128, int KSUB = 1, bool MN = false>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmEpi& e, int M, int N, int K,
                       int splits, int* status, cudaStream_t st) {
  // AROWS = 64: no tile list (never grouped); the last stage's 128-row operand read runs 8 KB past its A tile and
  // lands in the B region, which follows the A region
  constexpr size_t smem = 1024 + (size_t)STAGES * KSUB * (AROWS * BK * 2 + BN * BK * 2) + (2 * STAGES + 6) * 8 + 4 * 32 * 32 * 4 +
                          (AROWS == 128 ? kMaxLiveTiles * 4 : 0);
  static_assert(smem <= 232448, "shared memory per CTA");
  auto kern = gemm_bf16_kernel<BN, STAGES, AROWS, KSUB, MN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  const int n_tiles = ((N + BN - 1) / BN) * ((M + BM - 1) / BM) * splits;
  const int grid = n_tiles < sm_count() ? n_tiles : sm_count();
  return launch_pdl(kern, dim3(grid), dim3(192), smem, st, ta, tb, e, M, N, K, splits, status);
}

// A [M][K] (row stride lda), B [N][K] (row stride ldb), bf16, K-major.  Strides in elements and
// multiples of 8; base pointers 16-byte aligned.  tile_n: 0 = choose, else 64 / 128 / 256.
// `status` is a device int the kernel sets non-zero if one of its waits ran out.
B200_API int b200_gemm_bf16(const void* A, const void* B, int M, int N, int K, int lda, int ldb, float* out_f32,
                            void* out_bf16, int ldc, const float* bias, const float* resid_f32,
                            const void* resid_bf16, int act, int accumulate, int tile_n, int split_k, int* status,
                            int sym_mode, const SymTable* sym, size_t sym_off, int rows_per_rank, int wait_ready,
                            int ag_rows_per_rank, int ag_epoch, int mn_major, cudaStream_t st) {
  if (M <= 0 || N <= 0 || K <= 0 || (lda % 8) || (ldb % 8) || (!mn_major && (K % 8))) return B200_ERR_BAD_ARG;
  if (mn_major) {
    // D[M][N] = sum_k A[k][m] * B[k][n]: A is [K][M] (row stride lda), B is [K][N] (row stride ldb).  Plain epilogues only.
    if (sym_mode != SYM_NONE || ag_rows_per_rank || tile_n < 0 || split_k > 1 || act == ACT_SWIGLU_PAIR || (M % 8) || (N % 8))
      return B200_ERR_BAD_ARG;
    if ((out_bf16 && (ldc % 8)) || (out_f32 && (ldc % 4)) || (N % 4)) return B200_ERR_BAD_ARG;
    CUtensorMap ta, tb;
    int rc = make_tmap_2d(&ta, A, 2, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, BK, 64, true);
    if (rc) return rc;
    rc = make_tmap_2d(&tb, B, 2, (uint64_t)K, (uint64_t)N, (uint64_t)ldb * 2, BK, 64, true);
    if (rc) return rc;
    GemmEpi e = {};
    e.out_f32 = out_f32; e.out_bf16 = (__nv_bfloat16*)out_bf16; e.bias = bias; e.resid_f32 = resid_f32;
    e.resid_bf16 = (const __nv_bfloat16*)resid_bf16; e.ldc = ldc; e.act = act; e.accumulate = accumulate; e.rows_per_rank = 1;
    const long t256 = (long)((N + 255) / 256) * ((M + 127) / 128);
    if ((tile_n == 256 || (tile_n == 0 && N >= 256 && t256 >= 148)))
      return launch_gemm<256, 4, 128, 1, true>(ta, tb, e, M, N, K, 1, status, st);
    return launch_gemm<128, 6, 128, 1, true>(ta, tb, e, M, N, K, 1, status, st);
  }
  if ((out_bf16 && (ldc % 8)) || (out_f32 && (ldc % 4))) return B200_ERR_BAD_ARG;
  if (N % 4) return B200_ERR_BAD_ARG;
  if (sym_mode != SYM_NONE && (!sym || (ldc % 4) || (sym_off % 16))) return B200_ERR_BAD_ARG;
  if (ag_rows_per_rank < 0 || (ag_rows_per_rank > 0 && (!sym || tile_n == -1))) return B200_ERR_BAD_ARG;
  if (act == ACT_SWIGLU_PAIR && (!out_bf16 || out_f32 || bias || resid_f32 || resid_bf16 || accumulate || sym_mode != SYM_NONE ||
                                 tile_n == -1 || (N % 32) || (ldc % 8)))
    return B200_ERR_BAD_ARG;
  // Few tokens: stream the weights as the 128-row operand and the tokens as the narrow one, so that
  // most of every pipeline stage is weight bytes from HBM and none of the tile is padding.
  // Measured on the decode shapes (64 tokens), the swapped form is only faster for long K with few
  // rows, so it is opt-in: tile_n = -1.
  const bool swap = tile_n == -1 && M <= 256 && N >= 128;
  if (swap) {
    tile_n = M <= 64 ? 64 : M <= 128 ? 128 : 256;
    const void* tp = A; A = B; B = tp;
    const int ti = lda; lda = ldb; ldb = ti;
    const int tm = M; M = N; N = tm;
  }
  const long tiles_m = (M + 127) / 128;
  // Split K when the output tiles alone would leave most SMs idle and the epilogue is (or can be
  // turned into) a pure accumulation: the fused collectives already add into their destination, and
  // an in-place fp32 residual add (resid_f32 == out_f32) is the same thing as adding into out_f32.
  const bool red_ok = sym_mode != SYM_NONE ||
                      (out_f32 && !out_bf16 && !resid_bf16 && act == 0 &&
                       ((accumulate && !resid_f32) || (!accumulate && resid_f32 == out_f32)));
  if (tile_n == 0) {
    const long tiles256 = (long)((N + 255) / 256) * tiles_m, tiles128 = (long)((N + 127) / 128) * tiles_m;
    if (M <= 64 && !swap) {
      // One row tile, weight-streaming.  Measured inside CUDA graphs on the 8B decode shapes at 64 rows: where K may
      // be split, 128-wide tiles with 3-4 splits win (QKV 17 us against 25, down 28 against 38); where it may
      // not, the widest tile that still leaves about a hundred CTAs (gate/up 49 us at 256 against 54 at 128).
      if (red_ok) tile_n = N >= 128 ? 128 : 64;
      else tile_n = (N >= 256 && tiles256 >= 100) ? 256 : (N >= 128 && tiles128 >= 100) ? 128 : 64;
    } else {
      tile_n = (N >= 256 && tiles256 >= 148) ? 256 : (N >= 128 && tiles128 >= 148) ? 128 : (N > 64 ? 128 : 64);
      // Few tiles (decode batches): narrower tiles put more SMs on the weight stream.
      if (tile_n == 128 && tiles128 <= 74) tile_n = 64;
    }
  }
  CUtensorMap ta, tb;
  const bool few_rows = M <= 64 && gemm_deep_enabled();      // 64-row A box, deeper pipeline
  int rc = make_tmap_2d(&ta, A, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, few_rows ? 64 : BM, BK, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tb, B, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, (uint32_t)tile_n, BK, true);
  if (rc) return rc;
  GemmEpi e;
  e.out_f32 = out_f32; e.out_bf16 = (__nv_bfloat16*)out_bf16; e.bias = bias; e.resid_f32 = resid_f32;
  e.resid_bf16 = (const __nv_bfloat16*)resid_bf16; e.ldc = ldc; e.act = act; e.accumulate = accumulate;
  e.sym_mode = sym_mode; e.rows_per_rank = rows_per_rank > 0 ? rows_per_rank : 1; e.sym_off = sym_off;
  const long n_out_tiles = (long)((N + tile_n - 1) / tile_n) * tiles_m;
  const bool two_k = few_rows && tile_n != 256;      // two K blocks per stage (narrow tiles)
  const int k_unit = two_k ? 2 * BK : BK, min_per_split = two_k ? 4 : 8;
  const int KBt = (K + k_unit - 1) / k_unit;                       // K in the kernel's stage units
  int splits = 1;
  if (split_k > 0) splits = split_k;
  else if (red_ok && n_out_tiles <= 74) splits = (int)(148 / n_out_tiles);
  if (split_k <= 0 && sym_mode != SYM_NONE && splits > 2) splits = 2;   // every split's tile crosses NVLink
  if (splits > 1) {
    if (!red_ok) return B200_ERR_BAD_ARG;
    if (splits > 16) splits = 16;
    while (splits > 1 && KBt / splits < min_per_split) splits--;   // keep at least 8 K blocks (of 64) per split
    const int kps = (KBt + splits - 1) / splits;
    splits = (KBt + kps - 1) / kps;                            // no empty split
  }
  e.splitk_red = (splits > 1 && sym_mode == SYM_NONE) ? 1 : 0;
  e.transposed = swap ? 1 : 0;
  e.group_rows = 0; e.group_n = 0; e.group_counts = nullptr; e.moe_mode = 0; e.meta = nullptr; e.gate_w = nullptr;
  e.wait_ready = (sym_mode != SYM_NONE) ? wait_ready : 0;
  e.ag_rows_per_rank = ag_rows_per_rank; e.ag_epoch = (uint32_t)ag_epoch;
  if (sym_mode != SYM_NONE || ag_rows_per_rank > 0) {
    e.sym = *sym;
  } else {
    e.sym = SymTable{};
  }
  switch (tile_n) {
    case 256: return few_rows ? launch_gemm<256, 5, 64>(ta, tb, e, M, N, K, splits, status, st)
                              : launch_gemm<256, 4>(ta, tb, e, M, N, K, splits, status, st);
    case 128: return few_rows ? launch_gemm<128, 4, 64, 2>(ta, tb, e, M, N, K, splits, status, st)
                              : launch_gemm<128, 6>(ta, tb, e, M, N, K, splits, status, st);
    case 64: return few_rows ? launch_gemm<64, 6, 64, 2>(ta, tb, e, M, N, K, splits, status, st)
                             : launch_gemm<64, 8>(ta, tb, e, M, N, K, splits, status, st);
  }
  return B200_ERR_BAD_ARG;
}

// Grouped GEMM of a mixture-of-experts layer (see GemmEpi).  A [groups * group_rows][K] bf16 (row
// stride lda) holds each expert's gathered tokens, B [groups * N][K] bf16 its weights, counts[g] the
// live rows of group g (device memory, final before this kernel starts).
//   mode 1: B rows are interleaved (gate_0, up_0, gate_1, ...), N = 2 * ffn; out_bf16 [rows][ldc] gets
//           silu(gate) * up, N / 2 columns per row.
//   mode 2: N = d_model; row m is added, scaled by gate_w[m], into token meta[2m+1] of rank meta[2m]:
//           fp32 [tokens][ldc] at byte offset sym_off of that rank's symmetric heap.  The kernel ends
//           with the cross-rank barrier, so afterwards every rank's residual stream is complete.
B200_API int b200_moe_gemm(const void* A, const void* B, int groups, int group_rows, int N, int K, int lda, int ldb,
                           const int* counts, int mode, void* out_bf16, int ldc, const int* meta, const float* gate_w,
                           const SymTable* sym, size_t sym_off, int* status, cudaStream_t st) {
  if (groups <= 0 || group_rows <= 0 || group_rows % BM || N <= 0 || K <= 0 || (lda % 8) || (ldb % 8) || (K % 8) || (N % 4))
    return B200_ERR_BAD_ARG;
  if (mode == 1 ? (!out_bf16 || (ldc % 8) || (N % 32)) : (mode != 2 || !meta || !gate_w || !sym || (ldc % 4) || (sym_off % 16)))
    return B200_ERR_BAD_ARG;
  const int M = groups * group_rows;
  if ((long)groups * (group_rows / BM) > kMaxLiveTiles) return B200_ERR_BAD_ARG;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d(&ta, A, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, BM, BK, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tb, B, 2, (uint64_t)groups * N, (uint64_t)K, (uint64_t)ldb * 2, 128, BK, true);
  if (rc) return rc;
  GemmEpi e = {};
  e.out_bf16 = (__nv_bfloat16*)out_bf16; e.ldc = ldc;
  e.group_rows = group_rows; e.group_n = N; e.group_counts = counts; e.moe_mode = mode; e.meta = meta; e.gate_w = gate_w;
  e.rows_per_rank = 1;
  if (mode == 2) {
    e.sym_mode = SYM_ALLREDUCE;   // only so that the kernel ends with the cross-rank barrier
    e.sym = *sym;
    e.sym_off = sym_off;
  }
  return launch_gemm<128, 6>(ta, tb, e, M, N, K, 1, status, st);
}
