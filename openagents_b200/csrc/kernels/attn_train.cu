// Causal multi-head attention for training: forward (saving the log-sum-exp of every row) and backward
// (dQ, dK, dV), head size 64, bf16 in and out, fp32 accumulation and softmax.
//
// Layout: the fused projection output qkv [B*T][3][H][64] bf16 is read in place (no permute, no split), the attention
// output o and its gradient do are [B*T][H][64], the gradient dqkv has the layout of qkv, lse is [B][H][T] fp32.
//
// Flash-attention tiling with 64 x 64 blocks and four warps per CTA (a warp owns 16 rows of the block it accumulates):
//   forward      one CTA per (64 queries, head, sequence): S = Q K^T, online softmax, O += P V, lse = m + log(l)
//   backward dKV one CTA per (64 keys, head, sequence), looping over the query blocks at or after it:
//                P^T = exp(K Q^T - lse), dV += P^T dO, dP^T = V dO^T, dS^T = P^T (dP^T - D), dK += dS^T Q
//   backward dQ  one CTA per (64 queries, head, sequence), looping over the key blocks at or before it:
//                dS = P (dO V^T - D), dQ += dS K
// with D = rowsum(dO * O) from a small pre-pass.  The two backward kernels recompute P instead of exchanging it, so
// no atomics and no fp32 scratch are needed and the result is bit-reproducible.  Tiles are staged with cp.async
// (double-buffered) into 128-byte rows whose 16-byte chunks are XOR-swizzled by the row number, and fed to
// mma.sync m16n8k16 through ldmatrix; GPT-2-small spends under a tenth of its FLOPs here (the GEMMs are tcgen05).
//
// Math: apps/openagents.com/workers/api/src/cs336-a1-real-gradient-workload.ts:478-518 (forward: scores, causal
// softmax, weighted values) and :719-741 (backward: dV, dP, softmax Jacobian, dQ, dK).
#include "common.cuh"

using namespace b200;

namespace {

constexpr int HD = 64, BLK = 64, kThreads = 128;
constexpr int kTileBytes = BLK * HD * 2;     // 8 KB

struct AttnTrainArgs {
  const __nv_bfloat16* qkv;   // [B*T][3][H][64]
  __nv_bfloat16* o;           // forward: out; backward: in
  const __nv_bfloat16* d_o;   // backward
  __nv_bfloat16* dqkv;        // backward out
  float* lse;                 // [B][H][T]
  float* dsum;                // [B][H][T]  D = rowsum(dO * O)
  int B, T, H;
  float scale_log2;           // log2(e) / sqrt(64)
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// A tile is 64 rows x 128 bytes; the 16-byte chunk c of row r sits at chunk c ^ (r & 7).
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

// Copy a 64 x 64 bf16 tile (rows `row0`.., row stride `ld` elements) into a swizzled shared tile.
__device__ __forceinline__ void load_tile(uint32_t dst, const __nv_bfloat16* src, size_t ld) {
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int id = threadIdx.x + i * kThreads, row = id >> 3, chunk = id & 7;
    cp_async16(dst + tile_off(row, chunk), src + (size_t)row * ld + chunk * 8);
  }
}

// A fragments (16 rows x 64 columns = four k steps) of rows [r0, r0 + 16) of a tile.
__device__ __forceinline__ void load_a_frags(uint32_t tile, int r0, uint32_t (&a)[4][4]) {
  const int lane = threadIdx.x & 31;
  const int row = r0 + (lane & 15), half = lane >> 4;
#pragma unroll
  for (int ks = 0; ks < 4; ks++) ldsm4(tile + tile_off(row, ks * 2 + half), a[ks]);
}
// B fragments for C[m][n] = sum_k A[m][k] * X[n][k] (X row-major, "n rows, k contiguous"): n tiles nt, nt + 1 at k step ks.
// r = {b0, b1 of tile nt, b0, b1 of tile nt + 1}.
__device__ __forceinline__ void load_b_nk(uint32_t tile, int nt, int ks, uint32_t (&r)[4]) {
  const int lane = threadIdx.x & 31, mi = lane >> 3, rr = lane & 7;
  ldsm4(tile + tile_off((nt + (mi >> 1)) * 8 + rr, ks * 2 + (mi & 1)), r);
}
// B fragments for C[m][n] = sum_k A[m][k] * X[k][n] (X row-major, "k rows, n contiguous"): n tiles nt, nt + 1 at k step ks.
__device__ __forceinline__ void load_b_kn(uint32_t tile, int nt, int ks, uint32_t (&r)[4]) {
  const int lane = threadIdx.x & 31, mi = lane >> 3, rr = lane & 7;
  ldsm4t(tile + tile_off(ks * 16 + (mi & 1) * 8 + rr, nt + (mi >> 1)), r);
}

// acc[16 x 64] += A(16 x 64, fragments) * X^T with X [64 n][64 k] row-major in shared memory
__device__ __forceinline__ void gemm_nk(float (&acc)[8][4], const uint32_t (&a)[4][4], uint32_t tile) {
#pragma unroll
  for (int ks = 0; ks < 4; ks++)
#pragma unroll
    for (int nt = 0; nt < 8; nt += 2) {
      uint32_t b[4];
      load_b_nk(tile, nt, ks, b);
      mma16816(acc[nt], a[ks], b[0], b[1]);
      mma16816(acc[nt + 1], a[ks], b[2], b[3]);
    }
}
// acc[16 x 64] += A(16 x 64, fragments) * X with X [64 k][64 n] row-major in shared memory
__device__ __forceinline__ void gemm_kn(float (&acc)[8][4], const uint32_t (&a)[4][4], uint32_t tile) {
#pragma unroll
  for (int ks = 0; ks < 4; ks++)
#pragma unroll
    for (int nt = 0; nt < 8; nt += 2) {
      uint32_t b[4];
      load_b_kn(tile, nt, ks, b);
      mma16816(acc[nt], a[ks], b[0], b[1]);
      mma16816(acc[nt + 1], a[ks], b[2], b[3]);
    }
}
// Accumulator tile (16 x 64 fp32, C layout) -> A fragments of its bf16 rounding (16 x 64 = four k steps).
__device__ __forceinline__ void acc_to_a(const float (&c)[8][4], uint32_t (&a)[4][4]) {
#pragma unroll
  for (int ks = 0; ks < 4; ks++) {
    a[ks][0] = pack_bf16(c[2 * ks][0], c[2 * ks][1]);
    a[ks][1] = pack_bf16(c[2 * ks][2], c[2 * ks][3]);
    a[ks][2] = pack_bf16(c[2 * ks + 1][0], c[2 * ks + 1][1]);
    a[ks][3] = pack_bf16(c[2 * ks + 1][2], c[2 * ks + 1][3]);
  }
}
__device__ __forceinline__ void zero_acc(float (&c)[8][4]) {
#pragma unroll
  for (int i = 0; i < 8; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) c[i][j] = 0.f;
}
// Store a warp's 16 x 64 accumulator as bf16 rows [r0, r0 + 16) of a [rows][ld] tensor at column 0.
__device__ __forceinline__ void store_acc_bf16(__nv_bfloat16* dst, size_t ld, int r0, const float (&c)[8][4], float mul) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int nt = 0; nt < 8; nt++) {
    *(uint32_t*)(dst + (size_t)(r0 + g) * ld + nt * 8 + 2 * t) = pack_bf16(c[nt][0] * mul, c[nt][1] * mul);
    *(uint32_t*)(dst + (size_t)(r0 + g + 8) * ld + nt * 8 + 2 * t) = pack_bf16(c[nt][2] * mul, c[nt][3] * mul);
  }
}

// ---------------------------------------------------------------------------------------------------- forward
__global__ void __launch_bounds__(kThreads) attn_train_fwd_kernel(const AttnTrainArgs a) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sQ = smem_addr(smem), sK = sQ + kTileBytes, sV = sK + 2 * kTileBytes;   // K and V double-buffered
  const int qb = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;            // long rows first
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const size_t ld = (size_t)3 * a.H * HD;
  const __nv_bfloat16* base = a.qkv + (size_t)b * a.T * ld + (size_t)h * HD;
  const __nv_bfloat16 *Q = base + (size_t)qb * BLK * ld, *K = base + (size_t)a.H * HD, *V = base + (size_t)2 * a.H * HD;

  load_tile(sQ, Q, ld);
  load_tile(sK, K, ld);
  load_tile(sV, V, ld);
  cp_commit();
  uint32_t qa[4][4];
  float o[8][4];
  zero_acc(o);
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;      // rows g and g + 8 of this warp's 16
  for (int j = 0; j <= qb; j++) {
    const int buf = j & 1;
    if (j < qb) {                      // next key block into the other buffer
      load_tile(sK + (buf ^ 1) * kTileBytes, K + (size_t)(j + 1) * BLK * ld, ld);
      load_tile(sV + (buf ^ 1) * kTileBytes, V + (size_t)(j + 1) * BLK * ld, ld);
      cp_commit();
      cp_wait<1>();
    } else {
      cp_wait<0>();
    }
    __syncthreads();
    if (j == 0) load_a_frags(sQ, warp * 16, qa);
    float s[8][4];
    zero_acc(s);
    gemm_nk(s, qa, sK + buf * kTileBytes);
    // scale, causal mask on the diagonal block, online softmax in base 2
    const int r0 = warp * 16 + g;
    float mx0 = m0, mx1 = m1;
#pragma unroll
    for (int nt = 0; nt < 8; nt++) {
#pragma unroll
      for (int e = 0; e < 4; e++) {
        float v = s[nt][e] * a.scale_log2;
        if (j == qb && nt * 8 + 2 * t + (e & 1) > r0 + (e >> 1) * 8) v = -INFINITY;
        s[nt][e] = v;
      }
      mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
      mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float c0 = ex2(m0 - mx0), c1 = ex2(m1 - mx1);       // m = -inf on the first block: ex2(-inf) = 0
    m0 = mx0;
    m1 = mx1;
    float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
    for (int nt = 0; nt < 8; nt++) {
      s[nt][0] = ex2(s[nt][0] - m0);
      s[nt][1] = ex2(s[nt][1] - m0);
      s[nt][2] = ex2(s[nt][2] - m1);
      s[nt][3] = ex2(s[nt][3] - m1);
      rs0 += s[nt][0] + s[nt][1];
      rs1 += s[nt][2] + s[nt][3];
      o[nt][0] *= c0; o[nt][1] *= c0; o[nt][2] *= c1; o[nt][3] *= c1;
    }
    l0 = l0 * c0 + rs0;
    l1 = l1 * c1 + rs1;
    uint32_t pa[4][4];
    acc_to_a(s, pa);
    gemm_kn(o, pa, sV + buf * kTileBytes);
    __syncthreads();                   // everyone is done with this buffer before it is refilled
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float i0 = 1.f / l0, i1 = 1.f / l1;
  __nv_bfloat16* O = a.o + ((size_t)b * a.T + (size_t)qb * BLK) * a.H * HD + (size_t)h * HD;
  const int lane_r = warp * 16 + g;
#pragma unroll
  for (int nt = 0; nt < 8; nt++) {
    *(uint32_t*)(O + (size_t)lane_r * a.H * HD + nt * 8 + 2 * t) = pack_bf16(o[nt][0] * i0, o[nt][1] * i0);
    *(uint32_t*)(O + (size_t)(lane_r + 8) * a.H * HD + nt * 8 + 2 * t) = pack_bf16(o[nt][2] * i1, o[nt][3] * i1);
  }
  if (t == 0) {                        // log-sum-exp in base 2 of the scaled scores
    float* L = a.lse + ((size_t)b * a.H + h) * a.T + qb * BLK;
    L[lane_r] = m0 + log2f(l0);
    L[lane_r + 8] = m1 + log2f(l1);
  }
}

// ---------------------------------------------------------------------------------------------------- D = rowsum(dO * O)
__global__ void attn_train_dsum_kernel(const AttnTrainArgs a) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  const int total = a.B * a.T * a.H;
  if (row >= total) return;
  const int bt = row / a.H, h = row - bt * a.H;
  const __nv_bfloat162* po = (const __nv_bfloat162*)(a.o + (size_t)bt * a.H * HD + (size_t)h * HD);
  const __nv_bfloat162* pd = (const __nv_bfloat162*)(a.d_o + (size_t)bt * a.H * HD + (size_t)h * HD);
  const float2 x = __bfloat1622float2(po[lane]), y = __bfloat1622float2(pd[lane]);
  const float s = warp_sum(x.x * y.x + x.y * y.y);
  if (lane == 0) {
    const int bb = bt / a.T, tt = bt - bb * a.T;
    a.dsum[((size_t)bb * a.H + h) * a.T + tt] = s;
  }
}

// ---------------------------------------------------------------------------------------------------- backward: dK, dV
__global__ void __launch_bounds__(kThreads) attn_train_bwd_kv_kernel(const AttnTrainArgs a) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sK = smem_addr(smem), sV = sK + kTileBytes, sQ = sV + kTileBytes, sDO = sQ + 2 * kTileBytes;
  float* sL = (float*)(smem + 6 * kTileBytes);      // [2][64] lse, then [2][64] D
  float* sD = sL + 2 * BLK;
  const int kb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int nqb = a.T / BLK;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const size_t ld = (size_t)3 * a.H * HD, ldo = (size_t)a.H * HD;
  const __nv_bfloat16* base = a.qkv + (size_t)b * a.T * ld + (size_t)h * HD;
  const __nv_bfloat16 *Q = base, *K = base + (size_t)a.H * HD + (size_t)kb * BLK * ld, *V = base + (size_t)2 * a.H * HD + (size_t)kb * BLK * ld;
  const __nv_bfloat16* DO = a.d_o + (size_t)b * a.T * ldo + (size_t)h * HD;
  const float* L = a.lse + ((size_t)b * a.H + h) * a.T;
  const float* D = a.dsum + ((size_t)b * a.H + h) * a.T;

  auto stage = [&](int i, int buf) {     // query block i: Q, dO, lse, D
    load_tile(sQ + buf * kTileBytes, Q + (size_t)i * BLK * ld, ld);
    load_tile(sDO + buf * kTileBytes, DO + (size_t)i * BLK * ldo, ldo);
    if (threadIdx.x < 16) cp_async16(smem_addr(sL + buf * BLK) + threadIdx.x * 16, L + i * BLK + threadIdx.x * 4);
    else if (threadIdx.x < 32) cp_async16(smem_addr(sD + buf * BLK) + (threadIdx.x - 16) * 16, D + i * BLK + (threadIdx.x - 16) * 4);
  };
  load_tile(sK, K, ld);
  load_tile(sV, V, ld);
  stage(kb, 0);
  cp_commit();
  uint32_t ka[4][4], va[4][4];
  float dk[8][4], dv[8][4];
  zero_acc(dk);
  zero_acc(dv);
  const int key0 = warp * 16 + g;          // this thread's key rows (key0, key0 + 8) inside the block
  for (int i = kb; i < nqb; i++) {
    const int buf = (i - kb) & 1;
    if (i + 1 < nqb) {
      stage(i + 1, buf ^ 1);
      cp_commit();
      cp_wait<1>();
    } else {
      cp_wait<0>();
    }
    __syncthreads();
    if (i == kb) {
      load_a_frags(sK, warp * 16, ka);
      load_a_frags(sV, warp * 16, va);
    }
    const uint32_t tQ = sQ + buf * kTileBytes, tDO = sDO + buf * kTileBytes;
    const float* lse = sL + buf * BLK;
    const float* dsm = sD + buf * BLK;
    // S^T = K Q^T (keys x queries), P^T = 2^(S^T * scale - lse[query]), masked where key > query on the diagonal block
    float st[8][4];
    zero_acc(st);
    gemm_nk(st, ka, tQ);
#pragma unroll
    for (int nt = 0; nt < 8; nt++)
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int qi = nt * 8 + 2 * t + (e & 1), ki = key0 + (e >> 1) * 8;
        float p = ex2(st[nt][e] * a.scale_log2 - lse[qi]);
        if (i == kb && ki > qi) p = 0.f;
        st[nt][e] = p;
      }
    uint32_t pa[4][4];
    acc_to_a(st, pa);
    gemm_kn(dv, pa, tDO);                  // dV += P^T dO
    float dp[8][4];
    zero_acc(dp);
    gemm_nk(dp, va, tDO);                  // dP^T = V dO^T
#pragma unroll
    for (int nt = 0; nt < 8; nt++)
#pragma unroll
      for (int e = 0; e < 4; e++) dp[nt][e] = st[nt][e] * (dp[nt][e] - dsm[nt * 8 + 2 * t + (e & 1)]);
    acc_to_a(dp, pa);
    gemm_kn(dk, pa, tQ);                   // dK += dS^T Q
    __syncthreads();
  }
  const float sc = a.scale_log2 * 0.6931471805599453f;     // 1 / sqrt(64): dS carries one factor of the softmax scale
  __nv_bfloat16* DK = a.dqkv + ((size_t)b * a.T + (size_t)kb * BLK) * ld + (size_t)a.H * HD + (size_t)h * HD;
  __nv_bfloat16* DV = DK + (size_t)a.H * HD;
  store_acc_bf16(DK, ld, warp * 16, dk, sc);
  store_acc_bf16(DV, ld, warp * 16, dv, 1.f);
}

// ---------------------------------------------------------------------------------------------------- backward: dQ
__global__ void __launch_bounds__(kThreads) attn_train_bwd_q_kernel(const AttnTrainArgs a) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sQ = smem_addr(smem), sDO = sQ + kTileBytes, sK = sDO + kTileBytes, sV = sK + 2 * kTileBytes;
  const int qb = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const size_t ld = (size_t)3 * a.H * HD, ldo = (size_t)a.H * HD;
  const __nv_bfloat16* base = a.qkv + (size_t)b * a.T * ld + (size_t)h * HD;
  const __nv_bfloat16 *Q = base + (size_t)qb * BLK * ld, *K = base + (size_t)a.H * HD, *V = base + (size_t)2 * a.H * HD;
  const __nv_bfloat16* DO = a.d_o + ((size_t)b * a.T + (size_t)qb * BLK) * ldo + (size_t)h * HD;
  const int r0 = warp * 16 + g;
  const float* L = a.lse + ((size_t)b * a.H + h) * a.T + qb * BLK;
  const float* D = a.dsum + ((size_t)b * a.H + h) * a.T + qb * BLK;
  const float lse0 = L[r0], lse1 = L[r0 + 8], d0 = D[r0], d1 = D[r0 + 8];

  load_tile(sQ, Q, ld);
  load_tile(sDO, DO, ldo);
  load_tile(sK, K, ld);
  load_tile(sV, V, ld);
  cp_commit();
  uint32_t qa[4][4], doa[4][4];
  float dq[8][4];
  zero_acc(dq);
  for (int j = 0; j <= qb; j++) {
    const int buf = j & 1;
    if (j < qb) {
      load_tile(sK + (buf ^ 1) * kTileBytes, K + (size_t)(j + 1) * BLK * ld, ld);
      load_tile(sV + (buf ^ 1) * kTileBytes, V + (size_t)(j + 1) * BLK * ld, ld);
      cp_commit();
      cp_wait<1>();
    } else {
      cp_wait<0>();
    }
    __syncthreads();
    if (j == 0) {
      load_a_frags(sQ, warp * 16, qa);
      load_a_frags(sDO, warp * 16, doa);
    }
    float s[8][4];
    zero_acc(s);
    gemm_nk(s, qa, sK + buf * kTileBytes);
#pragma unroll
    for (int nt = 0; nt < 8; nt++)
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int ki = nt * 8 + 2 * t + (e & 1), qi = r0 + (e >> 1) * 8;
        float p = ex2(s[nt][e] * a.scale_log2 - ((e >> 1) ? lse1 : lse0));
        if (j == qb && ki > qi) p = 0.f;
        s[nt][e] = p;
      }
    float dp[8][4];
    zero_acc(dp);
    gemm_nk(dp, doa, sV + buf * kTileBytes);          // dP = dO V^T
#pragma unroll
    for (int nt = 0; nt < 8; nt++)
#pragma unroll
      for (int e = 0; e < 4; e++) dp[nt][e] = s[nt][e] * (dp[nt][e] - ((e >> 1) ? d1 : d0));
    uint32_t pa[4][4];
    acc_to_a(dp, pa);
    gemm_kn(dq, pa, sK + buf * kTileBytes);           // dQ += dS K
    __syncthreads();
  }
  const float sc = a.scale_log2 * 0.6931471805599453f;
  __nv_bfloat16* DQ = a.dqkv + ((size_t)b * a.T + (size_t)qb * BLK) * ld + (size_t)h * HD;
  store_acc_bf16(DQ, ld, warp * 16, dq, sc);
}

int check(const void* p) { return ((uintptr_t)p & 15) ? 1 : 0; }

}  // namespace

// Forward.  qkv [B*T][3][H][64] bf16 -> o [B*T][H][64] bf16, lse [B][H][T] fp32 (base-2 log-sum-exp of the scaled scores).
// T must be a multiple of 64.
B200_API int b200_attn_train_fwd(const void* qkv, void* o, float* lse, int B, int T, int H, int hd, cudaStream_t st) {
  if (hd != HD || T % BLK || B < 1 || H < 1 || check(qkv) || check(o) || check(lse)) return B200_ERR_BAD_ARG;
  AttnTrainArgs a = {};
  a.qkv = (const __nv_bfloat16*)qkv; a.o = (__nv_bfloat16*)o; a.lse = lse; a.B = B; a.T = T; a.H = H;
  a.scale_log2 = 1.4426950408889634f / 8.f;
  constexpr int smem = 5 * kTileBytes;
  static bool cfg = false;
  if (!cfg) {
    cudaError_t e = cudaFuncSetAttribute(attn_train_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    cfg = true;
  }
  attn_train_fwd_kernel<<<dim3(T / BLK, H, B), kThreads, smem, st>>>(a);
  return (int)cudaGetLastError();
}

// Backward.  Reads qkv, o, d_o [B*T][H][64] and the forward's lse; writes dqkv (layout of qkv); dsum [B][H][T] fp32 is
// working space the caller provides.
B200_API int b200_attn_train_bwd(const void* qkv, const void* o, const void* d_o, const float* lse, float* dsum, void* dqkv,
                                 int B, int T, int H, int hd, cudaStream_t st) {
  if (hd != HD || T % BLK || B < 1 || H < 1 || check(qkv) || check(o) || check(d_o) || check(lse) || check(dsum) || check(dqkv))
    return B200_ERR_BAD_ARG;
  AttnTrainArgs a = {};
  a.qkv = (const __nv_bfloat16*)qkv; a.o = (__nv_bfloat16*)o; a.d_o = (const __nv_bfloat16*)d_o; a.dqkv = (__nv_bfloat16*)dqkv;
  a.lse = (float*)lse; a.dsum = dsum; a.B = B; a.T = T; a.H = H;
  a.scale_log2 = 1.4426950408889634f / 8.f;
  constexpr int smem_kv = 6 * kTileBytes + 4 * BLK * 4, smem_q = 6 * kTileBytes;
  static bool cfg = false;
  if (!cfg) {
    cudaError_t e = cudaFuncSetAttribute(attn_train_bwd_kv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_kv);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_train_bwd_q_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_q);
    if (e != cudaSuccess) return (int)e;
    cfg = true;
  }
  const int rows = B * T * H;
  attn_train_dsum_kernel<<<(rows + 7) / 8, 256, 0, st>>>(a);
  attn_train_bwd_kv_kernel<<<dim3(T / BLK, H, B), kThreads, smem_kv, st>>>(a);
  attn_train_bwd_q_kernel<<<dim3(T / BLK, H, B), kThreads, smem_q, st>>>(a);
  return (int)cudaGetLastError();
}
