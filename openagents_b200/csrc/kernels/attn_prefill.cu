// Causal grouped-query flash attention over a paged fp16 K/V cache for many query tokens per
// sequence (prefill chunks and the training forward pass).  Sliding windows and learned sink
// logits are supported.  The K/V of the chunk itself must already be in the cache (the RoPE kernel
// writes them), so one code path serves cold prefill, chunked prefill and prefix reuse.
//
// One CTA = 64 query rows of one head; four warps own 16 rows each.  K/V tiles of 64 keys (four
// 16-token pages) stream through a double-buffered, XOR-swizzled shared-memory ring with cp.async;
// QK^T and PV run on mma.sync m16n8k16 with fp32 accumulation and an online softmax
// (max-subtract / exp / normalise as in cs336-a1-real-gradient-workload.ts:478-518).
#include "common.cuh"

using namespace b200;

struct AttnPreArgs {
  const __half* q;        // [T_total][Hq][HD], rotated, pre-scaled by 1/sqrt(HD)
  const __half* kc;       // [pages][Hkv][16][HD]
  const __half* vc;
  const int* page_table;  // [n_seqs][max_pages]; null = pages of sequence s start at s * max_pages
  const int* q_start;     // [n_seqs] first row of the sequence in q / out
  const int* q_len;       // [n_seqs]
  const int* ctx_len;     // [n_seqs] keys in the cache after this chunk
  const float* sinks;     // [Hq] or null
  int max_pages, Hq, Hkv, window;
  __nv_bfloat16* out_bf16;  // [T_total][Hq*HD] or null
  float* out_f32;           // or null
  float* lse;               // [T_total][Hq] natural-log sum-exp (training backward), or null
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N));
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *(uint32_t*)&h;
}

template <int HD>
__global__ void __launch_bounds__(128) attn_prefill_kernel(const AttnPreArgs a) {
  constexpr int ROW_B = HD * 2;          // bytes per row
  constexpr int CH = HD / 8;             // 16-byte chunks per row
  constexpr int TILE_B = 64 * ROW_B;     // bytes per 64-row tile
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* sQ = smem;                    // [64][HD]
  uint8_t* sK = smem + TILE_B;           // 2 x [64][HD]
  uint8_t* sV = smem + 3 * TILE_B;       // 2 x [64][HD]

  const int seq = blockIdx.z, h = blockIdx.y, qb = blockIdx.x;
  const int qlen = a.q_len[seq];
  const int q0 = qb * 64;
  if (q0 >= qlen) return;
  const int ctx = a.ctx_len[seq], qs = a.q_start[seq];
  const int kh = h / (a.Hq / a.Hkv);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
  const int pos_base = ctx - qlen;       // absolute position of query row 0
  const int* pt = a.page_table ? a.page_table + (size_t)seq * a.max_pages : nullptr;
  const int page_base = seq * a.max_pages;

  // ---- Q tile -> shared (swizzled), rows past q_len zero-filled
  for (int i = tid; i < 64 * CH; i += 128) {
    const int r = i / CH, c = i % CH;
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(sQ + r * ROW_B + ((c ^ (r & 7)) << 4));
    if (q0 + r < qlen)
      cp_async16(dst, a.q + ((size_t)(qs + q0 + r) * a.Hq + h) * HD + c * 8);
    else
      *(uint4*)(sQ + r * ROW_B + ((c ^ (r & 7)) << 4)) = make_uint4(0, 0, 0, 0);
  }
  cp_async_commit();

  // key range this query block can see
  const int qpos_lo = pos_base + q0, qpos_hi = pos_base + min(q0 + 63, qlen - 1);
  const int k_first = a.window > 0 ? max(0, qpos_lo - a.window + 1) : 0;
  const int k_last = min(ctx - 1, qpos_hi);
  const int t_begin = k_first / 64, t_end = k_last / 64 + 1;

  auto load_tile = [&](int tile, int buf) {
    for (int i = tid; i < 64 * CH; i += 128) {
      const int r = i / CH, c = i % CH;
      const int key = tile * 64 + r;
      const int sw = (c ^ (r & 7)) << 4;
      uint8_t* dk = sK + buf * TILE_B + r * ROW_B + sw;
      uint8_t* dv = sV + buf * TILE_B + r * ROW_B + sw;
      if (key < ctx) {
        const int p = key >> 4;
        const int pid = pt ? pt[p] : page_base + p;
        const size_t off = (((size_t)pid * a.Hkv + kh) * 16 + (key & 15)) * HD + c * 8;
        cp_async16((uint32_t)__cvta_generic_to_shared(dk), a.kc + off);
        cp_async16((uint32_t)__cvta_generic_to_shared(dv), a.vc + off);
      } else {
        *(uint4*)dk = make_uint4(0, 0, 0, 0);
        *(uint4*)dv = make_uint4(0, 0, 0, 0);
      }
    }
  };

  load_tile(t_begin, 0);
  cp_async_commit();

  float o[HD / 8][4];
#pragma unroll
  for (int j = 0; j < HD / 8; j++) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const float LOG2E = 1.4426950408889634f;

  uint32_t qf[HD / 16][4];
  bool q_loaded = false;
  const int row0 = q0 + warp * 16 + g, row1 = row0 + 8;      // query rows of this thread (chunk-local)
  const int qp0 = pos_base + row0, qp1 = pos_base + row1;

  for (int tile = t_begin; tile < t_end; tile++) {
    const int buf = (tile - t_begin) & 1;
    if (tile + 1 < t_end) load_tile(tile + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    if (!q_loaded) {
      q_loaded = true;
#pragma unroll
      for (int kk = 0; kk < HD / 16; kk++) {
        const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = 2 * kk + (lane >> 4);
        ldsm_x4((uint32_t)__cvta_generic_to_shared(sQ + r * ROW_B + ((c ^ (r & 7)) << 4)), qf[kk][0], qf[kk][1],
                qf[kk][2], qf[kk][3]);
      }
    }
    // ---- S = Q K^T  (16 x 64 per warp)
    float s[8][4];
#pragma unroll
    for (int j = 0; j < 8; j++) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    const uint8_t* kb = sK + buf * TILE_B;
#pragma unroll
    for (int kk = 0; kk < HD / 16; kk++) {
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        const int r = (j + (lane >> 4)) * 8 + (lane & 7);
        const int c = 2 * kk + ((lane >> 3) & 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4((uint32_t)__cvta_generic_to_shared(kb + r * ROW_B + ((c ^ (r & 7)) << 4)), b0, b1, b2, b3);
        mma16816(s[j], qf[kk], b0, b1);
        mma16816(s[j + 1], qf[kk], b2, b3);
      }
    }
    // ---- mask + online softmax
    const int kbase = tile * 64;
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; j++) {
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int kpos = kbase + j * 8 + t4 * 2 + (e & 1);
        const int qp = (e < 2) ? qp0 : qp1;
        bool ok = kpos <= qp && kpos < ctx;
        if (a.window > 0) ok = ok && (qp - kpos < a.window);
        s[j][e] = ok ? s[j][e] * LOG2E : -INFINITY;
      }
      mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
      mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float c0 = (m0 == -INFINITY) ? 0.f : exp2f(m0 - mn0);
    const float c1 = (m1 == -INFINITY) ? 0.f : exp2f(m1 - mn1);
    const float sub0 = (mn0 == -INFINITY) ? 0.f : mn0, sub1 = (mn1 == -INFINITY) ? 0.f : mn1;
    float rs0 = 0.f, rs1 = 0.f;
    uint32_t pf[4][4];
#pragma unroll
    for (int j = 0; j < 8; j++) {
      const float p0 = exp2f(s[j][0] - sub0), p1 = exp2f(s[j][1] - sub0);
      const float p2 = exp2f(s[j][2] - sub1), p3 = exp2f(s[j][3] - sub1);
      rs0 += p0 + p1;
      rs1 += p2 + p3;
      pf[j >> 1][(j & 1) * 2] = pack_h2(p0, p1);
      pf[j >> 1][(j & 1) * 2 + 1] = pack_h2(p2, p3);
    }
    l0 = l0 * c0 + rs0;
    l1 = l1 * c1 + rs1;
    m0 = mn0;
    m1 = mn1;
#pragma unroll
    for (int j = 0; j < HD / 8; j++) {
      o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1;
    }
    // ---- O += P V
    const uint8_t* vb = sV + buf * TILE_B;
#pragma unroll
    for (int kk = 0; kk < 4; kk++) {
#pragma unroll
      for (int jd = 0; jd < HD / 8; jd += 2) {
        const int r = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = jd + (lane >> 4);
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t((uint32_t)__cvta_generic_to_shared(vb + r * ROW_B + ((c ^ (r & 7)) << 4)), b0, b1, b2, b3);
        mma16816(o[jd], pf[kk], b0, b1);
        mma16816(o[jd + 1], pf[kk], b2, b3);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  // ---- finish: row sums across the quad, sinks, normalise, store
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  float sc0 = 1.f, sc1 = 1.f;
  if (a.sinks) {
    const float sk = a.sinks[h] * LOG2E;
    const float M0 = fmaxf(m0, sk), M1 = fmaxf(m1, sk);
    sc0 = (m0 == -INFINITY) ? 0.f : exp2f(m0 - M0);
    sc1 = (m1 == -INFINITY) ? 0.f : exp2f(m1 - M1);
    l0 = l0 * sc0 + exp2f(sk - M0);
    l1 = l1 * sc1 + exp2f(sk - M1);
    m0 = M0;
    m1 = M1;
  }
  const float inv0 = l0 > 0.f ? sc0 / l0 : 0.f, inv1 = l1 > 0.f ? sc1 / l1 : 0.f;
#pragma unroll
  for (int j = 0; j < HD / 8; j++) {
    const int col = h * HD + j * 8 + t4 * 2;
    if (row0 < qlen) {
      const size_t idx = (size_t)(qs + row0) * a.Hq * HD + col;
      if (a.out_bf16) *(__nv_bfloat162*)(a.out_bf16 + idx) = __floats2bfloat162_rn(o[j][0] * inv0, o[j][1] * inv0);
      if (a.out_f32) *(float2*)(a.out_f32 + idx) = make_float2(o[j][0] * inv0, o[j][1] * inv0);
    }
    if (row1 < qlen) {
      const size_t idx = (size_t)(qs + row1) * a.Hq * HD + col;
      if (a.out_bf16) *(__nv_bfloat162*)(a.out_bf16 + idx) = __floats2bfloat162_rn(o[j][2] * inv1, o[j][3] * inv1);
      if (a.out_f32) *(float2*)(a.out_f32 + idx) = make_float2(o[j][2] * inv1, o[j][3] * inv1);
    }
  }
  if (a.lse && t4 == 0) {
    const float LN2 = 0.6931471805599453f;
    if (row0 < qlen) a.lse[(size_t)(qs + row0) * a.Hq + h] = (m0 + log2f(l0)) * LN2;
    if (row1 < qlen) a.lse[(size_t)(qs + row1) * a.Hq + h] = (m1 + log2f(l1)) * LN2;
  }
}

B200_API int b200_attn_prefill(const void* q, const void* kc, const void* vc, const int* page_table, int max_pages,
                               const int* q_start, const int* q_len, const int* ctx_len, const float* sinks,
                               int n_seqs, int max_q_len, int Hq, int Hkv, int hd, int window, void* out_bf16,
                               float* out_f32, float* lse, cudaStream_t st) {
  if (Hq % Hkv) return B200_ERR_BAD_ARG;
  AttnPreArgs a;
  a.q = (const __half*)q; a.kc = (const __half*)kc; a.vc = (const __half*)vc; a.page_table = page_table;
  a.q_start = q_start; a.q_len = q_len; a.ctx_len = ctx_len; a.sinks = sinks; a.max_pages = max_pages;
  a.Hq = Hq; a.Hkv = Hkv; a.window = window; a.out_bf16 = (__nv_bfloat16*)out_bf16; a.out_f32 = out_f32;
  a.lse = lse;
  dim3 grid((max_q_len + 63) / 64, Hq, n_seqs);
  if (hd == 128) {
    const int smem = 5 * 64 * 256;
    static bool cfg = false;
    if (!cfg) {
      cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return (int)e;
      cfg = true;
    }
    attn_prefill_kernel<128><<<grid, 128, smem, st>>>(a);
  } else if (hd == 64) {
    const int smem = 5 * 64 * 128;
    static bool cfg = false;
    if (!cfg) {
      cudaError_t e = cudaFuncSetAttribute(attn_prefill_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return (int)e;
      cfg = true;
    }
    attn_prefill_kernel<64><<<grid, 128, smem, st>>>(a);
  } else {
    return B200_ERR_BAD_ARG;
  }
  return (int)cudaGetLastError();
}
