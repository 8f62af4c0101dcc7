// Paged-KV grouped-query attention for decode: one query token per sequence against a paged
// fp16 K/V cache with 16-token pages, optional sliding window and learned sink logits.
//
// Work split: grid = (splits, kv_heads, sequences).  A CTA streams its share of one sequence's
// pages for one KV head exactly once and serves all G query heads that share that KV head, so the
// cache is read once per KV head, not once per query head.  Pages arrive through swizzled 2-D TMA
// loads into a ring of shared-memory slots; each warp consumes whole pages on mma.sync tiles with
// the query heads of the group as the (padded) M dimension.  Splits are merged by whichever CTA
// finishes last (a counter, no waiting).
//
// The softmax follows the reference formulation (max-subtract, exp, normalise:
// apps/openagents.com/workers/api/src/cs336-a1-real-gradient-workload.ts:478-518).
#include "tc05.cuh"

using namespace b200;

struct AttnDecArgs {
  const float* q;          // [B][Hq*HD], rotated and pre-scaled by 1/sqrt(HD)
  const __half* kc;        // [pages][Hkv][16][HD]
  const __half* vc;
  const int* page_table;   // [B][max_pages]
  const int* seq_lens;     // [B] keys to attend (includes the current token)
  const float* sinks;      // [Hq] or null
  int max_pages, Hq, Hkv, window, S;
  int kv_rep, Hkv_cache;   // virtual KV heads per cache head (splits wide groups), heads in the cache
  float* out_f32;          // [B][Hq*HD] or null
  __nv_bfloat16* out_bf16; // [B][Hq*HD] or null
  int8_t* oq;              // quantized output for a following mat-vec, or null
  float* od;
  float* os16;
  float* part_acc;         // [B*Hkv*S*G][HD]
  float* part_ml;          // [B*Hkv*S*G][2]
  int* counters;           // [B*Hkv], zero before first use; left zero on exit
  int* status;             // set non-zero if a copy never arrived (may be null)
};

__device__ __forceinline__ float exp_scale(float m, float M) {
  return m == -INFINITY ? 0.f : __expf(m - M);
}

template <int HD, int G>
__device__ __forceinline__ void write_out(const AttnDecArgs& a, int b, int kh, int g, int e, float o) {
  const int col = (kh * G + g) * HD + e;
  const size_t row = (size_t)b * a.Hq * HD;
  if (a.out_f32) a.out_f32[row + col] = o;
  if (a.out_bf16) a.out_bf16[row + col] = __float2bfloat16(o);
  if (a.oq) {
    const int lane = threadIdx.x & 31;
    const int blk = col >> 5;
    const size_t nblk = (size_t)a.Hq * HD / 32;
    quantize_block32(o, lane, a.oq + row + (size_t)blk * 32, a.od + (size_t)b * nblk + blk,
                     a.os16 + ((size_t)b * nblk + blk) * 2);
  }
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
__device__ __forceinline__ uint32_t pack_h2(float x, float y) {
  __half2 h = __floats2half2_rn(x, y);
  return *(uint32_t*)&h;
}

constexpr int kStages = 8;   // pages in flight per CTA (two per warp)

// One CTA = (split, kv head, sequence).  Warp w owns pages w, w+4, w+8, ... of the CTA's range and
// the ring slots w and w+4: it waits for its own page, runs QK^T and PV on tensor-core tiles with
// the G query heads padded to a 16-row tile, and re-issues the TMA load for its next page itself,
// so no CTA-wide synchronisation happens inside the loop.  K/V tiles land in shared memory with the
// 128-byte swizzle, which makes every ldmatrix conflict-free.
template <int HD, int G>
__global__ void __launch_bounds__(128) attn_decode_kernel(const __grid_constant__ CUtensorMap tmK,
                                                           const __grid_constant__ CUtensorMap tmV,
                                                           const AttnDecArgs a) {
  constexpr int NBOX = HD / 64;        // 64-column (128-byte) boxes per tile
  constexpr int BOX = 16 * 128;        // bytes of one box: 16 tokens x 128 bytes
  constexpr int TILE = NBOX * BOX;     // bytes of one (page, head) K or V tile
  extern __shared__ uint8_t dyn_raw[];
  uint8_t* ring = (uint8_t*)(((uintptr_t)dyn_raw + 1023) & ~(uintptr_t)1023);   // kStages x (K, V)
  uint64_t* bars = (uint64_t*)(ring + kStages * 2 * TILE);
  int* s_pid = (int*)(bars + kStages);
  __shared__ float s_acc[4][G][HD];
  __shared__ float s_ml[4][G][2];
  __shared__ int s_last;
  __shared__ int s_abort;

  const int split = blockIdx.x, kh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g4 = lane >> 2, t4 = lane & 3;
  if (tid == 0) {
    for (int s = 0; s < kStages; s++) tc::mbar_init(tc::smem_u32(bars + s), 1);
    s_abort = 0;
    tc::fence_barrier_init();
    tc::tma_prefetch_desc(&tmK);
    tc::tma_prefetch_desc(&tmV);
  }
  // Everything above touches only this CTA's shared memory; lengths, page table, queries and the
  // cache come from earlier kernels.
  pdl_trigger();
  pdl_wait();
  const int len = a.seq_lens[b];
  const int first = (a.window > 0 && len > a.window) ? len - a.window : 0;
  const int p_first = first >> 4, p_last = (len + 15) >> 4;
  const int per = (p_last - p_first + a.S - 1) / a.S;
  const int pa = p_first + split * per;
  const int pb = min(p_last, pa + per);
  const int np = max(0, pb - pa);
  const int kh_cache = kh / a.kv_rep;

  const int* pt = a.page_table + (size_t)b * a.max_pages;
  for (int i = tid; i < np; i += 128) s_pid[i] = pt[pa + i];
  __syncthreads();

  auto issue = [&](int i) {   // one lane: fetch page i of the range into ring slot i % kStages
    const int s = i % kStages;
    const uint32_t bar = tc::smem_u32(bars + s);
    const int row = (s_pid[i] * a.Hkv_cache + kh_cache) * 16;
    tc::mbar_expect_tx(bar, 2 * TILE);
#pragma unroll
    for (int c = 0; c < NBOX; c++) {
      tc::tma_load_2d(tc::smem_u32(ring + (size_t)s * 2 * TILE + c * BOX), &tmK, bar, c * 64, row);
      tc::tma_load_2d(tc::smem_u32(ring + (size_t)s * 2 * TILE + TILE + c * BOX), &tmV, bar, c * 64, row);
    }
  };
  if (lane == 0) {
    if (warp < np) issue(warp);
    if (warp + 4 < np) issue(warp + 4);
  }

  // Q as the A operand: rows = query heads (zero beyond G), fp16, HD/16 k-steps.
  uint32_t qf[HD / 16][4];
  {
    const float* q0 = a.q + (size_t)b * a.Hq * HD + (size_t)(kh * G) * HD;
#pragma unroll
    for (int kk = 0; kk < HD / 16; kk++) {
      const int c0 = kk * 16 + t4 * 2;
      float2 v00 = make_float2(0.f, 0.f), v01 = v00, v10 = v00, v11 = v00;
      if (g4 < G) {
        v00 = *(const float2*)(q0 + g4 * HD + c0);
        v01 = *(const float2*)(q0 + g4 * HD + c0 + 8);
      }
      if (g4 + 8 < G) {
        v10 = *(const float2*)(q0 + (g4 + 8) * HD + c0);
        v11 = *(const float2*)(q0 + (g4 + 8) * HD + c0 + 8);
      }
      qf[kk][0] = pack_h2(v00.x, v00.y);
      qf[kk][1] = pack_h2(v10.x, v10.y);
      qf[kk][2] = pack_h2(v01.x, v01.y);
      qf[kk][3] = pack_h2(v11.x, v11.y);
    }
  }
  float o[HD / 8][4];
#pragma unroll
  for (int j = 0; j < HD / 8; j++) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // rows g4 and g4 + 8

  for (int i = warp; i < np; i += 4) {
    const int s = i % kStages;
    bool ok = tc::mbar_wait(tc::smem_u32(bars + s), (uint32_t)((i / kStages) & 1), &s_abort);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    const uint8_t* kt = ring + (size_t)s * 2 * TILE;
    const uint8_t* vt = kt + TILE;
    // ---- S = Q K^T : 16 heads x 16 tokens
    float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int kk = 0; kk < HD / 16; kk++) {
      const int r = (lane >> 4) * 8 + (lane & 7);            // token row
      const int c = 2 * kk + ((lane >> 3) & 1);              // 16-byte chunk of the full row
      const uint8_t* p = kt + (c >> 3) * BOX + r * 128 + (((c & 7) ^ (r & 7)) << 4);
      uint32_t b0, b1, b2, b3;
      ldsm_x4(tc::smem_u32(p), b0, b1, b2, b3);
      mma16816(sc[0], qf[kk], b0, b1);
      mma16816(sc[1], qf[kk], b2, b3);
    }
    // ---- mask, online softmax (rows g4, g4+8; this thread holds tokens 2*t4, 2*t4+1 of each 8)
    const int tbase = (pa + i) * 16;
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const int t = tbase + j * 8 + t4 * 2 + (e & 1);
        if (!(t >= first && t < len)) sc[j][e] = -INFINITY;
        if (e < 2) mx0 = fmaxf(mx0, sc[j][e]); else mx1 = fmaxf(mx1, sc[j][e]);
      }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float c0 = exp_scale(m0, mn0), c1 = exp_scale(m1, mn1);
    const float sub0 = mn0 == -INFINITY ? 0.f : mn0, sub1 = mn1 == -INFINITY ? 0.f : mn1;
    uint32_t pf[4];
    float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
    for (int j = 0; j < 2; j++) {
      const float p0 = __expf(sc[j][0] - sub0), p1 = __expf(sc[j][1] - sub0);
      const float p2 = __expf(sc[j][2] - sub1), p3 = __expf(sc[j][3] - sub1);
      rs0 += p0 + p1;
      rs1 += p2 + p3;
      pf[j * 2] = pack_h2(p0, p1);
      pf[j * 2 + 1] = pack_h2(p2, p3);
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
#pragma unroll
    for (int jd = 0; jd < HD / 8; jd += 2) {
      const int r = (lane & 7) + ((lane >> 3) & 1) * 8;      // token row
      const int c = jd + (lane >> 4);
      const uint8_t* p = vt + (c >> 3) * BOX + r * 128 + (((c & 7) ^ (r & 7)) << 4);
      uint32_t b0, b1, b2, b3;
      ldsm_x4_t(tc::smem_u32(p), b0, b1, b2, b3);
      mma16816(o[jd], pf, b0, b1);
      mma16816(o[jd + 1], pf, b2, b3);
    }
    __syncwarp();
    if (lane == 0 && i + kStages < np) issue(i + kStages);
  }
  if (tid == 0 && s_abort && a.status) atomicExch(a.status, (int)B200_ERR_TIMEOUT_TMA);

  // row sums live in the four lanes of a quad
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  // this warp's partial (m, l, O) for each real head -> shared
  if (g4 < G) {
#pragma unroll
    for (int j = 0; j < HD / 8; j++) {
      s_acc[warp][g4][j * 8 + t4 * 2] = o[j][0];
      s_acc[warp][g4][j * 8 + t4 * 2 + 1] = o[j][1];
    }
    if (t4 == 0) {
      s_ml[warp][g4][0] = m0;
      s_ml[warp][g4][1] = l0;
    }
  }
  if (g4 + 8 < G) {
#pragma unroll
    for (int j = 0; j < HD / 8; j++) {
      s_acc[warp][g4 + 8][j * 8 + t4 * 2] = o[j][2];
      s_acc[warp][g4 + 8][j * 8 + t4 * 2 + 1] = o[j][3];
    }
    if (t4 == 0) {
      s_ml[warp][g4 + 8][0] = m1;
      s_ml[warp][g4 + 8][1] = l1;
    }
  }
  __syncthreads();

  // merge the four warps: thread e owns output dim e
  const int e = tid;
  const size_t pbase = (((size_t)b * a.Hkv + kh) * a.S + split) * G;
  float fm[G], fl[G], fa[G];
#pragma unroll
  for (int g = 0; g < G; g++) {
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; w++) M = fmaxf(M, s_ml[w][g][0]);
    float L = 0.f, A = 0.f;
#pragma unroll
    for (int w = 0; w < 4; w++) {
      const float c = exp_scale(s_ml[w][g][0], M);
      L += s_ml[w][g][1] * c;
      if (e < HD) A += s_acc[w][g][e] * c;
    }
    fm[g] = M; fl[g] = L; fa[g] = A;
  }

  if (a.S > 1) {
#pragma unroll
    for (int g = 0; g < G; g++) {
      if (e < HD) a.part_acc[(pbase + g) * HD + e] = fa[g];
      if (e == 0) {
        a.part_ml[(pbase + g) * 2] = fm[g];
        a.part_ml[(pbase + g) * 2 + 1] = fl[g];
      }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const int done = atomicAdd(a.counters + b * a.Hkv + kh, 1);
      s_last = (done == a.S - 1);
      if (s_last) a.counters[b * a.Hkv + kh] = 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const size_t p0 = ((size_t)b * a.Hkv + kh) * a.S * G;
#pragma unroll
    for (int g = 0; g < G; g++) {
      float M = -INFINITY;
      for (int s = 0; s < a.S; s++) M = fmaxf(M, __ldcg(a.part_ml + (p0 + (size_t)s * G + g) * 2));
      float L = 0.f, A = 0.f;
      for (int s = 0; s < a.S; s++) {
        const size_t idx = p0 + (size_t)s * G + g;
        const float c = exp_scale(__ldcg(a.part_ml + idx * 2), M);
        L += __ldcg(a.part_ml + idx * 2 + 1) * c;
        if (e < HD) A += __ldcg(a.part_acc + idx * HD + e) * c;
      }
      fm[g] = M; fl[g] = L; fa[g] = A;
    }
  }

  if (warp * 32 < HD) {  // warps that own real output dims (all four when HD = 128)
#pragma unroll
    for (int g = 0; g < G; g++) {
      float M = fm[g], L = fl[g], A = fa[g];
      if (a.sinks) {
        const float sk = a.sinks[kh * G + g];
        const float M2 = fmaxf(M, sk);
        const float c = exp_scale(M, M2);
        L = L * c + __expf(sk - M2);
        A *= c;
      }
      const float o = L > 0.f ? A / L : 0.f;
      write_out<HD, G>(a, b, kh, g, e, o);
    }
  }
}

template <int HD, int G>
static int launch(const AttnDecArgs& a, int B, int n_pages, cudaStream_t st) {
  dim3 grid(a.S, a.Hkv, B);
  const int pages_per_cta = (a.max_pages + a.S - 1) / a.S + 1;
  const size_t smem = 1024 + (size_t)kStages * 2 * 16 * HD * 2 + kStages * 8 + (size_t)pages_per_cta * 4;
  if (smem > 200 * 1024) return B200_ERR_BAD_ARG;
  static size_t configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<HD, G>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  // The cache as a 2-D tensor: one row per (page, head, token), HD columns.
  CUtensorMap tk, tv;
  const uint64_t rows = (uint64_t)n_pages * a.Hkv_cache * 16;
  int rc = make_tmap_2d(&tk, a.kc, 2, rows, HD, (uint64_t)HD * 2, 16, 64, true);
  if (rc) return rc;
  rc = make_tmap_2d(&tv, a.vc, 2, rows, HD, (uint64_t)HD * 2, 16, 64, true);
  if (rc) return rc;
  return launch_pdl(attn_decode_kernel<HD, G>, grid, dim3(128), smem, st, tk, tv, a);
}

// Floats of scratch the split-merge needs: part_acc then part_ml, plus B*Hkv ints of counters.
B200_API size_t b200_attn_decode_scratch_floats(int B, int Hq, int Hkv, int hd, int S) {
  return (size_t)B * Hq * S * (hd + 2);
}

B200_API int b200_attn_decode(const float* q, const void* kc, const void* vc, const int* page_table,
                              int max_pages, int n_pages, const int* seq_lens, const float* sinks, int B,
                              int Hq, int Hkv, int hd, int window, int S, float* out_f32, void* out_bf16,
                              void* oq, float* od, float* os16, float* scratch, int* counters, int* status,
                              cudaStream_t st) {
  if (Hq % Hkv || S < 1) return B200_ERR_BAD_ARG;
  const int G = Hq / Hkv;
  if (G > 16) return B200_ERR_BAD_ARG;
  AttnDecArgs a;
  a.q = q; a.kc = (const __half*)kc; a.vc = (const __half*)vc; a.page_table = page_table;
  a.seq_lens = seq_lens; a.sinks = sinks; a.max_pages = max_pages; a.Hq = Hq; a.Hkv = Hkv;
  a.window = window; a.S = S; a.kv_rep = 1; a.Hkv_cache = Hkv; a.out_f32 = out_f32; a.out_bf16 = (__nv_bfloat16*)out_bf16;
  a.oq = (int8_t*)oq; a.od = od; a.os16 = os16;
  a.part_acc = scratch;
  a.part_ml = scratch ? scratch + (size_t)B * Hq * S * hd : nullptr;
  a.counters = counters;
  a.status = status;
  if (S > 1 && (!scratch || !counters)) return B200_ERR_BAD_ARG;
  if (hd == 128) {
    if (G == 1) return launch<128, 1>(a, B, n_pages, st);
    if (G == 2) return launch<128, 2>(a, B, n_pages, st);
    if (G == 4) return launch<128, 4>(a, B, n_pages, st);
    if (G == 8) return launch<128, 8>(a, B, n_pages, st);
    if (G == 16) return launch<128, 16>(a, B, n_pages, st);
  } else if (hd == 64) {
    if (G == 1) return launch<64, 1>(a, B, n_pages, st);
    if (G == 2) return launch<64, 2>(a, B, n_pages, st);
    if (G == 4) return launch<64, 4>(a, B, n_pages, st);
    if (G == 8) return launch<64, 8>(a, B, n_pages, st);
    if (G == 16) return launch<64, 16>(a, B, n_pages, st);
  }
  return B200_ERR_BAD_ARG;
}
