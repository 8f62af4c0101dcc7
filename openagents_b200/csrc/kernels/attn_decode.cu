// Paged-KV grouped-query attention for decode: one query token per sequence against a paged
// fp16 K/V cache with 16-token pages, optional sliding window and learned sink logits.
//
// Work split: grid = (splits, kv_heads, sequences).  A CTA streams its share of one sequence's
// pages for one KV head exactly once and serves all G query heads that share that KV head, so the
// cache is read once per KV head, not once per query head.  Inside a CTA the four warps each take
// four tokens of a 16-token page; eight lanes share a token (HD/8 dims each), so a dot product
// needs three shuffles.  Splits are merged by whichever CTA finishes last (a counter, no waiting).
//
// The softmax follows the reference formulation (max-subtract, exp, normalise:
// apps/openagents.com/workers/api/src/cs336-a1-real-gradient-workload.ts:478-518).
#include "common.cuh"

using namespace b200;

struct AttnDecArgs {
  const float* q;          // [B][Hq*HD], rotated and pre-scaled by 1/sqrt(HD)
  const __half* kc;        // [pages][Hkv][16][HD]
  const __half* vc;
  const int* page_table;   // [B][max_pages]
  const int* seq_lens;     // [B] keys to attend (includes the current token)
  const float* sinks;      // [Hq] or null
  int max_pages, Hq, Hkv, window, S;
  float* out_f32;          // [B][Hq*HD] or null
  __nv_bfloat16* out_bf16; // [B][Hq*HD] or null
  int8_t* oq;              // quantized output for a following mat-vec, or null
  float* od;
  float* os16;
  float* part_acc;         // [B*Hkv*S*G][HD]
  float* part_ml;          // [B*Hkv*S*G][2]
  int* counters;           // [B*Hkv], zero before first use; left zero on exit
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

template <int HD, int G>
__global__ void __launch_bounds__(128) attn_decode_kernel(const AttnDecArgs a) {
  constexpr int DL = HD / 8;  // dims per lane
  const int split = blockIdx.x, kh = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, grp = lane >> 3, sub = lane & 7;
  const int len = a.seq_lens[b];
  const int first = (a.window > 0 && len > a.window) ? len - a.window : 0;
  const int p_first = first >> 4, p_last = (len + 15) >> 4;
  const int per = (p_last - p_first + a.S - 1) / a.S;
  const int pa = p_first + split * per;
  const int pb = min(p_last, pa + per);

  __shared__ float s_acc[4][G][HD];
  __shared__ float s_ml[4][G][2];
  __shared__ int s_last;

  float q[G][DL], acc[G][DL], m[G], l[G];
#pragma unroll
  for (int g = 0; g < G; g++) {
    const float* qp = a.q + (size_t)b * a.Hq * HD + (size_t)(kh * G + g) * HD + sub * DL;
#pragma unroll
    for (int i = 0; i < DL; i += 4) {
      const float4 v = *(const float4*)(qp + i);
      q[g][i] = v.x; q[g][i + 1] = v.y; q[g][i + 2] = v.z; q[g][i + 3] = v.w;
    }
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < DL; i++) acc[g][i] = 0.f;
  }

  const int tok = warp * 4 + grp;
  const int* pt = a.page_table + (size_t)b * a.max_pages;
#pragma unroll 2
  for (int p = pa; p < pb; p++) {
    const int pid = pt[p];
    const int t = p * 16 + tok;
    const bool valid = t >= first && t < len;
    const size_t off = (((size_t)pid * a.Hkv + kh) * 16 + tok) * HD + sub * DL;
    float kf[DL], vf[DL];
#pragma unroll
    for (int i = 0; i < DL; i += 8) {
      const uint4 kr = ldg_stream(a.kc + off + i);
      const uint4 vr = ldg_stream(a.vc + off + i);
      const __half2* kh2 = (const __half2*)&kr;
      const __half2* vh2 = (const __half2*)&vr;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float2 kk = __half22float2(kh2[j]);
        const float2 vv = __half22float2(vh2[j]);
        kf[i + 2 * j] = kk.x; kf[i + 2 * j + 1] = kk.y;
        vf[i + 2 * j] = vv.x; vf[i + 2 * j + 1] = vv.y;
      }
    }
#pragma unroll
    for (int g = 0; g < G; g++) {
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < DL; i++) s += q[g][i] * kf[i];
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      if (valid) {
        const float mn = fmaxf(m[g], s);
        const float c = exp_scale(m[g], mn);
        const float pr = __expf(s - mn);
        l[g] = l[g] * c + pr;
#pragma unroll
        for (int i = 0; i < DL; i++) acc[g][i] = acc[g][i] * c + pr * vf[i];
        m[g] = mn;
      }
    }
  }

  // merge the four token groups of the warp
#pragma unroll
  for (int o = 8; o <= 16; o <<= 1) {
#pragma unroll
    for (int g = 0; g < G; g++) {
      const float mo = __shfl_xor_sync(0xffffffffu, m[g], o);
      const float lo = __shfl_xor_sync(0xffffffffu, l[g], o);
      const float M = fmaxf(m[g], mo);
      const float c0 = exp_scale(m[g], M), c1 = exp_scale(mo, M);
      l[g] = l[g] * c0 + lo * c1;
#pragma unroll
      for (int i = 0; i < DL; i++) {
        const float ao = __shfl_xor_sync(0xffffffffu, acc[g][i], o);
        acc[g][i] = acc[g][i] * c0 + ao * c1;
      }
      m[g] = M;
    }
  }
  if (grp == 0) {
#pragma unroll
    for (int g = 0; g < G; g++) {
#pragma unroll
      for (int i = 0; i < DL; i++) s_acc[warp][g][sub * DL + i] = acc[g][i];
      if (sub == 0) {
        s_ml[warp][g][0] = m[g];
        s_ml[warp][g][1] = l[g];
      }
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
static int launch(const AttnDecArgs& a, int B, cudaStream_t st) {
  dim3 grid(a.S, a.Hkv, B);
  attn_decode_kernel<HD, G><<<grid, 128, 0, st>>>(a);
  return (int)cudaGetLastError();
}

// Floats of scratch the split-merge needs: part_acc then part_ml, plus B*Hkv ints of counters.
B200_API size_t b200_attn_decode_scratch_floats(int B, int Hq, int Hkv, int hd, int S) {
  return (size_t)B * Hq * S * (hd + 2);
}

B200_API int b200_attn_decode(const float* q, const void* kc, const void* vc, const int* page_table,
                              int max_pages, const int* seq_lens, const float* sinks, int B, int Hq,
                              int Hkv, int hd, int window, int S, float* out_f32, void* out_bf16,
                              void* oq, float* od, float* os16, float* scratch, int* counters,
                              cudaStream_t st) {
  if (Hq % Hkv || S < 1) return B200_ERR_BAD_ARG;
  const int G = Hq / Hkv;
  AttnDecArgs a;
  a.q = q; a.kc = (const __half*)kc; a.vc = (const __half*)vc; a.page_table = page_table;
  a.seq_lens = seq_lens; a.sinks = sinks; a.max_pages = max_pages; a.Hq = Hq; a.Hkv = Hkv;
  a.window = window; a.S = S; a.out_f32 = out_f32; a.out_bf16 = (__nv_bfloat16*)out_bf16;
  a.oq = (int8_t*)oq; a.od = od; a.os16 = os16;
  a.part_acc = scratch;
  a.part_ml = scratch ? scratch + (size_t)B * Hq * S * hd : nullptr;
  a.counters = counters;
  if (S > 1 && (!scratch || !counters)) return B200_ERR_BAD_ARG;
  if (hd == 128) {
    switch (G) {
      case 1: return launch<128, 1>(a, B, st);
      case 2: return launch<128, 2>(a, B, st);
      case 4: return launch<128, 4>(a, B, st);
      case 8: return launch<128, 8>(a, B, st);
    }
  } else if (hd == 64) {
    switch (G) {
      case 1: return launch<64, 1>(a, B, st);
      case 2: return launch<64, 2>(a, B, st);
      case 4: return launch<64, 4>(a, B, st);
      case 8: return launch<64, 8>(a, B, st);
    }
  }
  return B200_ERR_BAD_ARG;
}
