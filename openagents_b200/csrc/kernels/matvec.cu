// Small-batch (1..8 tokens) quantized mat-vec: y[b][n] = sum_k W[n][k] * x[b][k], the decode-time
// projection of a GGUF-quantized weight.  Weights stream from HBM exactly once in their packed
// form; activations are pre-quantized to int8 (32-element blocks) so the inner product runs on
// dp4a and a whole CTA's activations fit in shared memory.  One CTA owns 32 output rows so the
// epilogue can emit a complete 32-element quantized block for the next mat-vec (fused SwiGLU +
// requantize), add the residual, or add a bias.
//
// Reference math: per-position projections of
// apps/openagents.com/workers/api/src/cs336-a1-real-gradient-workload.ts:459-475 (QKV),
// :520-528 (output projection + residual), :532-559 (SwiGLU FFN).
#include "../comm/sym.cuh"

using namespace b200;

enum { WT_Q4KR = 0, WT_Q6KR = 1, WT_Q8R = 2, WT_BF16 = 3 };
enum { EPI_STORE = 0, EPI_RESID = 1, EPI_SWIGLU_Q8 = 2, EPI_SWIGLU_F32 = 3, EPI_ALLREDUCE = 4, EPI_ROPE_KV = 5 };

struct MatvecArgs {
  const uint8_t* w;     // main plane
  const __half* w2;     // scale plane (Q6K-R: d per superblock; Q8-R: d per block)
  int N, K;             // output rows (per matrix when dual), reduction length
  int nb;               // live tokens (<= template B)
  const int8_t* xq;     // [nb][K] int8, x8 order
  const float* xd;      // [nb][K/32]
  const float* xs16;    // [nb][K/16]
  const float* xf;      // [nb][K] fp32 (bf16-weight path only)
  int epi;
  const float* bias;    // [N] or null (dual: [2N])
  const float* resid;   // [nb][ldy] (EPI_RESID)
  float* y;             // [nb][ldy]
  int ldy;
  int8_t* oq;           // EPI_SWIGLU_Q8 outputs
  float* od;
  float* os16;
  // EPI_ALLREDUCE: this rank's partial products are added into the fp32 tensor at byte offset
  // sym_off ([nb][ldy]) of EVERY rank's symmetric heap, and the kernel ends with a cross-rank
  // barrier, so on completion each replica holds resid + sum of all ranks' partials.
  SymTable sym;
  size_t sym_off;
  int prefetch;         // bring this CTA's weight rows into L2 before waiting for the previous kernel
  int wait_ready;       // EPI_ALLREDUCE: check the peers' "finished reading" signals before the first add
  // EPI_ROPE_KV: the matrix is the fused QKV projection of a model whose rotary pairs are ADJACENT rows (2j, 2j + 1).
  // The epilogue rotates q and k by the token's position, writes q (scaled) to q_out [nb][Hq * hd] and k / v as fp16
  // into the token's slot of the paged cache [page][Hkv][page_size][hd]: the separate rotary kernel's work.
  const int* pos;       // [nb]
  const int* slot;      // [nb] cache slot of the token (page * page_size + offset), < 0: do not write the cache
  const float2* tab;    // [tab_len][hd / 2] (cos, sin)
  int tab_len;
  float* q_out;
  __half* kc;
  __half* vc;
  int Hq, Hkv, hd, page_size;
  float q_scale, theta;
};

__device__ __forceinline__ int dp4a(uint32_t a, uint32_t b, int c) {
  return __dp4a((int)a, (int)b, c);
}

template <int WT>
__device__ __forceinline__ size_t row_bytes(int K) {
  if (WT == WT_Q4KR) return (size_t)(K / 256) * 144;
  if (WT == WT_Q6KR) return (size_t)(K / 256) * 208;
  return (size_t)K;  // Q8R
}

// Raw bytes of one 32-element unit of one weight row, fetched in a load phase that is kept apart
// from the arithmetic so that many loads are in flight per lane.
template <int WT>
struct UnitRaw {
  uint4 a;      // Q4K-R: header; Q6K-R: low nibbles; Q8-R: first 16 bytes
  uint4 b;      // Q4K-R: quants; Q6K-R: {T words, scales, d}; Q8-R: second 16 bytes
  uint32_t c;   // Q8-R: fp16 scale
};

template <int WT>
__device__ __forceinline__ UnitRaw<WT> unit_load(const uint8_t* __restrict__ wrow, const __half* __restrict__ w2row,
                                                 int u) {
  UnitRaw<WT> r;
  const int sb = u >> 3, j = u & 7;
  if constexpr (WT == WT_Q4KR) {
    const uint8_t* blk = wrow + (size_t)sb * 144;
    r.a = __ldg((const uint4*)blk);
    r.b = ldg_stream(blk + 16 + j * 16);
    r.c = 0;
  } else if constexpr (WT == WT_Q6KR) {
    const uint8_t* blk = wrow + (size_t)sb * 208;
    r.a = ldg_stream(blk + j * 16);
    const uint2 tw = ldg_stream2(blk + 128 + j * 8);
    r.b.x = tw.x;
    r.b.y = tw.y;
    r.b.z = ((const uint16_t*)(blk + 192))[j];
    r.b.w = __half_as_ushort(w2row[sb]);
    r.c = 0;
  } else {
    r.a = ldg_stream(wrow + (size_t)u * 32);
    r.b = ldg_stream(wrow + (size_t)u * 32 + 16);
    r.c = __half_as_ushort(w2row[u]);
  }
  return r;
}

// Dot of one loaded unit against all B tokens.
template <int WT, int B>
__device__ __forceinline__ void unit_dot(const UnitRaw<WT>& r, int u, int U, const uint4* __restrict__ xp0,
                                         const uint4* __restrict__ xp1, const float* __restrict__ sxd,
                                         const float2* __restrict__ sxs, float (&acc)[B]) {
  const int j = u & 7;
  if constexpr (WT == WT_Q4KR) {
    const uint4 hdr = r.a, q = r.b;
    const int sh = 8 * (j & 3);
    const uint32_t b0 = (hdr.y >> sh) & 0xFF, b1 = (hdr.z >> sh) & 0xFF, b2 = (hdr.w >> sh) & 0xFF;
    const uint32_t sc = j < 4 ? (b0 & 63) : ((b2 & 0xF) | ((b0 >> 6) << 4));
    const uint32_t mn = j < 4 ? (b1 & 63) : ((b2 >> 4) | ((b1 >> 6) << 4));
    const __half2 dd = *reinterpret_cast<const __half2*>(&hdr.x);
    const float a = __low2float(dd) * (float)sc, m = __high2float(dd) * (float)mn;
    const uint32_t l0 = q.x & 0x0F0F0F0Fu, h0 = (q.x >> 4) & 0x0F0F0F0Fu;
    const uint32_t l1 = q.y & 0x0F0F0F0Fu, h1 = (q.y >> 4) & 0x0F0F0F0Fu;
    const uint32_t l2 = q.z & 0x0F0F0F0Fu, h2 = (q.z >> 4) & 0x0F0F0F0Fu;
    const uint32_t l3 = q.w & 0x0F0F0F0Fu, h3 = (q.w >> 4) & 0x0F0F0F0Fu;
#pragma unroll
    for (int b = 0; b < B; b++) {
      const uint4 x0 = xp0[b * U + u], x1 = xp1[b * U + u];
      int s = dp4a(l0, x0.x, 0);
      s = dp4a(h0, x0.y, s);
      s = dp4a(l1, x0.z, s);
      s = dp4a(h1, x0.w, s);
      s = dp4a(l2, x1.x, s);
      s = dp4a(h2, x1.y, s);
      s = dp4a(l3, x1.z, s);
      s = dp4a(h3, x1.w, s);
      const float2 xs = sxs[b * U + u];
      acc[b] += a * sxd[b * U + u] * (float)s - m * (xs.x + xs.y);
    }
  } else if constexpr (WT == WT_Q6KR) {
    const uint4 lo = r.a;
    const uint2 tw = make_uint2(r.b.x, r.b.y);
    const uint32_t scw = r.b.z;
    const float d = __half2float(__ushort_as_half((unsigned short)r.b.w));
    const float sc0 = d * (float)(int8_t)(scw & 0xFF), sc1 = d * (float)(int8_t)(scw >> 8);
    const uint32_t m4 = 0x0F0F0F0Fu, m2 = 0x03030303u;
    const uint32_t a0 = (lo.x & m4) | ((tw.x & m2) << 4), a1 = ((lo.x >> 4) & m4) | (((tw.x >> 2) & m2) << 4);
    const uint32_t a2 = (lo.y & m4) | (((tw.x >> 4) & m2) << 4), a3 = ((lo.y >> 4) & m4) | (((tw.x >> 6) & m2) << 4);
    const uint32_t c0 = (lo.z & m4) | ((tw.y & m2) << 4), c1 = ((lo.z >> 4) & m4) | (((tw.y >> 2) & m2) << 4);
    const uint32_t c2 = (lo.w & m4) | (((tw.y >> 4) & m2) << 4), c3 = ((lo.w >> 4) & m4) | (((tw.y >> 6) & m2) << 4);
#pragma unroll
    for (int b = 0; b < B; b++) {
      const uint4 x0 = xp0[b * U + u], x1 = xp1[b * U + u];
      int s0 = dp4a(a0, x0.x, 0);
      s0 = dp4a(a1, x0.y, s0);
      s0 = dp4a(a2, x0.z, s0);
      s0 = dp4a(a3, x0.w, s0);
      int s1 = dp4a(c0, x1.x, 0);
      s1 = dp4a(c1, x1.y, s1);
      s1 = dp4a(c2, x1.z, s1);
      s1 = dp4a(c3, x1.w, s1);
      const float2 xs = sxs[b * U + u];
      const float xd = sxd[b * U + u];
      acc[b] += sc0 * (xd * (float)s0 - 32.f * xs.x) + sc1 * (xd * (float)s1 - 32.f * xs.y);
    }
  } else {  // WT_Q8R
    const uint4 q0 = r.a, q1 = r.b;
    const float d = __half2float(__ushort_as_half((unsigned short)r.c));
#pragma unroll
    for (int b = 0; b < B; b++) {
      const uint4 x0 = xp0[b * U + u], x1 = xp1[b * U + u];
      int s = dp4a(q0.x, x0.x, 0);
      s = dp4a(q0.y, x0.y, s);
      s = dp4a(q0.z, x0.z, s);
      s = dp4a(q0.w, x0.w, s);
      s = dp4a(q1.x, x1.x, s);
      s = dp4a(q1.y, x1.y, s);
      s = dp4a(q1.z, x1.z, s);
      s = dp4a(q1.w, x1.w, s);
      acc[b] += d * sxd[b * U + u] * (float)s;
    }
  }
}

// Shared epilogue: res[m][r][b] holds the R x B results of matrix m (m = 1 only when dual); R is the
// number of rows a CTA owns (32, or fewer for small matrices so that more CTAs share the stream).
template <int B, int R = 32>
__device__ __forceinline__ void matvec_epilogue(const MatvecArgs& a, const float* res, bool dual) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (w >= a.nb) return;
  const int b = w;
  const int n = blockIdx.x * R + lane;
  const bool live = lane < R && n < a.N;
  float v = res[lane * B + b];
  if (a.bias && live && (a.epi != EPI_ALLREDUCE || a.sym.rank == 0)) v += a.bias[dual ? 2 * n : n];
  if (a.epi == EPI_ROPE_KV) {
    const float other = __shfl_xor_sync(0xffffffffu, v, 1);      // the pair's partner row sits in the neighbouring lane
    if (!live) return;
    const int qd = a.Hq * a.hd, kd = a.Hkv * a.hd, half = a.hd >> 1;
    const int s = a.slot[b];
    const int page = s >= 0 ? s / a.page_size : 0, off = s >= 0 ? s % a.page_size : 0;
    if (n >= qd + kd) {
      if (s >= 0) {
        const int e = n - qd - kd, kh = e / a.hd, c = e % a.hd;
        a.vc[(((size_t)page * a.Hkv + kh) * a.page_size + off) * a.hd + c] = __float2half(v);
      }
      return;
    }
    const int h = n / a.hd, e = n % a.hd, j = e >> 1;
    const int p = a.pos[b];
    float cs, sn;
    if (a.tab && p >= 0 && p < a.tab_len) {
      const float2 t = a.tab[(size_t)p * half + j];
      cs = t.x;
      sn = t.y;
    } else {                       // outside the table: double precision, as the table was built
      const double inv = exp2(-2.0 * (double)j / (double)a.hd * log2((double)a.theta));
      double snd, csd;
      sincos((double)p * inv, &snd, &csd);
      sn = (float)snd;
      cs = (float)csd;
    }
    const float r = (e & 1) ? other * sn + v * cs : v * cs - other * sn;
    if (h < a.Hq) a.q_out[(size_t)b * qd + n] = r * a.q_scale;
    else if (s >= 0) a.kc[(((size_t)page * a.Hkv + (h - a.Hq)) * a.page_size + off) * a.hd + e] = __float2half(r);
    return;
  }
  if (a.epi == EPI_STORE) {
    if (live) a.y[(size_t)b * a.ldy + n] = v;
    if (dual && live) {
      float v2 = res[32 * B + lane * B + b] + (a.bias ? a.bias[2 * n + 1] : 0.f);
      a.y[(size_t)b * a.ldy + a.N + n] = v2;
    }
  } else if (a.epi == EPI_RESID) {
    if (live) a.y[(size_t)b * a.ldy + n] = a.resid[(size_t)b * a.ldy + n] + v;
  } else if (a.epi == EPI_ALLREDUCE) {
    if (live) sym_red_all_f32(a.sym, a.sym_off + ((size_t)b * a.ldy + n) * 4, v);
  } else {
    float u = res[32 * B + lane * B + b];
    if (a.bias && live) u += a.bias[2 * n + 1];
    const float act = live ? silu(v) * u : 0.f;
    if (a.epi == EPI_SWIGLU_F32) {
      if (live) a.y[(size_t)b * a.ldy + n] = act;
    } else {
      quantize_block32(act, lane, a.oq + (size_t)b * a.N + blockIdx.x * 32,
                       a.od + (size_t)b * (a.N / 32) + blockIdx.x,
                       a.os16 + (size_t)b * (a.N / 16) + blockIdx.x * 2);
    }
  }
}

template <int WT, int B, bool DUAL, int RW>
__global__ void __launch_bounds__(256) matvec_q_kernel(const MatvecArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  constexpr int R = 8 * RW;   // rows per CTA
  static_assert(!DUAL || RW == 4, "the SwiGLU epilogue quantizes 32-row blocks");
  const int U = a.K / 32;
  {
    // This CTA's weight rows are one contiguous range (two when dual).  Ask for them in L2 now: the
    // kernel before this one in the stream may still be running, and the weights do not depend on it.
    const size_t rbp = row_bytes<WT>(a.K);
    const int r0 = blockIdx.x * R;
    const int nr = min(R, a.N - r0);
    if (nr > 0 && a.prefetch) {
      // dual: the (gate, up) rows of output row n are rows 2n and 2n + 1 of the matrix, so one range of 2 nr rows
      const size_t total = (size_t)nr * rbp * (DUAL ? 2 : 1);     // multiple of 16: every row is
      constexpr uint32_t CH = 16384;
      const int nch = (int)((total + CH - 1) / CH);
      const uint8_t* base = a.w + (size_t)r0 * (DUAL ? 2 : 1) * rbp;
      for (int c = threadIdx.x; c < nch; c += 256) {
        const size_t off = (size_t)c * CH;
        prefetch_l2(base + off, (uint32_t)min((size_t)CH, total - off));
      }
    }
  }
  pdl_trigger();
  pdl_wait();
  uint4* xp0 = (uint4*)smem;                  // [B][U]
  uint4* xp1 = xp0 + B * U;                   // [B][U]
  float* sxd = (float*)(xp1 + B * U);         // [B][U]
  float2* sxs = (float2*)(sxd + B * U);       // [B][U]
  float* res = (float*)(sxs + B * U);         // [2][32][B]
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;

  // Stage the quantized activations (a few KB per token) into shared memory, split into two
  // 16-byte planes so a warp's reads are conflict-free.
  for (int i = tid; i < B * U; i += 256) {
    const int b = i / U, u = i - b * U;
    if (b < a.nb) {
      const uint4* src = (const uint4*)(a.xq + (size_t)b * a.K + (size_t)u * 32);
      xp0[i] = src[0];
      xp1[i] = src[1];
      sxd[i] = a.xd[(size_t)b * U + u];
      sxs[i] = ((const float2*)a.xs16)[(size_t)b * U + u];
    } else {
      xp0[i] = make_uint4(0, 0, 0, 0);
      xp1[i] = make_uint4(0, 0, 0, 0);
      sxd[i] = 0.f;
      sxs[i] = make_float2(0.f, 0.f);
    }
  }
  __syncthreads();

  const size_t rb = row_bytes<WT>(a.K);
  const int w2_per_row = (WT == WT_Q6KR) ? a.K / 256 : U;
  constexpr int NM = DUAL ? 2 : 1;  // matrices
  float acc[NM][RW][B];
#pragma unroll
  for (int mi = 0; mi < NM; mi++)
#pragma unroll
    for (int i = 0; i < RW; i++)
#pragma unroll
      for (int b = 0; b < B; b++) acc[mi][i][b] = 0.f;
  const uint8_t* wr[NM][RW];
  const __half* w2r[NM][RW];
  bool live[RW];
#pragma unroll
  for (int i = 0; i < RW; i++) {
    const int n = blockIdx.x * R + w + 8 * i;
    live[i] = n < a.N;
    const int nn = live[i] ? n : 0;
#pragma unroll
    for (int mi = 0; mi < NM; mi++) {
      const size_t wrow = DUAL ? (size_t)(2 * nn + mi) : (size_t)nn;     // dual: rows interleaved (gate_n, up_n)
      wr[mi][i] = a.w + wrow * rb;
      w2r[mi][i] = a.w2 ? a.w2 + wrow * w2_per_row : nullptr;
    }
  }
  // Load phase (all rows of the warp, both matrices) then compute phase, per 32-unit column block.
#pragma unroll 2
  for (int u = lane; u < U; u += 32) {
    UnitRaw<WT> raw[NM][RW];
#pragma unroll
    for (int mi = 0; mi < NM; mi++)
#pragma unroll
      for (int i = 0; i < RW; i++) raw[mi][i] = unit_load<WT>(wr[mi][i], w2r[mi][i], u);
#pragma unroll
    for (int mi = 0; mi < NM; mi++)
#pragma unroll
      for (int i = 0; i < RW; i++) unit_dot<WT, B>(raw[mi][i], u, U, xp0, xp1, sxd, sxs, acc[mi][i]);
  }
#pragma unroll
  for (int i = 0; i < RW; i++) {
    const int r = w + 8 * i;
#pragma unroll
    for (int b = 0; b < B; b++) {
      float v0 = warp_sum(acc[0][i][b]);
      if (lane == 0) res[r * B + b] = live[i] ? v0 : 0.f;
      if (DUAL) {
        float v1 = warp_sum(acc[NM - 1][i][b]);
        if (lane == 0) res[32 * B + r * B + b] = live[i] ? v1 : 0.f;
      }
    }
  }
  if (a.epi == EPI_ALLREDUCE && a.wait_ready && threadIdx.x == 0) sym_wait_ready(a.sym);
  __syncthreads();
  matvec_epilogue<B, R>(a, res, DUAL);
  if (a.epi == EPI_ALLREDUCE) sym_kernel_end_barrier(a.sym, 0, gridDim.x, a.wait_ready != 0);
}

// bf16 weights [N][K] against fp32 activations.
template <int B, bool DUAL>
__global__ void __launch_bounds__(256) matvec_bf16_kernel(const MatvecArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  float* xs = (float*)smem;            // [B][K]
  float* res = xs + (size_t)B * a.K;   // [2][32][B]
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  pdl_trigger();
  pdl_wait();
  for (int i = tid; i < B * a.K; i += 256) {
    const int b = i / a.K;
    xs[i] = b < a.nb ? a.xf[i] : 0.f;
  }
  __syncthreads();
  const __nv_bfloat16* W = (const __nv_bfloat16*)a.w;
#pragma unroll 1
  for (int i = 0; i < 4; i++) {
    const int r = w + 8 * i;
    const int n = blockIdx.x * 32 + r;
    float acc0[B], acc1[B];
#pragma unroll
    for (int b = 0; b < B; b++) acc0[b] = acc1[b] = 0.f;
    if (n < a.N) {
      const __nv_bfloat16* wr0 = W + (size_t)(DUAL ? 2 * n : n) * a.K;     // dual: rows interleaved (gate_n, up_n)
      const __nv_bfloat16* wr1 = W + (size_t)(2 * n + 1) * a.K;
#pragma unroll 2
      for (int k = lane * 8; k < a.K; k += 256) {
        const uint4 q0 = ldg_stream(wr0 + k);
        uint4 q1 = make_uint4(0, 0, 0, 0);
        if (DUAL) q1 = ldg_stream(wr1 + k);
        const __nv_bfloat162* p0 = (const __nv_bfloat162*)&q0;
        const __nv_bfloat162* p1 = (const __nv_bfloat162*)&q1;
#pragma unroll
        for (int b = 0; b < B; b++) {
          const float4 xa = *(const float4*)(xs + (size_t)b * a.K + k);
          const float4 xb = *(const float4*)(xs + (size_t)b * a.K + k + 4);
          float2 f;
          f = __bfloat1622float2(p0[0]); acc0[b] += f.x * xa.x + f.y * xa.y;
          f = __bfloat1622float2(p0[1]); acc0[b] += f.x * xa.z + f.y * xa.w;
          f = __bfloat1622float2(p0[2]); acc0[b] += f.x * xb.x + f.y * xb.y;
          f = __bfloat1622float2(p0[3]); acc0[b] += f.x * xb.z + f.y * xb.w;
          if (DUAL) {
            f = __bfloat1622float2(p1[0]); acc1[b] += f.x * xa.x + f.y * xa.y;
            f = __bfloat1622float2(p1[1]); acc1[b] += f.x * xa.z + f.y * xa.w;
            f = __bfloat1622float2(p1[2]); acc1[b] += f.x * xb.x + f.y * xb.y;
            f = __bfloat1622float2(p1[3]); acc1[b] += f.x * xb.z + f.y * xb.w;
          }
        }
      }
    }
#pragma unroll
    for (int b = 0; b < B; b++) {
      float v0 = warp_sum(acc0[b]);
      if (lane == 0) res[r * B + b] = v0;
      if (DUAL) {
        float v1 = warp_sum(acc1[b]);
        if (lane == 0) res[32 * B + r * B + b] = v1;
      }
    }
  }
  if (a.epi == EPI_ALLREDUCE && a.wait_ready && threadIdx.x == 0) sym_wait_ready(a.sym);
  __syncthreads();
  matvec_epilogue<B>(a, res, DUAL);
  if (a.epi == EPI_ALLREDUCE) sym_kernel_end_barrier(a.sym, 0, gridDim.x, a.wait_ready != 0);
}

template <int WT, int B, bool DUAL, int RW>
static int launch_q_rw(const MatvecArgs& a, cudaStream_t st) {
  const int U = a.K / 32;
  const size_t smem = (size_t)B * U * (16 + 16 + 4 + 8) + 2 * 32 * B * sizeof(float);
  auto kern = matvec_q_kernel<WT, B, DUAL, RW>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  constexpr int R = 8 * RW;
  return launch_pdl(kern, dim3((a.N + R - 1) / R), dim3(256), smem, st, a);
}
template <int WT, int B, bool DUAL>
static int launch_q(const MatvecArgs& a, cudaStream_t st) {
  // One or two tokens and a matrix of a few thousand rows: 32-row CTAs would leave SMs idle and too
  // few loads in flight, so a CTA takes 8 rows instead.
  if constexpr (!DUAL && B <= 2) {
    if ((a.N + 31) / 32 < 3 * 148) return launch_q_rw<WT, B, DUAL, 1>(a, st);
  }
  return launch_q_rw<WT, B, DUAL, 4>(a, st);
}
template <int B, bool DUAL>
static int launch_bf16(const MatvecArgs& a, cudaStream_t st) {
  const size_t smem = (size_t)B * a.K * 4 + 2 * 32 * B * sizeof(float);
  auto kern = matvec_bf16_kernel<B, DUAL>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  return launch_pdl(kern, dim3((a.N + 31) / 32), dim3(256), smem, st, a);
}

template <int B, bool DUAL>
static int dispatch_wt(int wt, const MatvecArgs& a, cudaStream_t st) {
  switch (wt) {
    case WT_Q4KR: return launch_q<WT_Q4KR, B, DUAL>(a, st);
    case WT_Q6KR: return launch_q<WT_Q6KR, B, DUAL>(a, st);
    case WT_Q8R: return launch_q<WT_Q8R, B, DUAL>(a, st);
    case WT_BF16: return launch_bf16<B, DUAL>(a, st);
  }
  return B200_ERR_BAD_ARG;
}

// wt: weight layout; nb: tokens (1..8).  For the SwiGLU epilogues `w` holds 2N rows, interleaved
// (gate_0, up_0, gate_1, ...: the order the GEMMs' SwiGLU epilogues pair rows in, so one copy of the matrix
// serves every batch size) and N is the width of one of them; a bias is interleaved the same way.
static int run_matvec(int wt, MatvecArgs& a, cudaStream_t st) {
  const int nb = a.nb, epi = a.epi;
  a.prefetch = b200_prefetch_enabled();
  const bool dual = epi == EPI_SWIGLU_Q8 || epi == EPI_SWIGLU_F32;
  const int B = nb <= 1 ? 1 : nb <= 2 ? 2 : nb <= 4 ? 4 : 8;
  if (dual) {
    switch (B) {
      case 1: return dispatch_wt<1, true>(wt, a, st);
      case 2: return dispatch_wt<2, true>(wt, a, st);
      case 4: return dispatch_wt<4, true>(wt, a, st);
      default: return dispatch_wt<8, true>(wt, a, st);
    }
  }
  switch (B) {
    case 1: return dispatch_wt<1, false>(wt, a, st);
    case 2: return dispatch_wt<2, false>(wt, a, st);
    case 4: return dispatch_wt<4, false>(wt, a, st);
    default: return dispatch_wt<8, false>(wt, a, st);
  }
}

B200_API int b200_matvec(int wt, const void* w, const void* w2, int N, int K, int nb, const void* xq,
                         const float* xd, const float* xs16, const float* xf, int epi, const float* bias,
                         const float* resid, float* y, int ldy, void* oq, float* od, float* os16,
                         const SymTable* sym, size_t sym_off, int wait_ready, cudaStream_t st) {
  if (nb < 1 || nb > 8 || epi == EPI_ROPE_KV) return B200_ERR_BAD_ARG;
  if (wt == WT_BF16 ? (K % 8 != 0) : (K % 256 != 0 && !(wt == WT_Q8R && K % 32 == 0))) return B200_ERR_BAD_ARG;
  if (epi == EPI_SWIGLU_Q8 && N % 32) return B200_ERR_BAD_ARG;
  MatvecArgs a = {};
  a.w = (const uint8_t*)w; a.w2 = (const __half*)w2; a.N = N; a.K = K; a.nb = nb;
  a.xq = (const int8_t*)xq; a.xd = xd; a.xs16 = xs16; a.xf = xf; a.epi = epi; a.bias = bias;
  a.resid = resid; a.y = y; a.ldy = ldy; a.oq = (int8_t*)oq; a.od = od; a.os16 = os16;
  if (epi == EPI_ALLREDUCE) {
    if (!sym) return B200_ERR_BAD_ARG;
    a.sym = *sym;
    a.sym_off = sym_off;
  } else {
    a.sym = SymTable{};
    a.sym_off = 0;
  }
  a.wait_ready = wait_ready;
  return run_matvec(wt, a, st);
}

// The fused QKV projection of 1-8 tokens with the rotary embedding and the paged-cache write in its epilogue
// (adjacent-pair rotary layout only).  N = (Hq + 2 Hkv) * hd rows; q_out [nb][Hq * hd] fp32, scaled by q_scale;
// kc / vc fp16 [n_pages][Hkv][page_size][hd]; slot[b] < 0 skips the cache write of token b.
B200_API int b200_matvec_rope_kv(int wt, const void* w, const void* w2, int K, int nb, const void* xq, const float* xd,
                                 const float* xs16, const float* xf, const float* bias, const int* pos, const int* slot,
                                 const void* tab, int tab_len, float* q_out, void* kc, void* vc, int Hq, int Hkv, int hd,
                                 int page_size, float theta, float q_scale, cudaStream_t st) {
  if (nb < 1 || nb > 8 || Hq < 1 || Hkv < 1 || hd < 2 || (hd & 1) || page_size < 1 || !pos || !slot || !q_out || !kc || !vc)
    return B200_ERR_BAD_ARG;
  if (wt == WT_BF16 ? (K % 8 != 0) : (K % 256 != 0 && !(wt == WT_Q8R && K % 32 == 0))) return B200_ERR_BAD_ARG;
  MatvecArgs a = {};
  a.w = (const uint8_t*)w; a.w2 = (const __half*)w2; a.N = (Hq + 2 * Hkv) * hd; a.K = K; a.nb = nb;
  a.xq = (const int8_t*)xq; a.xd = xd; a.xs16 = xs16; a.xf = xf; a.epi = EPI_ROPE_KV; a.bias = bias;
  a.sym = SymTable{};
  a.pos = pos; a.slot = slot; a.tab = (const float2*)tab; a.tab_len = tab ? tab_len : 0; a.q_out = q_out;
  a.kc = (__half*)kc; a.vc = (__half*)vc; a.Hq = Hq; a.Hkv = Hkv; a.hd = hd; a.page_size = page_size;
  a.q_scale = q_scale; a.theta = theta;
  return run_matvec(wt, a, st);
}
