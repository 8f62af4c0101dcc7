// Memory-bound decode-path operators: embedding gather with dequant, RMSNorm with fused activation
// quantization, RoPE fused with the paged KV-cache write, SwiGLU, residual add and greedy / top-k
// sampling.  The math follows the reference CPU workload
// (apps/openagents.com/workers/api/src/cs336-a1-real-gradient-workload.ts:351-375 RMSNorm,
// :532-549 SwiGLU, cs336-a2-benchmark-workload.ts:212-249 greedy arg-max decode).
#include "../comm/sym.cuh"

using namespace b200;

static int g_pdl = 1;
extern "C" __attribute__((visibility("default"))) int b200_pdl_enabled() { return g_pdl; }
// on = 0: launch every kernel fully serialised (no programmatic dependent launch).
B200_API int b200_set_pdl(int on) {
  g_pdl = on ? 1 : 0;
  return 0;
}
static int g_prefetch = 1;
extern "C" __attribute__((visibility("default"))) int b200_prefetch_enabled() { return g_prefetch; }
// on = 0: kernels do not prefetch their weights into L2 ahead of the dependency wait.
B200_API int b200_set_prefetch(int on) {
  g_prefetch = on ? 1 : 0;
  return 0;
}


// ------------------------------------------------------------------ embedding gather

// Weight types of the embedding table.
enum { EMB_F32 = 0, EMB_BF16 = 1, EMB_Q8R = 2, EMB_Q6KR = 3 };

// ids [T]; out fp32 [T][D].  `w` is the main plane, `w2` the scale plane (fp16) where one exists.
// vocab_lo / vocab_n select a vocabulary shard: rows outside it produce zeros (tensor-parallel
// embedding; the all-reduce that follows adds the one non-zero shard).
__global__ void embedding_kernel(const int* __restrict__ ids, float* __restrict__ out, int D, int type,
                                 const uint8_t* __restrict__ w, const __half* __restrict__ w2,
                                 int vocab_lo, int vocab_n) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t] - vocab_lo;
  float* o = out + (size_t)t * D;
  if (id < 0 || id >= vocab_n) {
    for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = 0.f;
    return;
  }
  if (type == EMB_F32) {
    const float* r = (const float*)w + (size_t)id * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = r[i];
  } else if (type == EMB_BF16) {
    const __nv_bfloat16* r = (const __nv_bfloat16*)w + (size_t)id * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = __bfloat162float(r[i]);
  } else if (type == EMB_Q8R) {
    const int8_t* r = (const int8_t*)w + (size_t)id * D;
    const __half* d = w2 + (size_t)id * (D / 32);
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
      int slot = (i & ~7) | x8_slot(i & 7);
      o[i] = __half2float(d[i >> 5]) * (float)r[slot];
    }
  } else {  // EMB_Q6KR: 208-byte superblocks [lo words 128][T words 64][scales 16] + d plane
    const int nsb = D / 256;
    const uint8_t* r = w + (size_t)id * nsb * 208;
    const __half* dp = w2 + (size_t)id * nsb;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
      const int sb = i >> 8, e = i & 255;
      const uint8_t* blk = r + sb * 208;
      const int word = e >> 3, ei = e & 7;
      const uint32_t lo = ((const uint32_t*)blk)[word];
      const uint32_t tw = ((const uint32_t*)(blk + 128))[word >> 1];
      const int nib = (lo >> (4 * (ei >> 1) + 16 * (ei & 1))) & 0xF;
      // 2-bit field: lane = slot & 3, half = slot >> 2 of the x8 slot, word parity selects +4
      const int slot = x8_slot(ei);
      const int hi = (tw >> (8 * (slot & 3) + 2 * (slot >> 2) + 4 * (word & 1))) & 3;
      const int q = (nib | (hi << 4)) - 32;
      const float sc = (float)((const int8_t*)(blk + 192))[e >> 4];
      o[i] = __half2float(dp[sb]) * sc * (float)q;
    }
  }
}

B200_API int b200_embedding(const int* ids, float* out, int T, int D, int type, const void* w,
                            const void* w2, int vocab_lo, int vocab_n, cudaStream_t st) {
  return launch_pdl(embedding_kernel, dim3(T), dim3(256), 0, st, ids, out, D, type, (const uint8_t*)w,
                    (const __half*)w2, vocab_lo, vocab_n);
}

// ------------------------------------------------------------------ RMSNorm (+ quantize)

// x fp32 [T][D] -> any of: quantized activations (xq int8 x8-order, xd [T][D/32], xs16 [T][D/16]),
// bf16 h [T][D], fp32 h [T][D].  One block per token; each warp owns 32-element blocks.  A decode
// step runs this on the critical path with one token, so the row and the gain are read once with
// all loads in flight together and kept in registers; only rows longer than kRmsRegs * 1024 fall
// back to re-reading.
constexpr int kRmsRegs = 8;
// sym_mode 1: tensor parallel, all-reduce form: x is replicated in the symmetric heap and peers add into it; the kernel
//             ends by telling them that this rank has finished reading (see sym_signal_ready).
// sym_mode 2: tensor parallel, slot form: this kernel IS the all-reduce.  The row-parallel projection before it left
//             this rank's partial result in `part` (local, fp32 [T][D]).  The CTA of row t pushes that row into this
//             rank's slot on every rank, raises the row's flag, waits for the world's pushes, adds the slots to x in
//             rank order (x <- x + sum, written back: x is this rank's private replica) and normalises the sum.  It
//             leaves its row of `part` zeroed, because the projection accumulates into it (K splits).  See sym.cuh.
__global__ void __launch_bounds__(1024) rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ g, float eps,
                                                       int D, int8_t* __restrict__ xq, float* __restrict__ xd,
                                                       float* __restrict__ xs16, __nv_bfloat16* __restrict__ hb,
                                                       float* __restrict__ hf, const __grid_constant__ SymTable sym, int sym_mode,
                                                       float4* __restrict__ zero, int zero_n4, size_t slot_off,
                                                       int slot_rows, float* __restrict__ part) {
  __shared__ float red[32];
  const int t = blockIdx.x;
  float* xr = x + (size_t)t * D;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int nblk = D / 32;
  float v[kRmsRegs], gg[kRmsRegs];
  float ss = 0.f;
  pdl_trigger();
#pragma unroll
  for (int k = 0; k < kRmsRegs; k++) {   // the gain is a weight: read it while the producer of x still runs
    const int blk = w + k * nw;
    gg[k] = (blk < nblk && g) ? g[blk * 32 + lane] : 1.f;
  }
  pdl_wait();
  const float* slot0 = nullptr;
  size_t slot_stride = 0;
  if (sym_mode == 2) {
    __shared__ uint32_t s_seq;
    SymControl* me = sym_ctl(sym, sym.rank);
    if (threadIdx.x == 0) s_seq = *(volatile uint32_t*)&me->row_seq[t] + 1u;
    __syncthreads();
    const uint32_t seq = s_seq;
    slot_stride = (size_t)slot_rows * D;
    const size_t par_off = (size_t)(seq & 1u) * sym.world * slot_stride + (size_t)t * D;      // in floats
    // push this rank's partial row, 16 bytes per lane, and leave it zeroed for the next projection
    float4* pr = (float4*)(part + (size_t)t * D);
    const size_t dst = slot_off + (par_off + (size_t)sym.rank * slot_stride) * 4;
    for (int i = threadIdx.x; i < D / 4; i += blockDim.x) {
      const float4 pv = pr[i];
      sym_st_all_v4(sym, dst + (size_t)i * 16, make_uint4(__float_as_uint(pv.x), __float_as_uint(pv.y), __float_as_uint(pv.z), __float_as_uint(pv.w)));
      pr[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      me->row_seq[t] = seq;
      sym_row_signal(sym, t);
      sym_row_wait(sym, t, seq);      // on a time-out the status word says so; the sum is then wrong, not hung
    }
    __syncthreads();
    slot0 = (const float*)(sym.base[sym.rank] + slot_off) + par_off;
  }
#pragma unroll
  for (int k = 0; k < kRmsRegs; k++) {
    const int blk = w + k * nw;
    v[k] = blk < nblk ? xr[blk * 32 + lane] : 0.f;
  }
  if (sym_mode == 2) {
#pragma unroll
    for (int k = 0; k < kRmsRegs; k++) {
      const int blk = w + k * nw;
      if (blk < nblk) {
        float acc = v[k];
        for (int r = 0; r < sym.world; r++) acc += __ldcg(slot0 + (size_t)r * slot_stride + blk * 32 + lane);
        v[k] = acc;
        xr[blk * 32 + lane] = acc;
      }
    }
    for (int blk = w + kRmsRegs * nw; blk < nblk; blk += nw) {     // long rows: the tail is re-read below, so sum it in place first
      float acc = xr[blk * 32 + lane];
      for (int r = 0; r < sym.world; r++) acc += __ldcg(slot0 + (size_t)r * slot_stride + blk * 32 + lane);
      xr[blk * 32 + lane] = acc;
    }
  }
  // Clear the output of the split-K GEMM that consumes this norm (its splits add their partial sums).
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < zero_n4; i += gridDim.x * blockDim.x)
    zero[i] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int k = 0; k < kRmsRegs; k++) ss += v[k] * v[k];
  for (int blk = w + kRmsRegs * nw; blk < nblk; blk += nw) {
    const float e = xr[blk * 32 + lane];
    ss += e * e;
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / (float)D + eps);
#pragma unroll
  for (int k = 0; k < kRmsRegs; k++) {
    const int blk = w + k * nw;
    if (blk < nblk) {
      const int i = blk * 32 + lane;
      const float o = v[k] * rstd * gg[k];
      if (hb) hb[(size_t)t * D + i] = __float2bfloat16(o);
      if (hf) hf[(size_t)t * D + i] = o;
      if (xq)
        quantize_block32(o, lane, xq + (size_t)t * D + blk * 32, xd + (size_t)t * (D / 32) + blk,
                         xs16 + (size_t)t * (D / 16) + blk * 2);
    }
  }
  for (int blk = w + kRmsRegs * nw; blk < nblk; blk += nw) {
    const int i = blk * 32 + lane;
    const float o = xr[i] * rstd * (g ? g[i] : 1.f);
    if (hb) hb[(size_t)t * D + i] = __float2bfloat16(o);
    if (hf) hf[(size_t)t * D + i] = o;
    if (xq)
      quantize_block32(o, lane, xq + (size_t)t * D + blk * 32, xd + (size_t)t * (D / 32) + blk,
                       xs16 + (size_t)t * (D / 16) + blk * 2);
  }
  // Tensor parallel, all-reduce form: x is replicated and peers add into it from their row-parallel kernels; tell them
  // this rank has finished reading the values it needed.
  if (sym_mode == 1) sym_signal_ready(sym, gridDim.x);
}

// sym_mode 0: plain.  1: x lives in the symmetric heap and the next row-parallel kernel of every rank will add into
// it; this kernel then ends by signalling that this rank has read x (see sym.cuh).  2: all-reduce this rank's partial
// rows `part` (fp32 [T][D], local) through the per-rank slots at heap offset slot_off ([2][world][slot_rows][D] fp32)
// and add the sum into x first (see the kernel).
// zero / zero_n: an fp32 buffer (16-byte aligned, zero_n a multiple of 4) that the kernel clears on the side.
B200_API int b200_rmsnorm(float* x, const float* g, float eps, int T, int D, void* xq, float* xd,
                          float* xs16, void* hb, float* hf, const SymTable* sym, int sym_mode, float* zero, long zero_n,
                          size_t slot_off, int slot_rows, float* part, cudaStream_t st) {
  if (D % 32 || (zero && ((zero_n % 4) || ((uintptr_t)zero % 16)))) return B200_ERR_BAD_ARG;
  if ((sym_mode != 0 && !sym) || sym_mode < 0 || sym_mode > 2 || (sym_mode == 2 && (T > slot_rows || slot_rows > kSymSlotRows || (slot_off % 16) || !part || (D % 4) || ((uintptr_t)part % 16)))) return B200_ERR_BAD_ARG;
  const int threads = D >= 4096 ? 1024 : D >= 1024 ? 512 : 256;
  return launch_pdl(rmsnorm_kernel, dim3(T), dim3(threads), 0, st, x, g, eps, D, (int8_t*)xq, xd, xs16,
                    (__nv_bfloat16*)hb, hf, sym ? *sym : SymTable{}, sym ? sym_mode : 0, (float4*)zero, zero ? (int)(zero_n / 4) : 0,
                    slot_off, slot_rows, part);
}

// Sequence-sharded tensor-parallel prefill: this rank owns rows [row0, row0 + T) of the residual
// stream.  Normalise them and push the bf16 result into EVERY rank's full [rows][D] tensor at byte
// offset hb_off of the symmetric heap (one multimem store per 16 bytes through NVSwitch, or one store
// per peer), then bump this rank's all-gather counter: the column-parallel GEMM that follows on each
// rank starts on the rows that have arrived (see sym_wait_rows).  This is the all-gather, fused into
// the kernel that produces the data.
__global__ void __launch_bounds__(512) rmsnorm_allgather_kernel(const float* __restrict__ x, const float* __restrict__ g,
                                                                float eps, int D, int row0, int n_rows, size_t hb_off,
                                                                const __grid_constant__ SymTable sym) {
  __shared__ float red[32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  if (t >= n_rows) {              // a rank without rows still counts as having pushed (one CTA, no data)
    sym_signal_rows(sym, gridDim.x);
    return;
  }
  const float4* xr = (const float4*)(x + (size_t)(row0 + t) * D);
  const int chunks = D / 8;                       // 8 elements = 32 bytes in, 16 bytes out
  float ss = 0.f;
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
    const float4 a = xr[2 * c], b = xr[2 * c + 1];
    ss += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / (float)D + eps);
  const float4* gr = (const float4*)g;
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
    const float4 a = xr[2 * c], b = xr[2 * c + 1];                 // second read of the row: L1 / L2
    const float4 ga = g ? gr[2 * c] : make_float4(1.f, 1.f, 1.f, 1.f), gb = g ? gr[2 * c + 1] : make_float4(1.f, 1.f, 1.f, 1.f);
    uint4 o;
    __nv_bfloat162* p = (__nv_bfloat162*)&o;
    p[0] = __floats2bfloat162_rn(a.x * rstd * ga.x, a.y * rstd * ga.y);
    p[1] = __floats2bfloat162_rn(a.z * rstd * ga.z, a.w * rstd * ga.w);
    p[2] = __floats2bfloat162_rn(b.x * rstd * gb.x, b.y * rstd * gb.y);
    p[3] = __floats2bfloat162_rn(b.z * rstd * gb.z, b.w * rstd * gb.w);
    sym_st_all_v4(sym, hb_off + ((size_t)(row0 + t) * D + (size_t)c * 8) * 2, o);
  }
  sym_signal_rows(sym, gridDim.x);
}

// x: this rank's full-size fp32 residual tensor [*][D] (only rows [row0, row0 + T) are read); the bf16
// result goes to rows [row0, row0 + T) of the [*][D] tensor at heap offset hb_off on every rank.
B200_API int b200_rmsnorm_allgather(const float* x, const float* g, float eps, int row0, int T, int D, size_t hb_off,
                                    const SymTable* sym, cudaStream_t st) {
  if (!sym || (D % 8) || (hb_off % 16) || T < 0) return B200_ERR_BAD_ARG;
  return launch_pdl(rmsnorm_allgather_kernel, dim3(T > 0 ? T : 1), dim3(D >= 4096 ? 512 : 256), 0, st, x, g, eps, D, row0, T,
                    hb_off, *sym);
}

// Plain activation quantization of fp32 rows (used where no norm precedes a quantized matvec).
__global__ void quantize_x_kernel(const float* __restrict__ x, int D, int8_t* __restrict__ xq,
                                  float* __restrict__ xd, float* __restrict__ xs16) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int blk = w; blk < D / 32; blk += nw) {
    const float v = x[(size_t)t * D + blk * 32 + lane];
    quantize_block32(v, lane, xq + (size_t)t * D + blk * 32, xd + (size_t)t * (D / 32) + blk,
                     xs16 + (size_t)t * (D / 16) + blk * 2);
  }
}
B200_API int b200_quantize_x(const float* x, int T, int D, void* xq, float* xd, float* xs16, cudaStream_t st) {
  if (D % 32) return B200_ERR_BAD_ARG;
  return launch_pdl(quantize_x_kernel, dim3(T), dim3(256), 0, st, x, D, (int8_t*)xq, xd, xs16);
}

// ------------------------------------------------------------------ RoPE + paged KV write

// qkv fp32 [T][(Hq + 2 Hkv) * hd] (q heads, then k heads, then v heads).
// pos [T] absolute positions; slot [T] = physical token slot in the cache (page * page_size + offset).
// Cache layout: [page][Hkv][page_size][hd] fp16, so one (page, head) is one contiguous tile.
// q_out fp32 and/or q_out_h fp16 [T][Hq*hd] receive the rotated queries scaled by `q_scale`.
// style 0: pairs (2i, 2i+1); style 1: halves (i, i + hd/2).
// tab [tab_len][hd/2] holds (cos, sin) of pos * theta^(-2j/hd), computed once in double precision
// by b200_rope_table; positions beyond the table (or a null table) are computed here in double,
// because fast-math sine loses accuracy at angles of thousands of radians.
// One thread per (head, pair) and per pair of V elements: a decode step has one token per
// sequence, so the work is spread over grid.y instead of looping inside one block.
__global__ void rope_kv_kernel(const float* __restrict__ qkv, const int* __restrict__ pos,
                               const int* __restrict__ slot, float* __restrict__ q_out, __half* __restrict__ q_out_h,
                               __half* __restrict__ kc, __half* __restrict__ vc, int Hq, int Hkv, int hd,
                               int page_size, float theta, int style, float q_scale,
                               const float2* __restrict__ tab, int tab_len) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int row = (Hq + 2 * Hkv) * hd;
  const float* in = qkv + (size_t)t * row;
  const int half = hd >> 1;
  const int n_rot = (Hq + Hkv) * half, n_v = Hkv * half;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= n_rot + n_v) return;
  const int s = slot[t];
  const int page = s >= 0 ? s / page_size : 0, off = s >= 0 ? s % page_size : 0;
  if (i >= n_rot) {
    if (s < 0) return;
    const int e = (i - n_rot) * 2, kh = e / hd, c = e % hd;
    const float2 v = *(const float2*)(in + (Hq + Hkv) * hd + e);
    *(__half2*)(vc + (((size_t)page * Hkv + kh) * page_size + off) * hd + c) = __floats2half2_rn(v.x, v.y);
    return;
  }
  const int h = i / half, j = i % half;
  const int p = pos[t];
  float sn, cs;
  if (tab && p >= 0 && p < tab_len) {
    const float2 e = tab[(size_t)p * half + j];
    cs = e.x;
    sn = e.y;
  } else {
    const double inv = exp2(-2.0 * (double)j / (double)hd * log2((double)theta));
    double snd, csd;
    sincos((double)p * inv, &snd, &csd);
    sn = (float)snd;
    cs = (float)csd;
  }
  const int i0 = style == 0 ? 2 * j : j;
  const int i1 = style == 0 ? 2 * j + 1 : j + half;
  const float a = in[h * hd + i0], b = in[h * hd + i1];
  const float r0 = a * cs - b * sn, r1 = a * sn + b * cs;
  if (h < Hq) {
    const size_t qi = (size_t)t * Hq * hd + h * hd;
    if (q_out) {
      q_out[qi + i0] = r0 * q_scale;
      q_out[qi + i1] = r1 * q_scale;
    }
    if (q_out_h) {
      q_out_h[qi + i0] = __float2half(r0 * q_scale);
      q_out_h[qi + i1] = __float2half(r1 * q_scale);
    }
  } else if (s >= 0) {
    const int kh = h - Hq;
    __half* dst = kc + (((size_t)page * Hkv + kh) * page_size + off) * hd;
    dst[i0] = __float2half(r0);
    dst[i1] = __float2half(r1);
  }
}

__global__ void rope_table_kernel(float2* __restrict__ tab, int n_pos, int hd, float theta) {
  const int half = hd >> 1;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_pos * half) return;
  const int p = i / half, j = i % half;
  const double inv = exp2(-2.0 * (double)j / (double)hd * log2((double)theta));
  double sn, cs;
  sincos((double)p * inv, &sn, &cs);
  tab[i] = make_float2((float)cs, (float)sn);
}

// (cos, sin) table [n_pos][hd/2] for b200_rope_kv; built once per engine.
B200_API int b200_rope_table(void* tab, int n_pos, int hd, float theta, cudaStream_t st) {
  if (hd % 2 || n_pos < 1) return B200_ERR_BAD_ARG;
  const int n = n_pos * (hd / 2);
  rope_table_kernel<<<(n + 255) / 256, 256, 0, st>>>((float2*)tab, n_pos, hd, theta);
  return (int)cudaGetLastError();
}

B200_API int b200_rope_kv(const float* qkv, const int* pos, const int* slot, float* q_out, void* q_out_h, void* kc,
                          void* vc, int T, int Hq, int Hkv, int hd, int page_size, float theta,
                          int style, float q_scale, const void* tab, int tab_len, cudaStream_t st) {
  if (hd % 2) return B200_ERR_BAD_ARG;
  const int items = (Hq + 2 * Hkv) * (hd / 2);
  return launch_pdl(rope_kv_kernel, dim3(T, (items + 255) / 256), dim3(256), 0, st, qkv, pos, slot, q_out,
                    (__half*)q_out_h, (__half*)kc, (__half*)vc, Hq, Hkv, hd, page_size, theta, style, q_scale,
                    (const float2*)tab, tab_len);
}

// ------------------------------------------------------------------ SwiGLU / add / bias

// gu fp32 [T][2F] with (gate_i, up_i) in adjacent columns (the row order of the fused gate/up matrix) -> bf16 and/or
// fp32 act [T][F].  zero_after: gu is cleared behind the read, for a producer that accumulates into it with K splits.
__global__ void swiglu_kernel(float* __restrict__ gu, int F, __nv_bfloat16* __restrict__ ob, float* __restrict__ of,
                              int zero_after) {
  pdl_trigger();
  pdl_wait();
  const size_t t = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= F) return;
  float2* p = (float2*)(gu + t * 2 * F) + i;
  const float2 g = *p;
  if (zero_after) *p = make_float2(0.f, 0.f);
  const float v = silu(g.x) * g.y;
  if (ob) ob[t * F + i] = __float2bfloat16(v);
  if (of) of[t * F + i] = v;
}
B200_API int b200_swiglu(float* gu, int T, int F, void* ob, float* of, int zero_after, cudaStream_t st) {
  if ((uintptr_t)gu % 8) return B200_ERR_BAD_ARG;
  dim3 grid((F + 255) / 256, T);
  return launch_pdl(swiglu_kernel, grid, dim3(256), 0, st, gu, F, (__nv_bfloat16*)ob, of, zero_after);
}

__global__ void add_kernel(float* __restrict__ x, const float* __restrict__ y, size_t n) {
  pdl_trigger();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) x[i] += y[i];
}
B200_API int b200_add_inplace(float* x, const float* y, size_t n, cudaStream_t st) {
  return launch_pdl(add_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, x, y, n);
}

// ------------------------------------------------------------------ sampling

// Greedy arg-max over logits [T][V] with the lowest index winning ties (matches torch.argmax on
// the first maximal element).  Optional vocab_offset for a tensor-parallel shard; writes the max
// value too so shards can be merged.
// A row is split over gridDim.y blocks.  Each block folds its part into a 64-bit key
// (order-preserving float bits, then ~index so that ties go to the lowest index) with atomicMax on
// keys[t]; the block that arrives last (tickets[t]) decodes the key, writes the result and zeroes
// both words again, so the scratch needs zeroing only once, when it is allocated.
__device__ __forceinline__ unsigned long long argmax_key(float v, int i) {
  uint32_t u = __float_as_uint(v);
  u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
  return ((unsigned long long)u << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)i);
}
__global__ void __launch_bounds__(256) argmax_kernel(const float* __restrict__ logits, int V, int* __restrict__ out_id,
                                                     float* __restrict__ out_val, int vocab_offset,
                                                     unsigned long long* __restrict__ keys, int* __restrict__ tickets) {
  __shared__ unsigned long long sk[8];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const float* l = logits + (size_t)t * V;
  const int per = (V + gridDim.y - 1) / gridDim.y;
  const int lo = blockIdx.y * per, hi = min(V, lo + per);
  unsigned long long best = 0;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const unsigned long long k = argmax_key(l[i], i);
    best = k > best ? k : best;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long ok = __shfl_xor_sync(0xffffffffu, best, o);
    best = ok > best ? ok : best;
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) sk[w] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int k = 1; k < (int)(blockDim.x >> 5); k++) best = sk[k] > best ? sk[k] : best;
    if (gridDim.y > 1) {
      atomicMax(&keys[t], best);
      __threadfence();
      if (atomicAdd(&tickets[t], 1) != (int)gridDim.y - 1) return;
      __threadfence();
      best = atomicExch(&keys[t], 0ull);
      tickets[t] = 0;
    }
    uint32_t u = (uint32_t)(best >> 32);
    u = (u & 0x80000000u) ? (u & 0x7FFFFFFFu) : ~u;
    out_id[t] = (int)(0xFFFFFFFFu - (uint32_t)best) + vocab_offset;
    if (out_val) out_val[t] = __uint_as_float(u);
  }
}
// scratch: T * 16 bytes, zeroed once by the caller (T 64-bit keys, then T tickets, then padding);
// null runs one block per row.
B200_API int b200_argmax(const float* logits, int T, int V, int* out_id, float* out_val,
                         int vocab_offset, void* scratch, cudaStream_t st) {
  int chunks = 1;
  if (scratch) chunks = max(1, min(64, V / 2048));
  unsigned long long* keys = (unsigned long long*)scratch;
  int* tickets = scratch ? (int*)(keys + T) : nullptr;
  return launch_pdl(argmax_kernel, dim3(T, chunks), dim3(256), 0, st, logits, V, out_id, out_val, vocab_offset, keys,
                    tickets);
}

// Tensor-parallel arg-max merge: every rank holds, per row, the best (value, id) of its vocabulary shard.  Each
// rank stores its pairs into its slot of a [2][world][rows][2] word tensor on every rank, raises its flag, waits for
// the world flags and picks the best pair (highest value, lowest id on ties) from identical data, so all ranks
// agree.  One CTA, one launch; slot parity and sequence number work as in the slot all-reduce (sym.cuh).
__global__ void __launch_bounds__(1024) argmax_merge_kernel(int* __restrict__ out_id, const float* __restrict__ out_val, int nb,
                                                            const __grid_constant__ SymTable sym, size_t merge_off, int rows) {
  __shared__ uint32_t s_seq;
  pdl_trigger();
  pdl_wait();
  SymControl* me = sym_ctl(sym, sym.rank);
  const uint32_t seq = *(volatile uint32_t*)&me->merge_seq + 1u;
  const size_t buf = seq & 1u;
  for (int b = threadIdx.x; b < nb; b += blockDim.x) {
    const size_t off = merge_off + (((buf * sym.world + sym.rank) * rows + b) * 2) * 4;
    sym_st_all_f32(sym, off, out_val[b]);
    sym_st_all_f32(sym, off + 4, __int_as_float(out_id[b]));
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    me->merge_seq = seq;
    s_seq = seq;
    __threadfence_system();
    const size_t foff = offsetof(SymControl, flag) + 4 * (kSymMergeCh0 + sym.rank);
    if (sym.use_mc) {
      asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(sym.mc_base + foff), "r"(1u) : "memory");
    } else {
      for (int p = 0; p < sym.world; p++)
        asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(sym.base[p] + foff), "r"(1u) : "memory");
    }
  }
  if (threadIdx.x < (unsigned)sym.world) sym_wait_flag(sym, kSymMergeCh0 + threadIdx.x, seq);
  __syncthreads();
  const float* slots = (const float*)(sym.base[sym.rank] + merge_off) + buf * sym.world * rows * 2;
  for (int b = threadIdx.x; b < nb; b += blockDim.x) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int r = 0; r < sym.world; r++) {
      const float v = __ldcg(slots + ((size_t)r * rows + b) * 2);
      const int i = __float_as_int(__ldcg(slots + ((size_t)r * rows + b) * 2 + 1));
      if (v > bv || (v == bv && i < bi)) {
        bv = v;
        bi = i;
      }
    }
    if (bi != 0x7fffffff) out_id[b] = bi;
  }
}
// out_id / out_val: this rank's per-row arg-max (global ids) and maxima; on return out_id holds the global winner.
// merge_off: heap offset of [2][world][rows][2] 32-bit words; nb <= rows.
B200_API int b200_argmax_merge(int* out_id, const float* out_val, int nb, const SymTable* sym, size_t merge_off, int rows,
                               cudaStream_t st) {
  if (!sym || nb < 1 || nb > rows || (merge_off % 16)) return B200_ERR_BAD_ARG;
  return launch_pdl(argmax_merge_kernel, dim3(1), dim3(nb <= 256 ? 256 : 1024), 0, st, out_id, out_val, nb, *sym, merge_off, rows);
}

// Temperature / top-k / top-p sampling of one token per row.  One block per row.  The candidate
// set is the top-k (k <= 64) found by repeated block arg-max, which is exact and cheap for the
// small k that serving uses; top-p then trims the sorted candidates.  `u` holds one uniform random
// number per row, supplied by the host so runs are reproducible.
__global__ void sample_topk_kernel(const float* __restrict__ logits, int V, float temperature, int top_k,
                                   float top_p, const float* __restrict__ u, int* __restrict__ out_id,
                                   float* __restrict__ scratch) {
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float cand_v[64];
  __shared__ int cand_i[64];
  __shared__ int n_cand, s_stop;      // candidates found; set when no finite entry is left (NaN rows, -inf tails)
  if (threadIdx.x == 0) {
    n_cand = 0;
    s_stop = 0;
  }
  const int t = blockIdx.x;
  const float* l = logits + (size_t)t * V;
  float* mask = scratch + (size_t)t * V;  // copy we can knock entries out of
  for (int i = threadIdx.x; i < V; i += blockDim.x) mask[i] = l[i];
  __syncthreads();
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int k = 0; k < top_k; k++) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      float v = mask[i];
      if (v > best) {
        best = v;
        bi = i;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (lane == 0) {
      sv[w] = best;
      si[w] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int j = 1; j < nw; j++)
        if (sv[j] > sv[0] || (sv[j] == sv[0] && si[j] < si[0])) {
          sv[0] = sv[j];
          si[0] = si[j];
        }
      if (si[0] >= 0 && si[0] < V) {
        cand_v[k] = sv[0];
        cand_i[k] = si[0];
        n_cand = k + 1;
        mask[si[0]] = -INFINITY;
      } else {
        s_stop = 1;          // nothing comparable left: every remaining entry is -inf or NaN
      }
    }
    __syncthreads();
    if (s_stop) break;
  }
  if (threadIdx.x == 0) {
    top_k = n_cand;
    if (top_k == 0) {        // a row without a single finite logit: a defined id instead of a sentinel
      out_id[t] = 0;
      return;
    }
    const float inv_t = 1.f / fmaxf(temperature, 1e-6f);
    const float m = cand_v[0];
    float p[64];
    float z = 0.f;
    for (int k = 0; k < top_k; k++) {
      p[k] = __expf((cand_v[k] - m) * inv_t);
      z += p[k];
    }
    // top-p: keep the shortest prefix whose mass reaches top_p
    int keep = top_k;
    float acc = 0.f;
    for (int k = 0; k < top_k; k++) {
      acc += p[k] / z;
      if (acc >= top_p) {
        keep = k + 1;
        break;
      }
    }
    float z2 = 0.f;
    for (int k = 0; k < keep; k++) z2 += p[k];
    float r = u[t] * z2, c = 0.f;
    int pick = cand_i[keep - 1];
    for (int k = 0; k < keep; k++) {
      c += p[k];
      if (r < c) {
        pick = cand_i[k];
        break;
      }
    }
    out_id[t] = pick;
  }
}
B200_API int b200_sample_topk(const float* logits, int T, int V, float temperature, int top_k, float top_p,
                              const float* u, int* out_id, float* scratch, cudaStream_t st) {
  if (top_k < 1 || top_k > 64 || top_k > V) return B200_ERR_BAD_ARG;
  sample_topk_kernel<<<T, 1024, 0, st>>>(logits, V, temperature, top_k, top_p, u, out_id, scratch);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ device-side autoregression

// Turns a decode step's outputs into the next step's inputs without a host round trip: the
// sampled id becomes the next input id, position and visible length grow by one, the cache slot
// is looked up in the (pre-extended) page table, and the id is appended to a history buffer.
__global__ void decode_advance_kernel(int* __restrict__ ids, const int* __restrict__ out_ids, int* __restrict__ pos,
                                      int* __restrict__ slot, int* __restrict__ seq_lens,
                                      const int* __restrict__ page_table, int max_pages, int page_size, int B,
                                      int* __restrict__ hist, int* __restrict__ step_counter, int hist_cap) {
  pdl_trigger();
  pdl_wait();
  const int step = *step_counter;
  for (int b = threadIdx.x; b < B; b += blockDim.x) {
    const int id = out_ids[b];
    ids[b] = id;
    const int p = pos[b] + 1;
    pos[b] = p;
    seq_lens[b] = p + 1;
    const int pg = p / page_size;
    slot[b] = pg < max_pages ? page_table[(size_t)b * max_pages + pg] * page_size + p % page_size : -1;
    if (hist && step < hist_cap) hist[(size_t)step * B + b] = id;
  }
  __syncthreads();
  if (threadIdx.x == 0) *step_counter = step + 1;
}
B200_API int b200_decode_advance(int* ids, const int* out_ids, int* pos, int* slot, int* seq_lens,
                                 const int* page_table, int max_pages, int page_size, int B, int* hist,
                                 int* step_counter, int hist_cap, cudaStream_t st) {
  return launch_pdl(decode_advance_kernel, dim3(1), dim3(256), 0, st, ids, out_ids, pos, slot, seq_lens, page_table,
                    max_pages, page_size, B, hist, step_counter, hist_cap);
}

// ------------------------------------------------------------------ allocation-free sampling
// See no_alloc.h.  The scratch lives in this translation unit; host code may not use the array's
// name as a pointer (on the host it is only a stand-in for the symbol), so the device address is
// fetched once per device with cudaGetSymbolAddress and handed to the kernel as an argument.
#include <cstdio>
#include <mutex>

#include "no_alloc.h"

static __device__ __align__(256) float g_noalloc_scratch[B200_SAMPLE_NOALLOC_MAX_ELEMS];

static float* noalloc_scratch_for_current_device(cudaError_t* err) {
  static std::mutex mu;
  static float* ptr[64] = {nullptr};
  int dev = 0;
  *err = cudaGetDevice(&dev);
  if (*err != cudaSuccess) return nullptr;
  if (dev < 0 || dev >= 64) {
    *err = cudaErrorInvalidDevice;
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!ptr[dev]) {
    float* p = nullptr;
    *err = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);   // device `dev` is current here
    if (*err != cudaSuccess) return nullptr;
    ptr[dev] = p;
  }
  return ptr[dev];
}

B200_API int b200_sample_topk_noalloc(const float* logits, int T, int V, float temperature, int top_k, float top_p,
                                      const float* u, int* out_id, cudaStream_t stream) {
  if (T < 1 || V < 1 || top_k < 1 || top_k > 64 || top_k > V) return B200_NOALLOC_ERR_BAD_ARG;
  if ((unsigned long long)T * (unsigned long long)V > (unsigned long long)B200_SAMPLE_NOALLOC_MAX_ELEMS) {
    std::fprintf(stderr, "b200_sample_topk_noalloc: T*V = %llu exceeds the built-in scratch of %u floats\n",
                 (unsigned long long)T * (unsigned long long)V, (unsigned)B200_SAMPLE_NOALLOC_MAX_ELEMS);
    return B200_NOALLOC_ERR_TOO_LARGE;
  }
  cudaError_t err;
  float* scratch = noalloc_scratch_for_current_device(&err);
  if (!scratch) return (int)err;
  sample_topk_kernel<<<T, 1024, 0, stream>>>(logits, V, temperature, top_k, top_p, u, out_id, scratch);
  return (int)cudaGetLastError();
}
