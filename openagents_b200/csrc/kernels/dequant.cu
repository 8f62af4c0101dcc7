// Expansion of the engine's packed weight layouts (Q4_K-R, Q6_K-R, Q8_0-R, MXFP4-R) to bf16
// [N][K] row-major.  Used where a weight feeds the dense tensor-core GEMM (prefill, training
// export) and as the GPU-side check of the repacked layouts against the CPU dequantizer.
#include "common.cuh"

using namespace b200;

enum { WT_Q4KR = 0, WT_Q6KR = 1, WT_Q8R = 2, WT_BF16 = 3, WT_MXFP4R = 4 };

// One thread expands one 8-element word.
__global__ void dequant_kernel(int wt, const uint8_t* __restrict__ w, const uint8_t* __restrict__ w2,
                               __nv_bfloat16* __restrict__ out, size_t n_words, int K) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_words) return;
  const size_t e0 = i * 8;                 // first element (row-major over [N][K])
  const size_t row = e0 / K;
  const int k = (int)(e0 - row * K);
  float v[8];
  if (wt == WT_Q4KR) {
    const int nsb = K / 256, sb = k >> 8, word = (k & 255) >> 3, j = word >> 2;
    const uint8_t* blk = w + (row * nsb + sb) * 144;
    const uint4 hdr = *(const uint4*)blk;
    const uint32_t q = ((const uint32_t*)(blk + 16))[word];
    const int sh = 8 * (j & 3);
    const uint32_t b0 = (hdr.y >> sh) & 0xFF, b1 = (hdr.z >> sh) & 0xFF, b2 = (hdr.w >> sh) & 0xFF;
    const uint32_t sc = j < 4 ? (b0 & 63) : ((b2 & 0xF) | ((b0 >> 6) << 4));
    const uint32_t mn = j < 4 ? (b1 & 63) : ((b2 >> 4) | ((b1 >> 6) << 4));
    const __half2 dd = *reinterpret_cast<const __half2*>(&hdr.x);
    const float a = __low2float(dd) * (float)sc, m = __high2float(dd) * (float)mn;
#pragma unroll
    for (int e = 0; e < 8; e++) v[e] = a * (float)((q >> (4 * (e >> 1) + 16 * (e & 1))) & 0xF) - m;
  } else if (wt == WT_Q6KR) {
    const int nsb = K / 256, sb = k >> 8, word = (k & 255) >> 3;
    const uint8_t* blk = w + (row * nsb + sb) * 208;
    const uint32_t lo = ((const uint32_t*)blk)[word];
    const uint32_t tw = ((const uint32_t*)(blk + 128))[word >> 1];
    const float d = __half2float(((const __half*)w2)[row * nsb + sb]);
    const float sc = d * (float)((const int8_t*)(blk + 192))[(k & 255) >> 4];
#pragma unroll
    for (int e = 0; e < 8; e++) {
      const int nib = (lo >> (4 * (e >> 1) + 16 * (e & 1))) & 0xF;
      const int slot = x8_slot(e);
      const int hi = (tw >> (8 * (slot & 3) + 2 * (slot >> 2) + 4 * (word & 1))) & 3;
      v[e] = sc * (float)((nib | (hi << 4)) - 32);
    }
  } else if (wt == WT_Q8R) {
    const int8_t* q = (const int8_t*)w + e0;
    const float d = __half2float(((const __half*)w2)[e0 >> 5]);
#pragma unroll
    for (int e = 0; e < 8; e++) v[e] = d * (float)q[x8_slot(e)];
  } else {  // WT_MXFP4R: nibble plane in Q4_K-R word order + E8M0 plane
    const uint32_t q = ((const uint32_t*)w)[i];
    const float s = exp2f((float)w2[e0 >> 5] - 127.f);
#pragma unroll
    for (int e = 0; e < 8; e++) {
      const int c = (q >> (4 * (e >> 1) + 16 * (e & 1))) & 0xF;
      const int mag = c & 7;
      const float f = mag < 2 ? 0.5f * mag : (mag < 4 ? 1.f + 0.5f * (mag - 2) : (mag < 6 ? 2.f + (mag - 4) : (mag == 6 ? 4.f : 6.f)));
      v[e] = (c & 8) ? -s * f : s * f;
    }
  }
  uint4 o;
  __nv_bfloat162* p = (__nv_bfloat162*)&o;
#pragma unroll
  for (int e = 0; e < 4; e++) p[e] = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
  *(uint4*)(out + e0) = o;
}

B200_API int b200_dequant_bf16(int wt, const void* w, const void* w2, void* out, size_t N, int K, cudaStream_t st) {
  if (K % 32) return B200_ERR_BAD_ARG;
  if ((wt == WT_Q4KR || wt == WT_Q6KR) && K % 256) return B200_ERR_BAD_ARG;
  const size_t n_words = N * (size_t)K / 8;
  dequant_kernel<<<(unsigned)((n_words + 255) / 256), 256, 0, st>>>(wt, (const uint8_t*)w, (const uint8_t*)w2,
                                                                     (__nv_bfloat16*)out, n_words, K);
  return (int)cudaGetLastError();
}

// fp32 -> bf16 and bf16 transpose helpers used around the dense GEMM.
__global__ void f32_to_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y, size_t n) {
  const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i + 3 < n) {
    const float4 v = *(const float4*)(x + i);
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 o;
    o.x = *(uint32_t*)&a;
    o.y = *(uint32_t*)&b;
    *(uint2*)(y + i) = o;
  } else {
    for (size_t j = i; j < n; j++) y[j] = __float2bfloat16(x[j]);
  }
}
B200_API int b200_f32_to_bf16(const float* x, void* y, size_t n, cudaStream_t st) {
  const size_t nt = (n + 3) / 4;
  f32_to_bf16_kernel<<<(unsigned)((nt + 255) / 256), 256, 0, st>>>(x, (__nv_bfloat16*)y, n);
  return (int)cudaGetLastError();
}

// out[c][r] = in[r][c] for a bf16 matrix [R][C]; 32x32 tiles through shared memory.
__global__ void transpose_bf16_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, int R, int C) {
  __shared__ __nv_bfloat16 tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int r = r0 + i, c = c0 + threadIdx.x;
    tile[i][threadIdx.x] = (r < R && c < C) ? in[(size_t)r * C + c] : __float2bfloat16(0.f);
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int c = c0 + i, r = r0 + threadIdx.x;
    if (r < R && c < C) out[(size_t)c * R + r] = tile[threadIdx.x][i];
  }
}
B200_API int b200_transpose_bf16(const void* in, void* out, int R, int C, cudaStream_t st) {
  dim3 grid((C + 31) / 32, (R + 31) / 32), block(32, 8);
  transpose_bf16_kernel<<<grid, block, 0, st>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, R, C);
  return (int)cudaGetLastError();
}
