// Sharded (ZeRO-1/2 style) AdamW fused with its collectives.
//
//   zero_reduce_norm   : gradient reduce-scatter fused with the averaging and the squared-norm
//                        partial: each rank pulls its shard of every rank's fp32 gradient buffer
//                        (multimem.ld_reduce through the switch, or peer loads), scales by 1/world,
//                        keeps the result locally and accumulates sum(g^2).
//   zero_adamw_gather  : clip + AdamW on the fp32 master shard, cast to bf16, and the parameter
//                        all-gather: the updated bf16 shard is stored straight into every rank's
//                        parameter buffer (multimem.st / peer stores); the kernel ends with the
//                        cross-rank barrier, so on completion every rank holds the new parameters.
//
// The update rule is the data-parallel mean followed by one optimizer step, as in the reference's
// aggregation (cs336-a1-real-gradient-workload.ts:872-891, plain SGD there); the clip uses the
// global L2 norm (:846-850 computes the same norm).
#include "sym.cuh"

using namespace b200;

// grads: fp32 [n_total] at grad_off in every heap.  This rank owns [lo, lo + n).  n % 4 == 0.
__global__ void zero_reduce_norm_kernel(const __grid_constant__ SymTable T, size_t grad_off, size_t lo, size_t n,
                                        float* __restrict__ gshard, float* __restrict__ norm2_out) {
  __shared__ float red[32];
  const float inv = 1.f / (float)T.world;
  float acc = 0.f;
  const size_t n4 = n / 4;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    float4 g = sym_ld_reduce_f32x4(T, grad_off + (lo + i * 4) * 4);
    g.x *= inv; g.y *= inv; g.z *= inv; g.w *= inv;
    ((float4*)gshard)[i] = g;
    acc += g.x * g.x + g.y * g.y + g.z * g.z + g.w * g.w;
  }
  acc = block_sum(acc, red);
  if (threadIdx.x == 0) atomicAdd(norm2_out, acc);
  sym_kernel_end_barrier(T, 3, gridDim.x);   // nobody may overwrite its gradients before all have read
}
B200_API int b200_zero_reduce_norm(const SymTable* T, size_t grad_off, size_t lo, size_t n, float* gshard,
                                   float* norm2_out, cudaStream_t st) {
  if (n % 4 || (grad_off % 16) || (lo % 4)) return B200_ERR_BAD_ARG;
  int grid = (int)min((size_t)148 * 4, (n / 4 + 255) / 256);
  if (grid < 1) grid = 1;
  zero_reduce_norm_kernel<<<grid, 256, 0, st>>>(*T, grad_off, lo, n, gshard, norm2_out);
  return (int)cudaGetLastError();
}

struct AdamArgs {
  float lr, beta1, beta2, eps, wd, bc1, bc2, max_norm;   // bc = 1 - beta^t
  size_t decay_end;   // global element index below which weight decay applies
};

// norm2: sum over ALL ranks of the shard squared norms (fp32 scalar, device memory).
__global__ void zero_adamw_gather_kernel(const __grid_constant__ SymTable T, size_t param_off, size_t lo, size_t n,
                                         const float* __restrict__ gshard, float* __restrict__ master,
                                         float* __restrict__ m, float* __restrict__ v,
                                         const float* __restrict__ norm2, const AdamArgs a) {
  const float gn = sqrtf(*norm2);
  const float clip = a.max_norm > 0.f ? fminf(1.f, a.max_norm / (gn + 1e-6f)) : 1.f;
  const size_t n8 = n / 8;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    uint4 packed;
    __nv_bfloat162* pb = (__nv_bfloat162*)&packed;
    float w8[8];
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const size_t k = i * 8 + h * 4;
      const float4 g4 = *(const float4*)(gshard + k);
      float4 m4 = *(const float4*)(m + k), v4 = *(const float4*)(v + k), w4 = *(const float4*)(master + k);
      const float gg[4] = {g4.x * clip, g4.y * clip, g4.z * clip, g4.w * clip};
      float mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w}, ww[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
      for (int e = 0; e < 4; e++) {
        mm[e] = a.beta1 * mm[e] + (1.f - a.beta1) * gg[e];
        vv[e] = a.beta2 * vv[e] + (1.f - a.beta2) * gg[e] * gg[e];
        const float mh = mm[e] / a.bc1, vh = vv[e] / a.bc2;
        const float decay = (lo + k + e) < a.decay_end ? a.wd : 0.f;
        ww[e] -= a.lr * (mh / (sqrtf(vh) + a.eps) + decay * ww[e]);
        w8[h * 4 + e] = ww[e];
      }
      *(float4*)(m + k) = make_float4(mm[0], mm[1], mm[2], mm[3]);
      *(float4*)(v + k) = make_float4(vv[0], vv[1], vv[2], vv[3]);
      *(float4*)(master + k) = make_float4(ww[0], ww[1], ww[2], ww[3]);
    }
#pragma unroll
    for (int e = 0; e < 4; e++) pb[e] = __floats2bfloat162_rn(w8[2 * e], w8[2 * e + 1]);
    sym_st_all_v4(T, param_off + (lo + i * 8) * 2, packed);
  }
  sym_kernel_end_barrier(T, 3, gridDim.x);
}
B200_API int b200_zero_adamw_gather(const SymTable* T, size_t param_off, size_t lo, size_t n, const float* gshard,
                                    float* master, float* m, float* v, const float* norm2, float lr, float beta1,
                                    float beta2, float eps, float wd, float bc1, float bc2, float max_norm,
                                    size_t decay_end, cudaStream_t st) {
  if (n % 8 || (param_off % 16) || (lo % 8)) return B200_ERR_BAD_ARG;
  AdamArgs a{lr, beta1, beta2, eps, wd, bc1, bc2, max_norm, decay_end};
  int grid = (int)min((size_t)148 * 4, (n / 8 + 255) / 256);
  if (grid < 1) grid = 1;
  zero_adamw_gather_kernel<<<grid, 256, 0, st>>>(*T, param_off, lo, n, gshard, master, m, v, norm2, a);
  return (int)cudaGetLastError();
}
