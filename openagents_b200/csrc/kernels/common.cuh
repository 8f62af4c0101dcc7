// Shared device helpers for the sm_100a kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define B200_API extern "C" __attribute__((visibility("default")))

// Status codes a kernel can leave in its status word (0 = fine).  A kernel never traps: a wait that
// runs out records where it gave up and the kernel returns.
enum B200Status : int {
  B200_OK = 0,
  B200_ERR_TIMEOUT_TMA = 1,     // a TMA-fed barrier never completed
  B200_ERR_TIMEOUT_MMA = 2,     // a tensor-core commit barrier never completed
  B200_ERR_TIMEOUT_PEER = 3,    // a flag owned by another rank never arrived
  B200_ERR_TIMEOUT_EPI = 4,     // the epilogue waited too long for the accumulator
  B200_ERR_BAD_ARG = 5,
};

// Programmatic dependent launch.  A kernel launched through launch_pdl may start while the kernel
// before it in the stream is still running; it must call pdl_wait() before it reads anything an
// earlier kernel wrote and before it writes anything at all.  What comes before the wait (barrier
// and tensor-memory set-up, L2 prefetch of weights, which no kernel writes) overlaps the previous
// kernel.  pdl_trigger() lets the NEXT kernel in the stream start its own preamble.
// b200_set_pdl(0) turns the attribute off, so every launch is then fully serialised.
extern "C" int b200_pdl_enabled();
extern "C" int b200_prefetch_enabled();

namespace b200 {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Ask for `bytes` (multiple of 16) at 16-byte aligned `p` to be brought into L2; nothing waits for it.
__device__ __forceinline__ void prefetch_l2(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

template <typename... KArgs, typename... Args>
static inline int launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                             Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = b200_pdl_enabled() ? 1 : 0;
  return (int)cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ int warp_sum_i(int v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Block-wide sum for blocks of up to 1024 threads; `red` is 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : -INFINITY;
  return warp_max(t);
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  // Read-once data (weights, KV pages): do not keep it in L1.
  uint4 v;
  asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ldg_stream2(const void* p) {
  uint2 v;
  asm("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float gelu_tanh(float x) {
  const float k = 0.7978845608028654f;
  float u = k * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.f + tanhf(u));
}

// Byte slot of element i (0..7) inside each group of eight quantized activations.  The order is
// chosen so that `v & 0x0F0F0F0F` / `(v >> 4) & 0x0F0F0F0F` of a repacked 4-bit weight word line up
// with two consecutive activation words for dp4a.
__device__ __forceinline__ int x8_slot(int i) {
  // element: 0 1 2 3 4 5 6 7  ->  slot: 0 2 4 6 1 3 5 7
  return ((i & 3) << 1) | (i >> 2);
}

// Quantize 32 consecutive activations held one per lane into int8 (x8 byte order) with one fp32
// scale, and produce the scaled sums of the two 16-element halves.
//   q     : base of this 32-byte block in the int8 plane
//   d_out : scale slot; s16_out: two floats (d * sum of q over elements 0..15 and 16..31)
__device__ __forceinline__ void quantize_block32(float v, int lane, int8_t* q, float* d_out,
                                                 float* s16_out) {
  float amax = warp_max(fabsf(v));
  float d = amax * (1.f / 127.f);
  float id = d > 0.f ? 1.f / d : 0.f;
  int qi = __float2int_rn(v * id);
  q[(lane & ~7) | x8_slot(lane & 7)] = (int8_t)qi;
  int s = qi;
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  s += __shfl_xor_sync(0xffffffffu, s, 2);
  s += __shfl_xor_sync(0xffffffffu, s, 4);
  s += __shfl_xor_sync(0xffffffffu, s, 8);
  if (lane == 0) *d_out = d;
  if ((lane & 15) == 0) s16_out[lane >> 4] = d * (float)s;
}

}  // namespace b200
