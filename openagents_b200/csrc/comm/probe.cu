// Bandwidth probes: the roofline inputs the framework reports against.
//   stream triad   a[i] = b[i] + s * c[i] over fp32 arrays larger than L2 (the device benchmark's memory
//                  case: apps/openagents.com/workers/api/src/cs336-a2-device-benchmark.ts:193-210)
//   peer copy      this rank reads (pull) or writes (push) a block of a peer's symmetric heap with plain
//                  16-byte loads / stores over NVLink, or writes every replica at once with multimem.st
// Timing is done by the caller with CUDA events; nothing here waits on another rank.
#include "sym.cuh"

using namespace b200;

namespace {

__global__ void __launch_bounds__(256) stream_triad_kernel(float4* __restrict__ a, const float4* __restrict__ b,
                                                           const float4* __restrict__ c, float s, size_t n4) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    const float4 x = b[i], y = c[i];
    a[i] = make_float4(x.x + s * y.x, x.y + s * y.y, x.z + s * y.z, x.w + s * y.w);
  }
}

// mode 0: pull (load from peer, store locally); 1: push (load locally, store to peer);
// 2: broadcast push (load locally, one multimem store reaches every replica; needs multicast)
__global__ void __launch_bounds__(256) peer_copy_kernel(const __grid_constant__ SymTable T, int peer, size_t src_off, size_t dst_off,
                                                        size_t n16, int mode) {
  const char* src = (mode == 0 ? T.base[peer] : T.base[T.rank]) + src_off;
  char* dst = (mode == 1 ? T.base[peer] : T.base[T.rank]) + dst_off;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(src + i * 16) : "memory");
    if (mode == 2) sym_st_all_v4(T, dst_off + i * 16, v);
    else asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst + i * 16), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
  }
}

}  // namespace

B200_API int b200_stream_triad(float* a, const float* b, const float* c, float s, size_t n, cudaStream_t st) {
  if (n % 4 || ((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) % 16) return B200_ERR_BAD_ARG;
  stream_triad_kernel<<<148 * 8, 256, 0, st>>>((float4*)a, (const float4*)b, (const float4*)c, s, n / 4);
  return (int)cudaGetLastError();
}

B200_API int b200_sym_peer_copy(const SymTable* T, int peer, size_t src_off, size_t dst_off, size_t bytes, int mode,
                                cudaStream_t st) {
  if (!T || peer < 0 || peer >= T->world || bytes % 16 || src_off % 16 || dst_off % 16 || mode < 0 || mode > 2) return B200_ERR_BAD_ARG;
  if (mode == 2 && !T->use_mc) return B200_ERR_BAD_ARG;
  peer_copy_kernel<<<148 * 4, 256, 0, st>>>(*T, peer, src_off, dst_off, bytes / 16, mode);
  return (int)cudaGetLastError();
}
