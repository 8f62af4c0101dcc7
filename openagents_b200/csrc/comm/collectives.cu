// Stand-alone collectives over the symmetric heap, issued from kernels: barrier, all-reduce,
// all-gather, reduce-scatter and all-to-all.  All of them address buffers by byte offset into the
// heap (the same offset on every rank).  They are the building blocks and the test vehicles for the
// fused compute+collective kernels; NCCL stays the bootstrap and the measured baseline.
//
// Contract shared by every kernel here: the inputs of all ranks are complete when the kernel
// starts (the previous kernel on each rank ended with a barrier, or `b200_sym_barrier` ran), and
// when the kernel completes its outputs are complete on every rank.
#include "sym.cuh"

using namespace b200;

__global__ void sym_barrier_kernel(const __grid_constant__ SymTable T, int ch) {
  if (threadIdx.x == 0) sym_barrier_thread(T, ch);
}
B200_API int b200_sym_barrier(const SymTable* T, int ch, cudaStream_t st) {
  sym_barrier_kernel<<<1, 32, 0, st>>>(*T, ch);
  return (int)cudaGetLastError();
}

// In-place all-reduce (sum) of n fp32 values at `off`: rank r sums slice r over all ranks and
// broadcasts it.  n must be a multiple of 4.
__global__ void sym_all_reduce_kernel(const __grid_constant__ SymTable T, size_t off, size_t n, int ch) {
  const size_t n4 = n / 4;
  const size_t per = (n4 + T.world - 1) / T.world;
  const size_t lo = per * T.rank, hi = min(n4, lo + per);
  for (size_t i = lo + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < hi; i += (size_t)gridDim.x * blockDim.x) {
    const float4 s = sym_ld_reduce_f32x4(T, off + i * 16);
    sym_st_all_v4(T, off + i * 16, make_uint4(__float_as_uint(s.x), __float_as_uint(s.y), __float_as_uint(s.z),
                                              __float_as_uint(s.w)));
  }
  sym_kernel_end_barrier(T, ch, gridDim.x);
}
B200_API int b200_sym_all_reduce_f32(const SymTable* T, size_t off, size_t n, int ch, cudaStream_t st) {
  if (n % 4 || off % 16) return B200_ERR_BAD_ARG;
  const size_t per = (n / 4 + T->world - 1) / T->world;
  int grid = (int)min((size_t)148, (per + 255) / 256);
  if (grid < 1) grid = 1;
  sym_all_reduce_kernel<<<grid, 256, 0, st>>>(*T, off, n, ch);
  return (int)cudaGetLastError();
}

// All-gather: every rank's `bytes` at src_off land at dst_off + rank * bytes on every rank.
__global__ void sym_all_gather_kernel(const __grid_constant__ SymTable T, size_t src_off, size_t dst_off, size_t bytes, int ch) {
  const uint4* src = (const uint4*)(T.base[T.rank] + src_off);
  const size_t n = bytes / 16;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    sym_st_all_v4(T, dst_off + (size_t)T.rank * bytes + i * 16, src[i]);
  sym_kernel_end_barrier(T, ch, gridDim.x);
}
B200_API int b200_sym_all_gather(const SymTable* T, size_t src_off, size_t dst_off, size_t bytes, int ch,
                                 cudaStream_t st) {
  if (bytes % 16 || src_off % 16 || dst_off % 16) return B200_ERR_BAD_ARG;
  int grid = (int)min((size_t)148, (bytes / 16 + 255) / 256);
  if (grid < 1) grid = 1;
  sym_all_gather_kernel<<<grid, 256, 0, st>>>(*T, src_off, dst_off, bytes, ch);
  return (int)cudaGetLastError();
}

// Reduce-scatter (sum): out[i] on rank r = sum over ranks p of in_p[r * n + i], fp32, n per rank.
__global__ void sym_reduce_scatter_kernel(const __grid_constant__ SymTable T, size_t in_off, size_t out_off, size_t n, int ch) {
  float4* out = (float4*)(T.base[T.rank] + out_off);
  const size_t n4 = n / 4;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x)
    out[i] = sym_ld_reduce_f32x4(T, in_off + ((size_t)T.rank * n4 + i) * 16);
  sym_kernel_end_barrier(T, ch, gridDim.x);
}
B200_API int b200_sym_reduce_scatter_f32(const SymTable* T, size_t in_off, size_t out_off, size_t n, int ch,
                                         cudaStream_t st) {
  if (n % 4 || in_off % 16 || out_off % 16) return B200_ERR_BAD_ARG;
  int grid = (int)min((size_t)148, (n / 4 + 255) / 256);
  if (grid < 1) grid = 1;
  sym_reduce_scatter_kernel<<<grid, 256, 0, st>>>(*T, in_off, out_off, n, ch);
  return (int)cudaGetLastError();
}

// All-to-all: chunk p (bytes) of this rank's source goes to dst_off + rank * bytes on rank p: one
// direct peer write per destination, every peer being one hop through the switch.
__global__ void sym_all_to_all_kernel(const __grid_constant__ SymTable T, size_t src_off, size_t dst_off, size_t bytes, int ch) {
  const size_t n = bytes / 16;
  for (int p = 0; p < T.world; p++) {
    const int dst = (T.rank + p) % T.world;   // stagger destinations across ranks
    const uint4* src = (const uint4*)(T.base[T.rank] + src_off + (size_t)dst * bytes);
    uint4* out = (uint4*)(T.base[dst] + dst_off + (size_t)T.rank * bytes);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
      out[i] = src[i];
  }
  sym_kernel_end_barrier(T, ch, gridDim.x);
}
B200_API int b200_sym_all_to_all(const SymTable* T, size_t src_off, size_t dst_off, size_t bytes, int ch,
                                 cudaStream_t st) {
  if (bytes % 16 || src_off % 16 || dst_off % 16) return B200_ERR_BAD_ARG;
  int grid = (int)min((size_t)148, (bytes / 16 + 255) / 256);
  if (grid < 1) grid = 1;
  sym_all_to_all_kernel<<<grid, 256, 0, st>>>(*T, src_off, dst_off, bytes, ch);
  return (int)cudaGetLastError();
}

// A wait on a flag nothing sets: exercises the timeout path on one GPU without involving a peer.
// The kernel returns after `wait_ns`, records the status in the control block and leaves the
// context usable.
__global__ void sym_wait_unset_flag_kernel(const __grid_constant__ SymTable T, int ch) {
  if (threadIdx.x == 0) {
    SymTable solo = T;
    solo.world = 2;            // expects two arrivals, only this rank will ever arrive
    solo.use_mc = 0;
    solo.base[1] = solo.base[0];
    solo.rank = 0;
    // Arrive once (on ourselves via base[0]) but not twice: target stays out of reach.
    SymControl* me = sym_ctl(solo, 0);
    const int e = me->epoch[ch];
    const uint32_t target = 2u * (uint32_t)(e + 1) + 1000000u;
    const unsigned long long t0 = sym_now_ns();
    bool ok = true;
    for (uint32_t spin = 0;; ++spin) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(&me->flag[ch]) : "memory");
      if ((int32_t)(v - target) >= 0) break;
      if ((spin & 63u) == 63u && sym_now_ns() - t0 > T.wait_ns) {
        ok = false;
        break;
      }
    }
    if (!ok) {
      me->status = (int)B200_ERR_TIMEOUT_PEER;
      atomicAdd(&me->timeouts, 1);
    }
  }
}
B200_API int b200_sym_wait_unset_flag(const SymTable* T, int ch, cudaStream_t st) {
  sym_wait_unset_flag_kernel<<<1, 32, 0, st>>>(*T, ch);
  return (int)cudaGetLastError();
}
