// Integer verification kernels over a prime field (p < 2^31): the arithmetic of the Freivalds check that training
// verification runs on a claimed matrix product: A (B r) == C r (mod p), and, when the exact product is demanded, A B == C.
// Every entry is an exact residue, so the results are bit-identical to the host arithmetic whatever the launch shape.
#include <cstdint>

#include "common.cuh"

namespace {

__device__ __forceinline__ uint32_t mulmod(uint32_t a, uint32_t b, uint32_t p) {
  return (uint32_t)(((unsigned long long)a * b) % p);
}

// y[i] = sum_j A[i][j] x[j] mod p.  One warp per row: every product is reduced first, so a lane's 64-bit sum cannot
// overflow for any row length that fits an int.
__global__ void modp_matvec_kernel(const uint32_t* __restrict__ A, const uint32_t* __restrict__ x, uint32_t* __restrict__ y,
                                   int rows, int cols, uint32_t p) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const uint32_t* a = A + (size_t)warp * cols;
  unsigned long long acc = 0;
  for (int j = lane; j < cols; j += 32) acc += mulmod(a[j], x[j], p);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
  if (lane == 0) y[warp] = (uint32_t)(acc % p);
}

// C = A B mod p with 16 x 16 shared-memory tiles.
constexpr int TILE = 16;
__global__ void modp_matmul_kernel(const uint32_t* __restrict__ A, const uint32_t* __restrict__ B, uint32_t* __restrict__ C,
                                   int n, int k, int m, uint32_t p) {
  __shared__ uint32_t sa[TILE][TILE], sb[TILE][TILE + 1];
  const int row = blockIdx.y * TILE + threadIdx.y, col = blockIdx.x * TILE + threadIdx.x;
  unsigned long long acc = 0;
  for (int t = 0; t < k; t += TILE) {
    sa[threadIdx.y][threadIdx.x] = (row < n && t + threadIdx.x < k) ? A[(size_t)row * k + t + threadIdx.x] : 0u;
    sb[threadIdx.y][threadIdx.x] = (col < m && t + threadIdx.y < k) ? B[(size_t)(t + threadIdx.y) * m + col] : 0u;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < TILE; i++) acc += mulmod(sa[threadIdx.y][i], sb[i][threadIdx.x], p);
    __syncthreads();
  }
  if (row < n && col < m) C[(size_t)row * m + col] = (uint32_t)(acc % p);
}

// mismatch[0] = number of positions where a != b
__global__ void count_mismatch_kernel(const uint32_t* __restrict__ a, const uint32_t* __restrict__ b, size_t n, int* __restrict__ mismatch) {
  int local = 0;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) local += a[i] != b[i];
  if (local) atomicAdd(mismatch, local);
}

}  // namespace

B200_API int b200_modp_matvec(const void* A, const void* x, void* y, int rows, int cols, unsigned p, cudaStream_t st) {
  if (rows <= 0 || cols <= 0 || p < 2 || p > 0x7fffffffu) return B200_ERR_BAD_ARG;
  const int warps_per_block = 8;
  modp_matvec_kernel<<<(rows + warps_per_block - 1) / warps_per_block, warps_per_block * 32, 0, st>>>(
      (const uint32_t*)A, (const uint32_t*)x, (uint32_t*)y, rows, cols, p);
  return (int)cudaGetLastError();
}
B200_API int b200_modp_matmul(const void* A, const void* B, void* C, int n, int k, int m, unsigned p, cudaStream_t st) {
  if (n <= 0 || k <= 0 || m <= 0 || p < 2 || p > 0x7fffffffu) return B200_ERR_BAD_ARG;
  modp_matmul_kernel<<<dim3((m + TILE - 1) / TILE, (n + TILE - 1) / TILE), dim3(TILE, TILE), 0, st>>>(
      (const uint32_t*)A, (const uint32_t*)B, (uint32_t*)C, n, k, m, p);
  return (int)cudaGetLastError();
}
B200_API int b200_count_mismatch(const void* a, const void* b, size_t n, int* mismatch, cudaStream_t st) {
  if (n == 0) return 0;
  const int blocks = (int)((n + 255) / 256 < 592 ? (n + 255) / 256 : 592);
  count_mismatch_kernel<<<blocks, 256, 0, st>>>((const uint32_t*)a, (const uint32_t*)b, n, mismatch);
  return (int)cudaGetLastError();
}
