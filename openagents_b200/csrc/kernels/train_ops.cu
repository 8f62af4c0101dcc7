// Training-path operators for the GPT-2-shape trainer: token+position embedding (forward and
// scatter-add backward), LayerNorm forward/backward, GELU forward/backward, bias gradients, and
// the fused softmax cross-entropy that writes the loss and dlogits in one pass.
//
// The loss follows the reference's formulation (soft-max with max subtraction, negative
// log-likelihood of the target, mean over positions:
// apps/openagents.com/workers/api/src/cs336-a1-real-gradient-workload.ts:580-595; its backward
// `p - onehot` is :609-615).
#include "common.cuh"

using namespace b200;
typedef __nv_bfloat16 bf16;

// ------------------------------------------------------------------ embedding
// x[t] = wte[id[t]] + wpe[t % T]   (bf16 tables, bf16 out)
__global__ void embed_fwd_kernel(const int* __restrict__ ids, const bf16* __restrict__ wte,
                                 const bf16* __restrict__ wpe, bf16* __restrict__ x, int T, int D) {
  const size_t t = blockIdx.x;
  const int id = ids[t];
  const int p = (int)(t % T);
  for (int i = threadIdx.x * 2; i < D; i += blockDim.x * 2) {
    const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)(wte + (size_t)id * D + i));
    const float2 b = __bfloat1622float2(*(const __nv_bfloat162*)(wpe + (size_t)p * D + i));
    *(__nv_bfloat162*)(x + t * D + i) = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
  }
}
B200_API int b200_embed_fwd(const int* ids, const void* wte, const void* wpe, void* x, int n_tok, int T, int D,
                            cudaStream_t st) {
  if (D % 2) return B200_ERR_BAD_ARG;
  embed_fwd_kernel<<<n_tok, 128, 0, st>>>(ids, (const bf16*)wte, (const bf16*)wpe, (bf16*)x, T, D);
  return (int)cudaGetLastError();
}
// gwte[id[t]] += dx[t]; gwpe[t % T] += dx[t]   (fp32 gradient buffers)
__global__ void embed_bwd_kernel(const int* __restrict__ ids, const bf16* __restrict__ dx, float* __restrict__ gwte,
                                 float* __restrict__ gwpe, int T, int D) {
  const size_t t = blockIdx.x;
  const int id = ids[t];
  const int p = (int)(t % T);
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    const float g = __bfloat162float(dx[t * D + i]);
    atomicAdd(gwte + (size_t)id * D + i, g);
    atomicAdd(gwpe + (size_t)p * D + i, g);
  }
}
B200_API int b200_embed_bwd(const int* ids, const void* dx, float* gwte, float* gwpe, int n_tok, int T, int D,
                            cudaStream_t st) {
  embed_bwd_kernel<<<n_tok, 256, 0, st>>>(ids, (const bf16*)dx, gwte, gwpe, T, D);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ LayerNorm
// One warp per row.  Saves mean and rstd for the backward pass.
// 16-byte loads and stores: eight bf16 per lane per step, a warp per row; the row stays in registers between the
// statistics pass and the output pass when it is at most 1024 wide.
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = (const __nv_bfloat162*)&u;
#pragma unroll
  for (int k = 0; k < 4; k++) {
    const float2 v = __bfloat1622float2(h[k]);
    f[2 * k] = v.x;
    f[2 * k + 1] = v.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* h = (__nv_bfloat162*)&u;
#pragma unroll
  for (int k = 0; k < 4; k++) h[k] = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
  return u;
}

__global__ void layernorm_fwd_kernel(const bf16* __restrict__ x, const float* __restrict__ g,
                                     const float* __restrict__ b, float eps, bf16* __restrict__ y,
                                     float* __restrict__ mean, float* __restrict__ rstd, int rows, int D) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const bf16* xr = x + (size_t)row * D;
  constexpr int MAXJ = 4;                      // register-resident rows: D <= 1024
  const bool in_regs = D <= MAXJ * 256;
  uint4 keep[MAXJ];
  float s = 0.f, ss = 0.f;
#pragma unroll
  for (int j = 0; j < MAXJ; j++) {
    const int i = lane * 8 + j * 256;
    if (i < D && in_regs) {
      keep[j] = *(const uint4*)(xr + i);
      float f[8];
      unpack8(keep[j], f);
#pragma unroll
      for (int k = 0; k < 8; k++) { s += f[k]; ss += f[k] * f[k]; }
    }
  }
  if (!in_regs)
    for (int i = lane * 8; i < D; i += 256) {
      float f[8];
      unpack8(*(const uint4*)(xr + i), f);
#pragma unroll
      for (int k = 0; k < 8; k++) { s += f[k]; ss += f[k] * f[k]; }
    }
  s = warp_sum(s);
  ss = warp_sum(ss);
  const float mu = s / D;
  const float var = fmaxf(ss / D - mu * mu, 0.f);
  const float rs = rsqrtf(var + eps);
  if (lane == 0) {
    mean[row] = mu;
    rstd[row] = rs;
  }
  auto emit = [&](int i, const uint4& u) {
    float f[8], o[8];
    unpack8(u, f);
    const float4 g0 = *(const float4*)(g + i), g1 = *(const float4*)(g + i + 4);
    const float4 b0 = *(const float4*)(b + i), b1 = *(const float4*)(b + i + 4);
    const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
    const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
    for (int k = 0; k < 8; k++) o[k] = (f[k] - mu) * rs * gg[k] + bb[k];
    *(uint4*)(y + (size_t)row * D + i) = pack8(o);
  };
  if (in_regs) {
#pragma unroll
    for (int j = 0; j < MAXJ; j++) {
      const int i = lane * 8 + j * 256;
      if (i < D) emit(i, keep[j]);
    }
  } else {
    for (int i = lane * 8; i < D; i += 256) emit(i, *(const uint4*)(xr + i));
  }
}
B200_API int b200_layernorm_fwd(const void* x, const float* g, const float* b, float eps, void* y, float* mean,
                                float* rstd, int rows, int D, cudaStream_t st) {
  if (D % 8) return B200_ERR_BAD_ARG;
  layernorm_fwd_kernel<<<(rows + 7) / 8, 256, 0, st>>>((const bf16*)x, g, b, eps, (bf16*)y, mean, rstd, rows, D);
  return (int)cudaGetLastError();
}

// dx = rstd * (dy*g - mean(dy*g) - xhat * mean(dy*g*xhat)); dgamma += dy*xhat; dbeta += dy.
// Each CTA walks rows with a grid stride, keeps its gamma/beta partial sums in shared memory and
// adds them to the fp32 gradients once at the end.  `dx_add`: accumulate into dx (residual branch).
__global__ void layernorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                     const float* __restrict__ g, const float* __restrict__ mean,
                                     const float* __restrict__ rstd, bf16* __restrict__ dx, int dx_add,
                                     float* __restrict__ dgamma, float* __restrict__ dbeta, int rows, int D) {
  extern __shared__ float sm[];   // [2][D]
  float* sg = sm;
  float* sb = sm + D;
  for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) sm[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  constexpr int MAXJ = 4;         // register-resident rows and column sums cover D <= 1024
  const bool in_regs = D <= MAXJ * 256;
  float rg[MAXJ][8], rb[MAXJ][8];
#pragma unroll
  for (int j = 0; j < MAXJ; j++)
#pragma unroll
    for (int k = 0; k < 8; k++) rg[j][k] = rb[j][k] = 0.f;
  for (int row = blockIdx.x * nw + w; row < rows; row += gridDim.x * nw) {
    const bf16* xr = x + (size_t)row * D;
    const bf16* dr = dy + (size_t)row * D;
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
    if (in_regs) {
      uint4 kx[MAXJ], kd[MAXJ];
#pragma unroll
      for (int j = 0; j < MAXJ; j++) {
        const int i = lane * 8 + j * 256;
        if (i < D) {
          kx[j] = *(const uint4*)(xr + i);
          kd[j] = *(const uint4*)(dr + i);
        }
      }
#pragma unroll
      for (int j = 0; j < MAXJ; j++) {
        const int i = lane * 8 + j * 256;
        if (i < D) {
          float xv[8], dv[8];
          unpack8(kx[j], xv);
          unpack8(kd[j], dv);
          const float4 g0 = *(const float4*)(g + i), g1 = *(const float4*)(g + i + 4);
          const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
          for (int k = 0; k < 8; k++) {
            const float h = (xv[k] - mu) * rs, a = dv[k] * gg[k];
            s1 += a;
            s2 += a * h;
            rg[j][k] += dv[k] * h;
            rb[j][k] += dv[k];
          }
        }
      }
      s1 = warp_sum(s1) / D;
      s2 = warp_sum(s2) / D;
#pragma unroll
      for (int j = 0; j < MAXJ; j++) {
        const int i = lane * 8 + j * 256;
        if (i < D) {
          float xv[8], dv[8], o[8];
          unpack8(kx[j], xv);
          unpack8(kd[j], dv);
          const float4 g0 = *(const float4*)(g + i), g1 = *(const float4*)(g + i + 4);
          const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
          for (int k = 0; k < 8; k++) o[k] = rs * (dv[k] * gg[k] - s1 - (xv[k] - mu) * rs * s2);
          uint4* dst = (uint4*)(dx + (size_t)row * D + i);
          if (dx_add) {
            float p[8];
            unpack8(*dst, p);
#pragma unroll
            for (int k = 0; k < 8; k++) o[k] += p[k];
          }
          *dst = pack8(o);
        }
      }
      continue;
    }
    for (int i = lane * 2; i < D; i += 64) {
      const float2 xv = __bfloat1622float2(*(const __nv_bfloat162*)(xr + i));
      const float2 dv = __bfloat1622float2(*(const __nv_bfloat162*)(dr + i));
      const float h0 = (xv.x - mu) * rs, h1 = (xv.y - mu) * rs;
      const float a0 = dv.x * g[i], a1 = dv.y * g[i + 1];
      s1 += a0 + a1;
      s2 += a0 * h0 + a1 * h1;
      atomicAdd(sg + i, dv.x * h0);
      atomicAdd(sg + i + 1, dv.y * h1);
      atomicAdd(sb + i, dv.x);
      atomicAdd(sb + i + 1, dv.y);
    }
    s1 = warp_sum(s1) / D;
    s2 = warp_sum(s2) / D;
    for (int i = lane * 2; i < D; i += 64) {
      const float2 xv = __bfloat1622float2(*(const __nv_bfloat162*)(xr + i));
      const float2 dv = __bfloat1622float2(*(const __nv_bfloat162*)(dr + i));
      const float h0 = (xv.x - mu) * rs, h1 = (xv.y - mu) * rs;
      float o0 = rs * (dv.x * g[i] - s1 - h0 * s2), o1 = rs * (dv.y * g[i + 1] - s1 - h1 * s2);
      __nv_bfloat162* dst = (__nv_bfloat162*)(dx + (size_t)row * D + i);
      if (dx_add) {
        const float2 p = __bfloat1622float2(*dst);
        o0 += p.x;
        o1 += p.y;
      }
      *dst = __floats2bfloat162_rn(o0, o1);
    }
  }
  if (in_regs) {
#pragma unroll
    for (int j = 0; j < MAXJ; j++) {
      const int i = lane * 8 + j * 256;
      if (i < D) {
#pragma unroll
        for (int k = 0; k < 8; k++) {
          atomicAdd(sg + i + k, rg[j][k]);
          atomicAdd(sb + i + k, rb[j][k]);
        }
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    atomicAdd(dgamma + i, sg[i]);
    atomicAdd(dbeta + i, sb[i]);
  }
}
B200_API int b200_layernorm_bwd(const void* dy, const void* x, const float* g, const float* mean, const float* rstd,
                                void* dx, int dx_add, float* dgamma, float* dbeta, int rows, int D,
                                cudaStream_t st) {
  if (D % 8) return B200_ERR_BAD_ARG;
  const int grid = min((rows + 7) / 8, 148);      // 158 registers x 256 threads: one CTA per SM
  layernorm_bwd_kernel<<<grid, 256, 2 * D * sizeof(float), st>>>((const bf16*)dy, (const bf16*)x, g, mean, rstd,
                                                                  (bf16*)dx, dx_add, dgamma, dbeta, rows, D);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ GELU (tanh form)
__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float k = 0.7978845608028654f;
  const float u = k * (x + 0.044715f * x * x * x);
  const float t = tanhf(u);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k * (1.f + 3.f * 0.044715f * x * x);
}
// Eight elements (16 bytes) per thread per step, grid-stride.
__global__ void gelu_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, size_t n8) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float f[8];
    unpack8(((const uint4*)x)[i], f);
#pragma unroll
    for (int k = 0; k < 8; k++) f[k] = gelu_tanh(f[k]);
    ((uint4*)y)[i] = pack8(f);
  }
}
// dx = dy * gelu'(x), in place over dy.
__global__ void gelu_bwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ dy, size_t n8) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    float f[8], d[8];
    unpack8(((const uint4*)x)[i], f);
    unpack8(((const uint4*)dy)[i], d);
#pragma unroll
    for (int k = 0; k < 8; k++) d[k] *= gelu_tanh_grad(f[k]);
    ((uint4*)dy)[i] = pack8(d);
  }
}
static unsigned ew_grid(size_t n8) { return (unsigned)min((size_t)148 * 16, (n8 + 255) / 256); }
B200_API int b200_gelu_fwd(const void* x, void* y, size_t n, cudaStream_t st) {
  if (n % 8) return B200_ERR_BAD_ARG;
  gelu_fwd_kernel<<<ew_grid(n / 8), 256, 0, st>>>((const bf16*)x, (bf16*)y, n / 8);
  return (int)cudaGetLastError();
}
B200_API int b200_gelu_bwd(const void* x, void* dy, size_t n, cudaStream_t st) {
  if (n % 8) return B200_ERR_BAD_ARG;
  gelu_bwd_kernel<<<ew_grid(n / 8), 256, 0, st>>>((const bf16*)x, (bf16*)dy, n / 8);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ bias gradient
// gb[n] += sum_m dy[m][n].  A CTA owns 256 columns (a warp reads 512 contiguous bytes of a row) and a slice of rows;
// each thread sums eight columns over its rows, the eight row lanes meet in shared memory, one atomic per column.
__global__ void bias_grad_kernel(const bf16* __restrict__ dy, float* __restrict__ gb, int M, int N) {
  __shared__ float part[8][256];
  const int cg = threadIdx.x & 31, r0 = threadIdx.x >> 5;          // column group of 8, row lane
  const int c = blockIdx.x * 256 + cg * 8;
  float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (c < N) {
    const int stride = gridDim.y * 8;
    int m = blockIdx.y * 8 + r0;
    for (; m + stride < M; m += 2 * stride) {                      // two rows in flight per thread
      const uint4 u0 = *(const uint4*)(dy + (size_t)m * N + c);
      const uint4 u1 = *(const uint4*)(dy + (size_t)(m + stride) * N + c);
      float f[8], h[8];
      unpack8(u0, f);
      unpack8(u1, h);
#pragma unroll
      for (int k = 0; k < 8; k++) s[k] += f[k] + h[k];
    }
    for (; m < M; m += stride) {
      float f[8];
      unpack8(*(const uint4*)(dy + (size_t)m * N + c), f);
#pragma unroll
      for (int k = 0; k < 8; k++) s[k] += f[k];
    }
  }
#pragma unroll
  for (int k = 0; k < 8; k++) part[r0][cg * 8 + k] = s[k];
  __syncthreads();
  const int col = blockIdx.x * 256 + threadIdx.x;
  if (col < N) {
    float t = 0.f;
#pragma unroll
    for (int r = 0; r < 8; r++) t += part[r][threadIdx.x];
    atomicAdd(gb + col, t);
  }
}
B200_API int b200_bias_grad(const void* dy, float* gb, int M, int N, cudaStream_t st) {
  if (N % 8) return B200_ERR_BAD_ARG;
  const int cb = (N + 255) / 256;
  int gy = (148 * 4 + cb - 1) / cb;                 // about four CTAs per SM in total
  gy = max(1, min(gy, (M + 7) / 8));
  bias_grad_kernel<<<dim3(cb, gy), 256, 0, st>>>((const bf16*)dy, gb, M, N);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ fused cross-entropy
// logits bf16 [M][ldl] (only the first V columns are real vocabulary; the padding is ignored and
// its gradient is zero).  Per row: loss = logsumexp - logit[target]; dlogits = (softmax - onehot) *
// scale, written in place over the logits.  One CTA per row; 16-byte accesses; maximum and sum in ONE pass
// (running maximum per thread, rescaled sums), so a row is read twice and written once.
// row_scale (optional): one factor per row that replaces `scale` (preference optimisation weights every sequence's rows by
// a signed coefficient).  write_grad = 0 stops after the loss: the logits stay as they are, so the caller can derive the
// row factors from the losses and call again.
__global__ void __launch_bounds__(512) ce_fused_kernel(bf16* __restrict__ logits, const int* __restrict__ targets, float* __restrict__ loss,
                                                       float scale, const float* __restrict__ row_scale, int write_grad, int V, int ldl) {
  __shared__ float red[32];
  const size_t row = blockIdx.x;
  bf16* l = logits + row * ldl;
  float mx = -INFINITY, se = 0.f;
  for (int i = threadIdx.x * 8; i < ldl; i += blockDim.x * 8) {
    float f[8];
    unpack8(*(const uint4*)(l + i), f);
    float cm = -INFINITY;
#pragma unroll
    for (int k = 0; k < 8; k++) {
      if (i + k >= V) f[k] = -INFINITY;
      cm = fmaxf(cm, f[k]);
    }
    if (cm > mx) {
      se *= __expf(mx - cm);             // exp(-inf) = 0 on the first chunk
      mx = cm;
    }
    if (mx > -INFINITY) {
#pragma unroll
      for (int k = 0; k < 8; k++) se += __expf(f[k] - mx);
    }
  }
  const float gmx = block_max(mx, red);
  se = block_sum(mx > -INFINITY ? se * __expf(mx - gmx) : 0.f, red);
  const int tgt = targets[row];
  const float lse = gmx + __logf(se);
  if (threadIdx.x == 0) loss[row] = tgt >= 0 ? lse - __bfloat162float(l[tgt]) : 0.f;
  if (!write_grad) return;
  __syncthreads();                       // the target logit is read before anyone overwrites it
  const float inv = 1.f / se;
  const float sc = tgt >= 0 ? (row_scale ? row_scale[row] : scale) : 0.f;   // a negative target masks the position
  for (int i = threadIdx.x * 8; i < ldl; i += blockDim.x * 8) {
    float f[8];
    unpack8(*(const uint4*)(l + i), f);
#pragma unroll
    for (int k = 0; k < 8; k++)
      f[k] = i + k < V ? (__expf(f[k] - gmx) * inv - (i + k == tgt ? 1.f : 0.f)) * sc : 0.f;
    *(uint4*)(l + i) = pack8(f);
  }
}
B200_API int b200_ce_fused(void* logits, const int* targets, float* loss, float scale, int M, int V, int ldl,
                           cudaStream_t st) {
  if (ldl % 8) return B200_ERR_BAD_ARG;
  ce_fused_kernel<<<M, 512, 0, st>>>((bf16*)logits, targets, loss, scale, nullptr, 1, V, ldl);
  return (int)cudaGetLastError();
}
B200_API int b200_ce_fused_rows(void* logits, const int* targets, float* loss, const float* row_scale, int write_grad, int M, int V, int ldl,
                                cudaStream_t st) {
  if (ldl % 8 || (write_grad && !row_scale)) return B200_ERR_BAD_ARG;
  ce_fused_kernel<<<M, 512, 0, st>>>((bf16*)logits, targets, loss, 0.f, row_scale, write_grad, V, ldl);
  return (int)cudaGetLastError();
}
