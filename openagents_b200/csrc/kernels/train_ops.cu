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
__global__ void layernorm_fwd_kernel(const bf16* __restrict__ x, const float* __restrict__ g,
                                     const float* __restrict__ b, float eps, bf16* __restrict__ y,
                                     float* __restrict__ mean, float* __restrict__ rstd, int rows, int D) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const bf16* xr = x + (size_t)row * D;
  float s = 0.f, ss = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    const float2 v = __bfloat1622float2(*(const __nv_bfloat162*)(xr + i));
    s += v.x + v.y;
    ss += v.x * v.x + v.y * v.y;
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
  for (int i = lane * 2; i < D; i += 64) {
    const float2 v = __bfloat1622float2(*(const __nv_bfloat162*)(xr + i));
    *(__nv_bfloat162*)(y + (size_t)row * D + i) =
        __floats2bfloat162_rn((v.x - mu) * rs * g[i] + b[i], (v.y - mu) * rs * g[i + 1] + b[i + 1]);
  }
}
B200_API int b200_layernorm_fwd(const void* x, const float* g, const float* b, float eps, void* y, float* mean,
                                float* rstd, int rows, int D, cudaStream_t st) {
  if (D % 2) return B200_ERR_BAD_ARG;
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
  constexpr int MAXJ = 16;        // register-resident column sums cover D <= 1024
  const bool in_regs = D <= MAXJ * 64;
  float rg[MAXJ][2], rb[MAXJ][2];
#pragma unroll
  for (int j = 0; j < MAXJ; j++) rg[j][0] = rg[j][1] = rb[j][0] = rb[j][1] = 0.f;
  for (int row = blockIdx.x * nw + w; row < rows; row += gridDim.x * nw) {
    const bf16* xr = x + (size_t)row * D;
    const bf16* dr = dy + (size_t)row * D;
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int j = 0; j < MAXJ; j++) {
      const int i = lane * 2 + j * 64;
      if (i < D && in_regs) {
        const float2 xv = __bfloat1622float2(*(const __nv_bfloat162*)(xr + i));
        const float2 dv = __bfloat1622float2(*(const __nv_bfloat162*)(dr + i));
        const float h0 = (xv.x - mu) * rs, h1 = (xv.y - mu) * rs;
        const float a0 = dv.x * g[i], a1 = dv.y * g[i + 1];
        s1 += a0 + a1;
        s2 += a0 * h0 + a1 * h1;
        rg[j][0] += dv.x * h0; rg[j][1] += dv.y * h1;
        rb[j][0] += dv.x;      rb[j][1] += dv.y;
      }
    }
    if (!in_regs) {
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
      const int i = lane * 2 + j * 64;
      if (i < D) {
        atomicAdd(sg + i, rg[j][0]);
        atomicAdd(sg + i + 1, rg[j][1]);
        atomicAdd(sb + i, rb[j][0]);
        atomicAdd(sb + i + 1, rb[j][1]);
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
  if (D % 2) return B200_ERR_BAD_ARG;
  const int grid = min((rows + 7) / 8, 148 * 2);
  layernorm_bwd_kernel<<<grid, 256, 2 * D * sizeof(float), st>>>((const bf16*)dy, (const bf16*)x, g, mean, rstd,
                                                                  (bf16*)dx, dx_add, dgamma, dbeta, rows, D);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ GELU (tanh form)
__global__ void gelu_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, size_t n2) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n2) return;
  const float2 v = __bfloat1622float2(((const __nv_bfloat162*)x)[i]);
  ((__nv_bfloat162*)y)[i] = __floats2bfloat162_rn(gelu_tanh(v.x), gelu_tanh(v.y));
}
__device__ __forceinline__ float gelu_tanh_grad(float x) {
  const float k = 0.7978845608028654f;
  const float u = k * (x + 0.044715f * x * x * x);
  const float t = tanhf(u);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k * (1.f + 3.f * 0.044715f * x * x);
}
// dx = dy * gelu'(x), in place over dy.
__global__ void gelu_bwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ dy, size_t n2) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n2) return;
  const float2 v = __bfloat1622float2(((const __nv_bfloat162*)x)[i]);
  const float2 d = __bfloat1622float2(((__nv_bfloat162*)dy)[i]);
  ((__nv_bfloat162*)dy)[i] = __floats2bfloat162_rn(d.x * gelu_tanh_grad(v.x), d.y * gelu_tanh_grad(v.y));
}
B200_API int b200_gelu_fwd(const void* x, void* y, size_t n, cudaStream_t st) {
  if (n % 2) return B200_ERR_BAD_ARG;
  gelu_fwd_kernel<<<(unsigned)((n / 2 + 255) / 256), 256, 0, st>>>((const bf16*)x, (bf16*)y, n / 2);
  return (int)cudaGetLastError();
}
B200_API int b200_gelu_bwd(const void* x, void* dy, size_t n, cudaStream_t st) {
  if (n % 2) return B200_ERR_BAD_ARG;
  gelu_bwd_kernel<<<(unsigned)((n / 2 + 255) / 256), 256, 0, st>>>((const bf16*)x, (bf16*)dy, n / 2);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ bias gradient
// gb[n] += sum_m dy[m][n]; each CTA owns 64 columns and a slice of rows.
__global__ void bias_grad_kernel(const bf16* __restrict__ dy, float* __restrict__ gb, int M, int N) {
  __shared__ float part[8][64];
  const int c = blockIdx.x * 64 + (threadIdx.x & 63);
  const int r0 = threadIdx.x >> 6;   // 0..3 with 256 threads
  float s = 0.f;
  if (c < N)
    for (int m = blockIdx.y * 4 + r0; m < M; m += gridDim.y * 4) s += __bfloat162float(dy[(size_t)m * N + c]);
  part[r0][threadIdx.x & 63] = s;
  __syncthreads();
  if (r0 == 0 && c < N) atomicAdd(gb + c, part[0][threadIdx.x] + part[1][threadIdx.x] + part[2][threadIdx.x] + part[3][threadIdx.x]);
}
B200_API int b200_bias_grad(const void* dy, float* gb, int M, int N, cudaStream_t st) {
  dim3 grid((N + 63) / 64, min(64, (M + 3) / 4));
  bias_grad_kernel<<<grid, 256, 0, st>>>((const bf16*)dy, gb, M, N);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ fused cross-entropy
// logits bf16 [M][ldl] (only the first V columns are real vocabulary; the padding is ignored and
// its gradient is zero).  Per row: loss = logsumexp - logit[target]; dlogits = (softmax - onehot) *
// scale, written in place over the logits.  One CTA per row.
__global__ void ce_fused_kernel(bf16* __restrict__ logits, const int* __restrict__ targets, float* __restrict__ loss,
                                float scale, int V, int ldl) {
  __shared__ float red[32];
  const size_t row = blockIdx.x;
  bf16* l = logits + row * ldl;
  float mx = -INFINITY;
  for (int i = threadIdx.x * 2; i < V; i += blockDim.x * 2) {
    const float2 v = __bfloat1622float2(*(const __nv_bfloat162*)(l + i));
    mx = fmaxf(mx, v.x);
    if (i + 1 < V) mx = fmaxf(mx, v.y);
  }
  mx = block_max(mx, red);
  float se = 0.f;
  for (int i = threadIdx.x * 2; i < V; i += blockDim.x * 2) {
    const float2 v = __bfloat1622float2(*(const __nv_bfloat162*)(l + i));
    se += __expf(v.x - mx);
    if (i + 1 < V) se += __expf(v.y - mx);
  }
  se = block_sum(se, red);
  const int tgt = targets[row];
  const float lse = mx + __logf(se);
  if (threadIdx.x == 0) loss[row] = tgt >= 0 ? lse - __bfloat162float(l[tgt]) : 0.f;
  const float inv = 1.f / se;
  const float sc = tgt >= 0 ? scale : 0.f;   // a negative target masks the position
  for (int i = threadIdx.x * 2; i < ldl; i += blockDim.x * 2) {
    const float2 v = __bfloat1622float2(*(const __nv_bfloat162*)(l + i));
    float g0 = i < V ? (__expf(v.x - mx) * inv - (i == tgt ? 1.f : 0.f)) * sc : 0.f;
    float g1 = i + 1 < V ? (__expf(v.y - mx) * inv - (i + 1 == tgt ? 1.f : 0.f)) * sc : 0.f;
    *(__nv_bfloat162*)(l + i) = __floats2bfloat162_rn(g0, g1);
  }
}
B200_API int b200_ce_fused(void* logits, const int* targets, float* loss, float scale, int M, int V, int ldl,
                           cudaStream_t st) {
  if (ldl % 2) return B200_ERR_BAD_ARG;
  ce_fused_kernel<<<M, 512, 0, st>>>((bf16*)logits, targets, loss, scale, V, ldl);
  return (int)cudaGetLastError();
}
