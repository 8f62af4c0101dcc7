// Mixture-of-experts routing fused with the expert-parallel dispatch.
//
// One CTA per token: router logits (an [E][d] fp32 mat-vec against the normalised hidden row), top-k,
// softmax over the selected k (the gpt-oss convention), and then, for each selected expert, the row is
// written straight into the receive buffer of the rank that owns the expert: a slot is claimed with
// one atomic on the owner's counter and the 16-byte stores go over NVLink peer memory (or stay local).
// There is no separate gather, no send buffer and no all-to-all launch; the kernel ends with the
// cross-rank barrier, after which every rank's receive buffers and counters are final and the grouped
// GEMM (gemm_tc05.cu, group mode) can run on them.
//
// The reference names this topology only: Psionic's `sparse_expert` placement with "explicit expert
// ranges and a stable placement digest" (docs/teardowns/2026-07-21-buzz-teardown.md:676-679); the
// routing math is the top-k softmax router of the CPU oracle in this package.
#include "../comm/sym.cuh"

using namespace b200;

constexpr int kMoeMaxExperts = 256;
constexpr int kMoeMaxTopK = 8;

struct MoeDispatchArgs {
  const __nv_bfloat16* h;     // [T][d] normalised hidden rows of this rank's tokens (what the experts multiply)
  const float* hf;            // [T][d] the same rows in fp32 (what the router sees), or null: use h
  const float* wr;            // [E][d] router weights, fp32: a top-k decision should not hinge on bf16 rounding
  const float* br;            // [E] router bias or null
  int T, d, E, top_k, E_local, C;
  // Byte offsets in every rank's symmetric heap:
  size_t recv_x_off;          // bf16 [E_local][C][d]
  size_t recv_meta_off;       // int32 [E_local][C][2] = (source rank, source token)
  size_t recv_w_off;          // fp32 [E_local][C] gate weight
  size_t counts_off;          // int32 [E_local] rows claimed so far (zero before the layer starts)
  int* topk_ids;              // optional [T][top_k] (this rank), for tests and telemetry
  float* topk_w;              // optional [T][top_k]
  int* status;
  SymTable sym;
};

__global__ void __launch_bounds__(256) moe_route_dispatch_kernel(const MoeDispatchArgs a) {
  __shared__ float s_logit[kMoeMaxExperts];
  __shared__ int s_sel[kMoeMaxTopK];
  __shared__ float s_w[kMoeMaxTopK];
  __shared__ int s_slot[kMoeMaxTopK];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const __nv_bfloat16* hr = a.h + (size_t)t * a.d;

  // Router logits: warp w takes experts w, w + 8, ... FOUR at a time (the hidden row is read once per group and four
  // weight rows stream beside it, so a warp has five independent loads in flight per step instead of two).
  const float* hfr = a.hf ? a.hf + (size_t)t * a.d : nullptr;
  for (int e0 = w; e0 < a.E; e0 += 32) {
    const float* wr[4];
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 4; j++) wr[j] = a.wr + (size_t)min(e0 + 8 * j, a.E - 1) * a.d;
#pragma unroll 2
    for (int i = lane * 2; i < a.d; i += 64) {
      const float2 x = hfr ? *(const float2*)(hfr + i) : __bfloat1622float2(*(const __nv_bfloat162*)(hr + i));
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float2 y = *(const float2*)(wr[j] + i);
        acc[j] += x.x * y.x + x.y * y.y;
      }
    }
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float v = warp_sum(acc[j]);
      const int e = e0 + 8 * j;
      if (lane == 0 && e < a.E) s_logit[e] = v + (a.br ? a.br[e] : 0.f);
    }
  }
  __syncthreads();

  if (w == 0) {
    // top-k by repeated arg-max over the warp (lowest index wins ties), softmax over the k winners, then lane k claims
    // a row in its expert's receive buffer: the k remote atomics are in flight together instead of one after another
    float mine[(kMoeMaxExperts + 31) / 32];
#pragma unroll
    for (int j = 0; j < (kMoeMaxExperts + 31) / 32; j++) mine[j] = lane + 32 * j < a.E ? s_logit[lane + 32 * j] : -INFINITY;
    float my_val = 0.f;
    int my_sel = 0;
    float mx = 0.f, sum = 0.f;
    for (int k = 0; k < a.top_k; k++) {
      float best = -INFINITY;
      int bi = 0x7fffffff;
#pragma unroll
      for (int j = 0; j < (kMoeMaxExperts + 31) / 32; j++)
        if (mine[j] > best) { best = mine[j]; bi = lane + 32 * j; }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      if (bi == 0x7fffffff) bi = 0;              // a row without a finite logit
      if (k == 0) mx = best;
      const float ex = __expf(best - mx);
      sum += ex;
      if (lane == k) { my_val = ex; my_sel = bi; }
#pragma unroll
      for (int j = 0; j < (kMoeMaxExperts + 31) / 32; j++)
        if (lane + 32 * j == bi) mine[j] = -INFINITY;
    }
    if (lane < a.top_k) {
      const int k = lane;
      const float wgt = my_val / sum;
      s_sel[k] = my_sel;
      s_w[k] = wgt;
      if (a.topk_ids) a.topk_ids[(size_t)t * a.top_k + k] = my_sel;
      if (a.topk_w) a.topk_w[(size_t)t * a.top_k + k] = wgt;
      const int owner = my_sel / a.E_local, el = my_sel % a.E_local;
      unsigned slot;
      asm volatile("atom.relaxed.sys.global.add.u32 %0, [%1], %2;" : "=r"(slot)
                   : "l"(a.sym.base[owner] + a.counts_off + (size_t)el * 4), "r"(1u) : "memory");
      if ((int)slot >= a.C) {       // cannot happen when C covers every token of every rank; never write past it
        if (a.status) atomicExch(a.status, (int)B200_ERR_BAD_ARG);
        s_slot[k] = -1;
      } else {
        s_slot[k] = (int)slot;
        char* base = a.sym.base[owner];
        int* meta = (int*)(base + a.recv_meta_off) + ((size_t)el * a.C + slot) * 2;
        asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1,%2};" ::"l"(meta), "r"(a.sym.rank), "r"(t) : "memory");
        asm volatile("st.relaxed.sys.global.f32 [%0], %1;" ::"l"((float*)(base + a.recv_w_off) + (size_t)el * a.C + slot),
                     "f"(wgt) : "memory");
      }
    }
  }
  __syncthreads();

  // Copy the row to each owner, 16 bytes per thread per step (d * 2 bytes is a multiple of 16).
  const int n16 = a.d / 8;
  const uint4* src = (const uint4*)hr;
  for (int k = 0; k < a.top_k; k++) {
    if (s_slot[k] < 0) continue;
    const int owner = s_sel[k] / a.E_local, el = s_sel[k] % a.E_local;
    char* dst = a.sym.base[owner] + a.recv_x_off + ((size_t)el * a.C + s_slot[k]) * (size_t)a.d * 2;
    for (int i = tid; i < n16; i += 256) {
      const uint4 v = src[i];
      asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst + (size_t)i * 16), "r"(v.x), "r"(v.y),
                   "r"(v.z), "r"(v.w) : "memory");
    }
  }
  sym_kernel_end_barrier(a.sym, 3, gridDim.x);
}

// Zero a small int array (the expert counters of the other layer parity) on this rank.
__global__ void moe_zero_kernel(int* p, int n) {
  pdl_trigger();
  pdl_wait();
  for (int i = threadIdx.x; i < n; i += blockDim.x) p[i] = 0;
}

B200_API int b200_moe_route_dispatch(const void* h, const float* hf, const float* wr, const float* br, int T, int d, int E, int top_k,
                                     int E_local, int C, size_t recv_x_off, size_t recv_meta_off, size_t recv_w_off,
                                     size_t counts_off, int* topk_ids, float* topk_w, const SymTable* sym, int* status,
                                     cudaStream_t st) {
  if (!sym || T < 1 || E < 1 || E > kMoeMaxExperts || top_k < 1 || top_k > kMoeMaxTopK || top_k > E || (d % 8) ||
      E_local < 1 || (E % E_local) || E / E_local != sym->world || (recv_x_off % 16) || (recv_meta_off % 8))
    return B200_ERR_BAD_ARG;
  MoeDispatchArgs a;
  a.h = (const __nv_bfloat16*)h; a.hf = hf; a.wr = wr; a.br = br; a.T = T; a.d = d; a.E = E; a.top_k = top_k;
  a.E_local = E_local; a.C = C; a.recv_x_off = recv_x_off; a.recv_meta_off = recv_meta_off; a.recv_w_off = recv_w_off;
  a.counts_off = counts_off; a.topk_ids = topk_ids; a.topk_w = topk_w; a.status = status; a.sym = *sym;
  return launch_pdl(moe_route_dispatch_kernel, dim3(T), dim3(256), 0, st, a);
}

B200_API int b200_moe_zero(int* p, int n, cudaStream_t st) {
  return launch_pdl(moe_zero_kernel, dim3(1), dim3(256), 0, st, p, n);
}
