// CPU dequantizers and quantizers for the GGUF block formats.  These are the oracle for every
// GPU dequant path and the packer used when a model is saved.
#include "quant.h"

#include <algorithm>
#include <cmath>
#include <cstring>

namespace b200 {

static const TypeTraits kTraits[] = {
    {GGML_F32, "F32", 1, 4},         {GGML_F16, "F16", 1, 2},
    {GGML_BF16, "BF16", 1, 2},       {GGML_Q8_0, "Q8_0", 32, 34},
    {GGML_Q4_K, "Q4_K", 256, 144},   {GGML_Q5_K, "Q5_K", 256, 176},
    {GGML_Q6_K, "Q6_K", 256, 210},   {GGML_MXFP4, "MXFP4", 32, 17},
};

const TypeTraits* type_traits(uint32_t type) {
  for (const auto& t : kTraits)
    if (t.type == type) return &t;
  return nullptr;
}

size_t tensor_bytes(uint32_t type, uint64_t n) {
  const TypeTraits* t = type_traits(type);
  if (!t || n % t->block_elems) return 0;
  return (size_t)(n / t->block_elems) * t->block_bytes;
}

uint16_t f32_to_f16(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  int32_t exp = (int32_t)((x >> 23) & 0xFF) - 127 + 15;
  uint32_t man = x & 0x7FFFFFu;
  if (((x >> 23) & 0xFF) == 0xFF) return (uint16_t)(sign | 0x7C00u | (man ? 0x200u : 0));
  if (exp >= 31) return (uint16_t)(sign | 0x7C00u);
  if (exp <= 0) {
    if (exp < -10) return (uint16_t)sign;
    man |= 0x800000u;
    int shift = 14 - exp;
    uint32_t half = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1);
    uint32_t mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1))) half++;
    return (uint16_t)(sign | half);
  }
  uint32_t half = ((uint32_t)exp << 10) | (man >> 13);
  uint32_t rem = man & 0x1FFFu;
  if (rem > 0x1000u || (rem == 0x1000u && (half & 1))) half++;
  return (uint16_t)(sign | half);
}

float f16_to_f32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1F;
  uint32_t man = h & 0x3FFu;
  uint32_t x;
  if (exp == 0) {
    if (man == 0) {
      x = sign;
    } else {
      int e = -1;
      do {
        man <<= 1;
        e++;
      } while (!(man & 0x400u));
      man &= 0x3FFu;
      x = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    x = sign | 0x7F800000u | (man << 13);
  } else {
    x = sign | ((exp - 15 + 127) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &x, 4);
  return f;
}

uint16_t f32_to_bf16(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x40u);
  x += 0x7FFFu + ((x >> 16) & 1);
  return (uint16_t)(x >> 16);
}

float bf16_to_f32(uint16_t h) {
  uint32_t x = (uint32_t)h << 16;
  float f;
  std::memcpy(&f, &x, 4);
  return f;
}

static const float kE2M1[16] = {0.f,  0.5f,  1.f,  1.5f,  2.f,  3.f,  4.f,  6.f,
                                -0.f, -0.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

float e2m1_value(uint8_t code) { return kE2M1[code & 15]; }

float e8m0_value(uint8_t e) {
  // 2^(e-127); e == 0 is 2^-127 (a subnormal in fp32), e == 255 is NaN in the MX spec.
  if (e == 255) return NAN;
  return std::ldexp(1.0f, (int)e - 127);
}

// ---------------------------------------------------------------- dequantize

static void dq_q8_0(const BlockQ8_0* b, float* y, uint64_t nb) {
  for (uint64_t i = 0; i < nb; i++) {
    float d = f16_to_f32(b[i].d);
    for (int j = 0; j < 32; j++) y[i * 32 + j] = d * b[i].qs[j];
  }
}

static void dq_q4_k(const BlockQ4K* b, float* y, uint64_t nb) {
  for (uint64_t i = 0; i < nb; i++) {
    const uint8_t* q = b[i].qs;
    float d = f16_to_f32(b[i].d), dmin = f16_to_f32(b[i].dmin);
    float* o = y + i * 256;
    for (int g = 0; g < 4; g++) {
      uint8_t sc, mn;
      unpack_scale_min_k4(2 * g, b[i].scales, &sc, &mn);
      float d1 = d * sc, m1 = dmin * mn;
      unpack_scale_min_k4(2 * g + 1, b[i].scales, &sc, &mn);
      float d2 = d * sc, m2 = dmin * mn;
      for (int l = 0; l < 32; l++) o[l] = d1 * (q[l] & 0xF) - m1;
      for (int l = 0; l < 32; l++) o[32 + l] = d2 * (q[l] >> 4) - m2;
      q += 32;
      o += 64;
    }
  }
}

static void dq_q5_k(const BlockQ5K* b, float* y, uint64_t nb) {
  for (uint64_t i = 0; i < nb; i++) {
    const uint8_t* ql = b[i].qs;
    const uint8_t* qh = b[i].qh;
    float d = f16_to_f32(b[i].d), dmin = f16_to_f32(b[i].dmin);
    float* o = y + i * 256;
    uint8_t u1 = 1, u2 = 2;
    for (int g = 0; g < 4; g++) {
      uint8_t sc, mn;
      unpack_scale_min_k4(2 * g, b[i].scales, &sc, &mn);
      float d1 = d * sc, m1 = dmin * mn;
      unpack_scale_min_k4(2 * g + 1, b[i].scales, &sc, &mn);
      float d2 = d * sc, m2 = dmin * mn;
      for (int l = 0; l < 32; l++) o[l] = d1 * ((ql[l] & 0xF) + ((qh[l] & u1) ? 16 : 0)) - m1;
      for (int l = 0; l < 32; l++) o[32 + l] = d2 * ((ql[l] >> 4) + ((qh[l] & u2) ? 16 : 0)) - m2;
      ql += 32;
      o += 64;
      u1 <<= 2;
      u2 <<= 2;
    }
  }
}

static void dq_q6_k(const BlockQ6K* b, float* y, uint64_t nb) {
  for (uint64_t i = 0; i < nb; i++) {
    float d = f16_to_f32(b[i].d);
    const uint8_t* ql = b[i].ql;
    const uint8_t* qh = b[i].qh;
    const int8_t* sc = b[i].scales;
    float* o = y + i * 256;
    for (int half = 0; half < 2; half++) {
      for (int l = 0; l < 32; l++) {
        int is = l / 16;
        int q1 = (int)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
        int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
        int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
        int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
        o[l] = d * sc[is] * q1;
        o[l + 32] = d * sc[is + 2] * q2;
        o[l + 64] = d * sc[is + 4] * q3;
        o[l + 96] = d * sc[is + 6] * q4;
      }
      o += 128;
      ql += 64;
      qh += 32;
      sc += 8;
    }
  }
}

static void dq_mxfp4(const BlockMXFP4* b, float* y, uint64_t nb) {
  for (uint64_t i = 0; i < nb; i++) {
    float s = e8m0_value(b[i].e);
    for (int j = 0; j < 16; j++) {
      y[i * 32 + j] = s * kE2M1[b[i].qs[j] & 0xF];
      y[i * 32 + j + 16] = s * kE2M1[b[i].qs[j] >> 4];
    }
  }
}

int dequantize(uint32_t type, const void* src, float* dst, uint64_t n) {
  const TypeTraits* t = type_traits(type);
  if (!t || n % t->block_elems) return -1;
  uint64_t nb = n / t->block_elems;
  switch (type) {
    case GGML_F32:
      std::memcpy(dst, src, n * 4);
      return 0;
    case GGML_F16:
      for (uint64_t i = 0; i < n; i++) dst[i] = f16_to_f32(((const uint16_t*)src)[i]);
      return 0;
    case GGML_BF16:
      for (uint64_t i = 0; i < n; i++) dst[i] = bf16_to_f32(((const uint16_t*)src)[i]);
      return 0;
    case GGML_Q8_0:
      dq_q8_0((const BlockQ8_0*)src, dst, nb);
      return 0;
    case GGML_Q4_K:
      dq_q4_k((const BlockQ4K*)src, dst, nb);
      return 0;
    case GGML_Q5_K:
      dq_q5_k((const BlockQ5K*)src, dst, nb);
      return 0;
    case GGML_Q6_K:
      dq_q6_k((const BlockQ6K*)src, dst, nb);
      return 0;
    case GGML_MXFP4:
      dq_mxfp4((const BlockMXFP4*)src, dst, nb);
      return 0;
  }
  return -1;
}

// ---------------------------------------------------------------- quantize

static inline int nearest_int(float v) { return (int)std::lrintf(v); }

static void q_q8_0(const float* x, BlockQ8_0* b, uint64_t nb) {
  for (uint64_t i = 0; i < nb; i++) {
    float amax = 0.f;
    for (int j = 0; j < 32; j++) amax = std::max(amax, std::fabs(x[i * 32 + j]));
    float d = amax / 127.f;
    // The stored scale is the fp16 rounding of d; quantize against what the reader will see.
    b[i].d = f32_to_f16(d);
    float dr = f16_to_f32(b[i].d);
    float id = dr > 0.f ? 1.f / dr : 0.f;
    for (int j = 0; j < 32; j++)
      b[i].qs[j] = (int8_t)std::max(-127, std::min(127, nearest_int(x[i * 32 + j] * id)));
  }
}

// Pack eight six-bit scales and mins into the 12-byte Q4_K / Q5_K field.
static void pack_scale_min_k4(const uint8_t* ls, const uint8_t* lm, uint8_t* q) {
  std::memset(q, 0, 12);
  for (int j = 0; j < 8; j++) {
    if (j < 4) {
      q[j] |= ls[j] & 63;
      q[j + 4] |= lm[j] & 63;
    } else {
      q[j + 4] = (ls[j] & 0xF) | ((lm[j] & 0xF) << 4);
      q[j - 4] |= (ls[j] >> 4) << 6;
      q[j] |= (lm[j] >> 4) << 6;
    }
  }
}

// Shared by Q4_K (nmax 15) and Q5_K (nmax 31): affine sub-blocks x ~ a*q - m with m >= 0.
static void kquant_scales(const float* x, int nmax, float* d_out, float* dmin_out, uint8_t* ls,
                          uint8_t* lm) {
  float scales[8], mins[8];
  float max_scale = 0.f, max_min = 0.f;
  for (int j = 0; j < 8; j++) {
    float lo = x[j * 32], hi = x[j * 32];
    for (int l = 1; l < 32; l++) {
      lo = std::min(lo, x[j * 32 + l]);
      hi = std::max(hi, x[j * 32 + l]);
    }
    if (lo > 0.f) lo = 0.f;
    if (hi < lo) hi = lo;
    scales[j] = (hi - lo) / nmax;
    mins[j] = -lo;
    max_scale = std::max(max_scale, scales[j]);
    max_min = std::max(max_min, mins[j]);
  }
  float d = f16_to_f32(f32_to_f16(max_scale / 63.f));
  float dmin = f16_to_f32(f32_to_f16(max_min / 63.f));
  for (int j = 0; j < 8; j++) {
    ls[j] = (uint8_t)std::min(63, std::max(0, d > 0.f ? nearest_int(scales[j] / d) : 0));
    lm[j] = (uint8_t)std::min(63, std::max(0, dmin > 0.f ? nearest_int(mins[j] / dmin) : 0));
  }
  *d_out = d;
  *dmin_out = dmin;
}

static void q_q4_k(const float* x, BlockQ4K* b, uint64_t nb) {
  for (uint64_t i = 0; i < nb; i++) {
    const float* xb = x + i * 256;
    float d, dmin;
    uint8_t ls[8], lm[8], L[256];
    kquant_scales(xb, 15, &d, &dmin, ls, lm);
    b[i].d = f32_to_f16(d);
    b[i].dmin = f32_to_f16(dmin);
    pack_scale_min_k4(ls, lm, b[i].scales);
    for (int j = 0; j < 8; j++) {
      float a = d * ls[j], m = dmin * lm[j];
      for (int l = 0; l < 32; l++) {
        int q = a > 0.f ? nearest_int((xb[j * 32 + l] + m) / a) : 0;
        L[j * 32 + l] = (uint8_t)std::max(0, std::min(15, q));
      }
    }
    uint8_t* q = b[i].qs;
    for (int g = 0; g < 4; g++) {
      for (int l = 0; l < 32; l++) q[l] = L[g * 64 + l] | (L[g * 64 + 32 + l] << 4);
      q += 32;
    }
  }
}

static void q_q5_k(const float* x, BlockQ5K* b, uint64_t nb) {
  for (uint64_t i = 0; i < nb; i++) {
    const float* xb = x + i * 256;
    float d, dmin;
    uint8_t ls[8], lm[8], L[256];
    kquant_scales(xb, 31, &d, &dmin, ls, lm);
    b[i].d = f32_to_f16(d);
    b[i].dmin = f32_to_f16(dmin);
    pack_scale_min_k4(ls, lm, b[i].scales);
    for (int j = 0; j < 8; j++) {
      float a = d * ls[j], m = dmin * lm[j];
      for (int l = 0; l < 32; l++) {
        int q = a > 0.f ? nearest_int((xb[j * 32 + l] + m) / a) : 0;
        L[j * 32 + l] = (uint8_t)std::max(0, std::min(31, q));
      }
    }
    std::memset(b[i].qh, 0, 32);
    uint8_t* ql = b[i].qs;
    uint8_t m1 = 1, m2 = 2;
    for (int g = 0; g < 4; g++) {
      for (int l = 0; l < 32; l++) {
        uint8_t l1 = L[g * 64 + l], l2 = L[g * 64 + 32 + l];
        if (l1 > 15) {
          l1 -= 16;
          b[i].qh[l] |= m1;
        }
        if (l2 > 15) {
          l2 -= 16;
          b[i].qh[l] |= m2;
        }
        ql[l] = l1 | (l2 << 4);
      }
      ql += 32;
      m1 <<= 2;
      m2 <<= 2;
    }
  }
}

static void q_q6_k(const float* x, BlockQ6K* b, uint64_t nb) {
  for (uint64_t i = 0; i < nb; i++) {
    const float* xb = x + i * 256;
    float scales[16];
    float max_scale = 0.f;
    for (int j = 0; j < 16; j++) {
      float amax = 0.f;
      for (int l = 0; l < 16; l++) amax = std::max(amax, std::fabs(xb[j * 16 + l]));
      scales[j] = amax / 31.f;
      max_scale = std::max(max_scale, scales[j]);
    }
    float d = f16_to_f32(f32_to_f16(max_scale / 127.f));
    b[i].d = f32_to_f16(d);
    uint8_t L[256];
    for (int j = 0; j < 16; j++) {
      int s = d > 0.f ? std::min(127, std::max(0, nearest_int(scales[j] / d))) : 0;
      b[i].scales[j] = (int8_t)s;
      float a = d * s;
      for (int l = 0; l < 16; l++) {
        int q = a > 0.f ? nearest_int(xb[j * 16 + l] / a) : 0;
        L[j * 16 + l] = (uint8_t)(std::max(-32, std::min(31, q)) + 32);
      }
    }
    uint8_t* ql = b[i].ql;
    uint8_t* qh = b[i].qh;
    for (int half = 0; half < 2; half++) {
      const uint8_t* Lh = L + half * 128;
      for (int l = 0; l < 32; l++) {
        uint8_t q1 = Lh[l], q2 = Lh[l + 32], q3 = Lh[l + 64], q4 = Lh[l + 96];
        ql[l] = (q1 & 0xF) | ((q3 & 0xF) << 4);
        ql[l + 32] = (q2 & 0xF) | ((q4 & 0xF) << 4);
        qh[l] = (q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6);
      }
      ql += 64;
      qh += 32;
    }
  }
}

static uint8_t nearest_e2m1(float v) {
  uint8_t sign = v < 0.f ? 8 : 0;
  float a = std::fabs(v);
  // Midpoints between consecutive magnitudes; ties go to the even mantissa.
  uint8_t code;
  if (a < 0.25f) code = 0;
  else if (a == 0.25f) code = 0;
  else if (a < 0.75f) code = 1;
  else if (a == 0.75f) code = 2;
  else if (a < 1.25f) code = 2;
  else if (a == 1.25f) code = 2;
  else if (a < 1.75f) code = 3;
  else if (a == 1.75f) code = 4;
  else if (a < 2.5f) code = 4;
  else if (a == 2.5f) code = 4;
  else if (a < 3.5f) code = 5;
  else if (a == 3.5f) code = 6;
  else if (a < 5.0f) code = 6;
  else if (a == 5.0f) code = 6;
  else code = 7;
  return sign | code;
}

static void q_mxfp4(const float* x, BlockMXFP4* b, uint64_t nb) {
  for (uint64_t i = 0; i < nb; i++) {
    float amax = 0.f;
    for (int j = 0; j < 32; j++) amax = std::max(amax, std::fabs(x[i * 32 + j]));
    int e = 0;
    if (amax > 0.f) {
      int ex;
      std::frexp(amax, &ex);          // amax = m * 2^ex, m in [0.5, 1)  =>  floor(log2) = ex - 1
      e = (ex - 1) - 2 + 127;         // shared exponent = floor(log2(amax)) - emax(E2M1)
      e = std::max(0, std::min(254, e));
    }
    b[i].e = (uint8_t)e;
    float inv = 1.0f / e8m0_value((uint8_t)e);
    for (int j = 0; j < 16; j++) {
      uint8_t lo = nearest_e2m1(x[i * 32 + j] * inv);
      uint8_t hi = nearest_e2m1(x[i * 32 + j + 16] * inv);
      b[i].qs[j] = lo | (hi << 4);
    }
  }
}

int quantize(uint32_t type, const float* src, void* dst, uint64_t n) {
  const TypeTraits* t = type_traits(type);
  if (!t || n % t->block_elems) return -1;
  uint64_t nb = n / t->block_elems;
  switch (type) {
    case GGML_F32:
      std::memcpy(dst, src, n * 4);
      return 0;
    case GGML_F16:
      for (uint64_t i = 0; i < n; i++) ((uint16_t*)dst)[i] = f32_to_f16(src[i]);
      return 0;
    case GGML_BF16:
      for (uint64_t i = 0; i < n; i++) ((uint16_t*)dst)[i] = f32_to_bf16(src[i]);
      return 0;
    case GGML_Q8_0:
      q_q8_0(src, (BlockQ8_0*)dst, nb);
      return 0;
    case GGML_Q4_K:
      q_q4_k(src, (BlockQ4K*)dst, nb);
      return 0;
    case GGML_Q5_K:
      q_q5_k(src, (BlockQ5K*)dst, nb);
      return 0;
    case GGML_Q6_K:
      q_q6_k(src, (BlockQ6K*)dst, nb);
      return 0;
    case GGML_MXFP4:
      q_mxfp4(src, (BlockMXFP4*)dst, nb);
      return 0;
  }
  return -1;
}

}  // namespace b200
