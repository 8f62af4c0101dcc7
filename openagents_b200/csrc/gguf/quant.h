// Block-quantized tensor formats of the GGUF container: layouts, CPU dequantizers and
// CPU quantizers.  The layouts follow the public ggml specification (the reference tree
// holds no quantization code; it only names the formats its model server loads:
// docs/muse/muse-glimmer.md:112 "Q4_K, Q5_K, Q6_K, and other GGUF quantizations").
#pragma once
#include <cstddef>
#include <cstdint>

namespace b200 {

enum GgmlType : uint32_t {
  GGML_F32 = 0,
  GGML_F16 = 1,
  GGML_Q8_0 = 8,
  GGML_Q4_K = 12,
  GGML_Q5_K = 13,
  GGML_Q6_K = 14,
  GGML_BF16 = 30,
  GGML_MXFP4 = 39,
};

struct TypeTraits {
  uint32_t type;
  const char* name;
  uint32_t block_elems;  // elements per block
  uint32_t block_bytes;  // bytes per block
};

// Returns nullptr for a type this library does not handle.
const TypeTraits* type_traits(uint32_t type);

// Bytes of a row-major tensor with `n` elements (n must be a multiple of block_elems).
size_t tensor_bytes(uint32_t type, uint64_t n);

uint16_t f32_to_f16(float f);
float f16_to_f32(uint16_t h);
uint16_t f32_to_bf16(float f);
float bf16_to_f32(uint16_t h);

#pragma pack(push, 1)
struct BlockQ8_0 {  // 32 elements, 34 bytes
  uint16_t d;       // fp16 scale
  int8_t qs[32];
};
struct BlockQ4K {      // 256 elements, 144 bytes
  uint16_t d;          // fp16 super-scale of the sub-block scales
  uint16_t dmin;       // fp16 super-scale of the sub-block mins
  uint8_t scales[12];  // 8 six-bit scales and 8 six-bit mins
  uint8_t qs[128];     // 4-bit quants: each 32-byte group holds 64 elements
};
struct BlockQ5K {      // 256 elements, 176 bytes
  uint16_t d;
  uint16_t dmin;
  uint8_t scales[12];
  uint8_t qh[32];      // fifth bit
  uint8_t qs[128];
};
struct BlockQ6K {      // 256 elements, 210 bytes
  uint8_t ql[128];     // low 4 bits
  uint8_t qh[64];      // high 2 bits
  int8_t scales[16];   // one per 16 elements
  uint16_t d;          // fp16 super-scale
};
struct BlockMXFP4 {    // 32 elements, 17 bytes
  uint8_t e;           // E8M0 shared exponent
  uint8_t qs[16];      // two E2M1 values per byte: low nibble = j, high nibble = j + 16
};
#pragma pack(pop)

static_assert(sizeof(BlockQ8_0) == 34, "q8_0");
static_assert(sizeof(BlockQ4K) == 144, "q4_k");
static_assert(sizeof(BlockQ5K) == 176, "q5_k");
static_assert(sizeof(BlockQ6K) == 210, "q6_k");
static_assert(sizeof(BlockMXFP4) == 17, "mxfp4");

// Unpack the j-th (0..7) six-bit scale and min of a Q4_K / Q5_K superblock.
inline void unpack_scale_min_k4(int j, const uint8_t* q, uint8_t* sc, uint8_t* mn) {
  if (j < 4) {
    *sc = q[j] & 63;
    *mn = q[j + 4] & 63;
  } else {
    *sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
    *mn = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
}

// E2M1 code (0..15) -> value.
float e2m1_value(uint8_t code);
// E8M0 exponent byte -> scale (2^(e-127)).
float e8m0_value(uint8_t e);

// n elements (multiple of the block size) from `src` into fp32 `dst`.  Returns 0, or -1 for an
// unknown type or a bad element count.
int dequantize(uint32_t type, const void* src, float* dst, uint64_t n);
// n fp32 elements into `dst` (tensor_bytes(type, n) bytes).  Deterministic; returns 0 or -1.
int quantize(uint32_t type, const float* src, void* dst, uint64_t n);

}  // namespace b200
