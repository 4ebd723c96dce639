// Device helpers shared by the two tensor-core quantized-matmul kernels (qmm.cu, qmm_t.cu): scalar loads by dtype
// code, the 4- and 8-bit dequantizers over the prepared code layout, and the epilogue activations.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "host_util.cuh"
#include "ptx.cuh"

namespace mfx {
namespace qmm {

__device__ __forceinline__ float load_scalar(const void* p, int dtype, int64_t i) {
  if (dtype == MFX_F32) return __ldg(static_cast<const float*>(p) + i);
  if (dtype == MFX_BF16) return __bfloat162float(__ldg(static_cast<const __nv_bfloat16*>(p) + i));
  return __half2float(__ldg(static_cast<const __half*>(p) + i));
}

// d = (a - magic) * s + b on packed 16-bit pairs: the subtraction is exact (small integers),
// the fma rounds once.
__device__ __forceinline__ uint32_t sub_fma(uint32_t a, uint32_t magic, uint32_t s, uint32_t b) {
  uint32_t d;
  asm("{\n\t.reg .b32 t;\n\t"
      "sub.rn.bf16x2 t, %1, %2;\n\t"
      "fma.rn.bf16x2 %0, t, %3, %4;\n\t}"
      : "=r"(d)
      : "r"(a), "r"(magic), "r"(s), "r"(b));
  return d;
}

// 8 four-bit codes of one prepared uint32 (nibble order e0,e2,e4,e6,e1,e3,e5,e7) -> 8 values in K order:
// nibble j lands in the low half and nibble 4+j in the high half of one masked word.
__device__ __forceinline__ uint4 dequant_w4(uint32_t q, uint32_t s2, uint32_t b2) {
  constexpr uint32_t MAGIC = 0x43004300u;  // bf16 128.0 twice: ulp 1 up to 255
  uint4 r;
  r.x = sub_fma((q & 0x000F000Fu) | MAGIC, MAGIC, s2, b2);          // (e0, e1)
  r.y = sub_fma(((q >> 4) & 0x000F000Fu) | MAGIC, MAGIC, s2, b2);   // (e2, e3)
  r.z = sub_fma(((q >> 8) & 0x000F000Fu) | MAGIC, MAGIC, s2, b2);   // (e4, e5)
  r.w = sub_fma(((q >> 12) & 0x000F000Fu) | MAGIC, MAGIC, s2, b2);  // (e6, e7)
  return r;
}

// 4 eight-bit codes of one prepared uint32 (byte order e0,e2,e1,e3) -> 4 values in K order, through float32:
// a byte placed under the exponent of 2^23 is the float 2^23 + code exactly; subtracting 2^23 and one fma with
// the group's scale and bias (packed f32x2 instructions) give the value, rounded once more when packed to bf16.
// sc2 / bi2 are (scale, scale) / (bias, bias) as float32 pairs.
__device__ __forceinline__ uint2 dequant_w8_f32(uint32_t q, uint64_t sc2, uint64_t bi2) {
  constexpr uint32_t TWO23 = 0x4B000000u;
  const uint64_t neg = 0xCB000000CB000000ull;  // (-2^23, -2^23)
  uint64_t v01, v23;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v01) : "r"(__byte_perm(q, TWO23, 0x7440)), "r"(__byte_perm(q, TWO23, 0x7442)));
  asm("mov.b64 %0, {%1, %2};" : "=l"(v23) : "r"(__byte_perm(q, TWO23, 0x7441)), "r"(__byte_perm(q, TWO23, 0x7443)));
  asm("add.rn.f32x2 %0, %0, %1;" : "+l"(v01) : "l"(neg));
  asm("add.rn.f32x2 %0, %0, %1;" : "+l"(v23) : "l"(neg));
  asm("fma.rn.f32x2 %0, %0, %1, %2;" : "+l"(v01) : "l"(sc2), "l"(bi2));
  asm("fma.rn.f32x2 %0, %0, %1, %2;" : "+l"(v23) : "l"(sc2), "l"(bi2));
  float a, b, c, d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v01));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(c), "=f"(d) : "l"(v23));
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 r;
  r.x = *reinterpret_cast<const uint32_t*>(&lo);
  r.y = *reinterpret_cast<const uint32_t*>(&hi);
  return r;
}

// Out of line on purpose: the epilogue runs beside the main loop of the next tile; a 32-fold unrolled inline
// erf/tanh body would crowd the small hot loops of the other warps out of the instruction cache.
static __device__ __noinline__ float gelu_erf(float v) { return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f)); }
static __device__ __noinline__ float gelu_tanh(float v) {
  const float u = 0.7978845608028654f * (v + 0.044715f * v * v * v);
  return 0.5f * v * (1.0f + tanhf(u));
}
__device__ __forceinline__ float silu(float v) { return v / (1.0f + __expf(-v)); }

}  // namespace qmm
}  // namespace mfx
