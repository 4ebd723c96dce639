// Group-wise affine weight quantizer and dequantizer (HBM-bound, load-time kernels).
//
// Semantics follow mx.quantize(w, group_size=64, bits) as reached from the reference through
// mlx.nn.quantize (src/mflux/models/common/weights/loading/weight_applier.py:93-103): groups of 64
// along the input dimension, float32 arithmetic, codes packed little-end first: code j of a row occupies
// bits [j*bits, (j+1)*bits) of the row's bit stream, which for 4 and 8 bits is "8 / 4 codes per uint32" and for
// 3, 5 and 6 bits (the other widths the reference's CLI offers, src/mflux/cli/defaults/defaults.py:63) lets
// codes straddle byte and word boundaries (8 codes in 3 or 5 bytes, 4 codes in 3 bytes).
// Eight lanes own one group (8 values each); min/max go through warp shuffles.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "host_util.cuh"

namespace mfx {
namespace {

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]) {
  if constexpr (sizeof(T) == 4) {
    const float4 a = __ldg(reinterpret_cast<const float4*>(p));
    const float4 b = __ldg(reinterpret_cast<const float4*>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p));
    const T* h = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = to_f32<T>(h[i]);
  }
}

// One thread: 8 consecutive values of a row; lanes 8g..8g+7 of a warp form one 64-wide group.
template <typename T, int BITS, int QMODE>
__global__ void __launch_bounds__(256) quantize_kernel(const T* __restrict__ w, int64_t n_groups_total,
                                                       uint32_t* __restrict__ wq, T* __restrict__ scales,
                                                       T* __restrict__ biases) {
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t group = tid >> 3;
  const bool active = group < n_groups_total;
  const int64_t g = active ? group : n_groups_total - 1;  // keep whole warps in the shuffles
  const int sub = static_cast<int>(tid & 7);
  const T* src = w + g * 64 + sub * 8;
  float v[8];
  load8<T>(src, v);
  float mx = v[0], mn = v[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) {
    mx = fmaxf(mx, v[i]);
    mn = fminf(mn, v[i]);
  }
#pragma unroll
  for (int off = 4; off >= 1; off >>= 1) {
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, off));
  }
  const float n_bins = static_cast<float>((1 << BITS) - 1);
  float scale, bias;
  if (QMODE == MFX_QMODE_MLX) {
    scale = fmaxf(__fdiv_rn(__fsub_rn(mx, mn), n_bins), 1e-7f);
    const bool side = fabsf(mn) > fabsf(mx);
    scale = side ? scale : -scale;
    const float edge = side ? mn : mx;
    const float q0 = rintf(__fdiv_rn(edge, scale));
    if (q0 == 0.0f) {
      bias = 0.0f;
    } else {
      scale = __fdiv_rn(edge, q0);
      bias = edge;
    }
  } else {
    scale = __fdiv_rn(__fsub_rn(mx, mn), n_bins);
    bias = mn;
  }
  uint32_t codes[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float q = rintf(__fdiv_rn(__fsub_rn(v[i], bias), scale));
    if (!(fabsf(q) <= 3.0e38f)) q = 0.0f;  // constant group with scale == 0: code 0
    q = fminf(fmaxf(q, 0.0f), n_bins);
    codes[i] = static_cast<uint32_t>(q);
  }
  if (!active) return;
  if (BITS == 4) {
    uint32_t word = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) word |= codes[i] << (4 * i);
    wq[g * 8 + sub] = word;
  } else if (BITS == 8) {
    uint2 words;
    words.x = codes[0] | (codes[1] << 8) | (codes[2] << 16) | (codes[3] << 24);
    words.y = codes[4] | (codes[5] << 8) | (codes[6] << 16) | (codes[7] << 24);
    reinterpret_cast<uint2*>(wq)[g * 8 + sub] = words;
  } else {
    // 8 codes = BITS bytes of the bit stream, starting at byte (8 * thread) * BITS / 8 of the tensor
    unsigned long long stream = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) stream |= static_cast<unsigned long long>(codes[i]) << (BITS * i);
    uint8_t* dst = reinterpret_cast<uint8_t*>(wq) + (g * 8 + sub) * BITS;
#pragma unroll
    for (int i = 0; i < BITS; ++i) dst[i] = static_cast<uint8_t>(stream >> (8 * i));
  }
  if (sub == 0) {
    scales[g] = from_f32<T>(scale);
    biases[g] = from_f32<T>(bias);
  }
}

// One thread: 8 consecutive outputs of a row.
template <typename SB, typename OUT, int BITS>
__global__ void __launch_bounds__(256) dequantize_kernel(const uint32_t* __restrict__ wq,
                                                         const SB* __restrict__ scales,
                                                         const SB* __restrict__ biases, int64_t n_chunks,
                                                         OUT* __restrict__ out) {
  const int64_t tid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (tid >= n_chunks) return;
  const int64_t g = tid >> 3;
  const float s = to_f32<SB>(scales[g]);
  const float b = to_f32<SB>(biases[g]);
  uint32_t codes[8];
  if (BITS == 4) {
    const uint32_t word = __ldg(wq + tid);
#pragma unroll
    for (int i = 0; i < 8; ++i) codes[i] = (word >> (4 * i)) & 0xF;
  } else if (BITS == 8) {
    const uint2 words = __ldg(reinterpret_cast<const uint2*>(wq) + tid);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      codes[i] = (words.x >> (8 * i)) & 0xFF;
      codes[4 + i] = (words.y >> (8 * i)) & 0xFF;
    }
  } else {
    const uint8_t* src = reinterpret_cast<const uint8_t*>(wq) + tid * BITS;
    unsigned long long stream = 0;
#pragma unroll
    for (int i = 0; i < BITS; ++i) stream |= static_cast<unsigned long long>(__ldg(src + i)) << (8 * i);
#pragma unroll
    for (int i = 0; i < 8; ++i) codes[i] = static_cast<uint32_t>(stream >> (BITS * i)) & ((1u << BITS) - 1u);
  }
  OUT res[8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
    res[i] = from_f32<OUT>(__fadd_rn(__fmul_rn(static_cast<float>(codes[i]), s), b));
  OUT* dst = out + tid * 8;
  if constexpr (sizeof(OUT) == 4) {
    reinterpret_cast<float4*>(dst)[0] = *reinterpret_cast<float4*>(&res[0]);
    reinterpret_cast<float4*>(dst)[1] = *reinterpret_cast<float4*>(&res[4]);
  } else {
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<uint4*>(&res[0]);
  }
}

template <typename T>
int launch_quantize(const void* w, int64_t n_groups, int bits, int qmode, uint32_t* wq, void* scales, void* biases,
                    cudaStream_t st) {
  const int64_t threads = n_groups * 8;
  const unsigned blocks = static_cast<unsigned>((threads + 255) / 256);
  const T* wp = static_cast<const T*>(w);
  T* sp = static_cast<T*>(scales);
  T* bp = static_cast<T*>(biases);
#define MFX_QUANT_CASE(B)                                                                        \
  case B:                                                                                       \
    if (qmode == MFX_QMODE_MLX)                                                                 \
      quantize_kernel<T, B, MFX_QMODE_MLX><<<blocks, 256, 0, st>>>(wp, n_groups, wq, sp, bp);   \
    else                                                                                        \
      quantize_kernel<T, B, MFX_QMODE_DOC><<<blocks, 256, 0, st>>>(wp, n_groups, wq, sp, bp);   \
    break;
  switch (bits) {
    MFX_QUANT_CASE(3)
    MFX_QUANT_CASE(4)
    MFX_QUANT_CASE(5)
    MFX_QUANT_CASE(6)
    MFX_QUANT_CASE(8)
    default: return MFX_ERR_UNSUPPORTED_BITS;
  }
#undef MFX_QUANT_CASE
  MFX_CUDA_TRY(cudaGetLastError());
  return MFX_OK;
}

template <typename SB, typename OUT>
int launch_dequantize(const uint32_t* wq, const void* scales, const void* biases, int64_t n_chunks, int bits,
                      void* out, cudaStream_t st) {
  const unsigned blocks = static_cast<unsigned>((n_chunks + 255) / 256);
  const SB* sp = static_cast<const SB*>(scales);
  const SB* bp = static_cast<const SB*>(biases);
  OUT* op = static_cast<OUT*>(out);
  switch (bits) {
    case 3: dequantize_kernel<SB, OUT, 3><<<blocks, 256, 0, st>>>(wq, sp, bp, n_chunks, op); break;
    case 4: dequantize_kernel<SB, OUT, 4><<<blocks, 256, 0, st>>>(wq, sp, bp, n_chunks, op); break;
    case 5: dequantize_kernel<SB, OUT, 5><<<blocks, 256, 0, st>>>(wq, sp, bp, n_chunks, op); break;
    case 6: dequantize_kernel<SB, OUT, 6><<<blocks, 256, 0, st>>>(wq, sp, bp, n_chunks, op); break;
    case 8: dequantize_kernel<SB, OUT, 8><<<blocks, 256, 0, st>>>(wq, sp, bp, n_chunks, op); break;
    default: return MFX_ERR_UNSUPPORTED_BITS;
  }
  MFX_CUDA_TRY(cudaGetLastError());
  return MFX_OK;
}

template <typename SB>
int dispatch_dequant_out(const uint32_t* wq, const void* scales, const void* biases, int64_t n_chunks, int bits,
                         void* out, int out_dtype, cudaStream_t st) {
  switch (out_dtype) {
    case MFX_F32: return launch_dequantize<SB, float>(wq, scales, biases, n_chunks, bits, out, st);
    case MFX_BF16: return launch_dequantize<SB, __nv_bfloat16>(wq, scales, biases, n_chunks, bits, out, st);
    case MFX_F16: return launch_dequantize<SB, __half>(wq, scales, biases, n_chunks, bits, out, st);
    default: return MFX_ERR_DTYPE;
  }
}

}  // namespace
}  // namespace mfx

extern "C" {

int mfx_quantize_affine(const void* w, int w_dtype, int64_t N, int64_t K, int bits, int group_size, int qmode,
                        uint32_t* wq, void* scales, void* biases, void* stream) {
  using namespace mfx;
  if (!w || !wq || !scales || !biases) return MFX_ERR_NULL;
  if (!valid_bits(bits) || group_size != 64) return MFX_ERR_UNSUPPORTED_BITS;
  if (qmode != MFX_QMODE_MLX && qmode != MFX_QMODE_DOC) return MFX_ERR_SHAPE;
  if (N <= 0 || K <= 0 || K % 64 != 0) return MFX_ERR_SHAPE;
  if (!valid_dtype(w_dtype)) return MFX_ERR_DTYPE;
  if (!aligned16(w) || !aligned16(wq)) return MFX_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t n_groups = N * (K / 64);
  switch (w_dtype) {
    case MFX_F32: return launch_quantize<float>(w, n_groups, bits, qmode, wq, scales, biases, st);
    case MFX_BF16: return launch_quantize<__nv_bfloat16>(w, n_groups, bits, qmode, wq, scales, biases, st);
    default: return launch_quantize<__half>(w, n_groups, bits, qmode, wq, scales, biases, st);
  }
}

int mfx_dequantize_affine(const uint32_t* wq, const void* scales, const void* biases, int sb_dtype, int64_t N,
                          int64_t K, int bits, int group_size, void* out, int out_dtype, void* stream) {
  using namespace mfx;
  if (!wq || !scales || !biases || !out) return MFX_ERR_NULL;
  if (!valid_bits(bits) || group_size != 64) return MFX_ERR_UNSUPPORTED_BITS;
  if (N <= 0 || K <= 0 || K % 64 != 0) return MFX_ERR_SHAPE;
  if (!valid_dtype(sb_dtype) || !valid_dtype(out_dtype)) return MFX_ERR_DTYPE;
  if (!aligned16(wq) || !aligned16(out)) return MFX_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t n_chunks = N * K / 8;
  switch (sb_dtype) {
    case MFX_F32: return dispatch_dequant_out<float>(wq, scales, biases, n_chunks, bits, out, out_dtype, st);
    case MFX_BF16:
      return dispatch_dequant_out<__nv_bfloat16>(wq, scales, biases, n_chunks, bits, out, out_dtype, st);
    default: return dispatch_dequant_out<__half>(wq, scales, biases, n_chunks, bits, out, out_dtype, st);
  }
}

}  // extern "C"
