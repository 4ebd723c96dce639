// Quantized linear for at most 16 activation rows (the AdaLN / embedder linears that see one vector per image):
// y[M, N] = x[M, K] . dequant(W)^T + bias, M <= 16. The work is streaming the packed weights once, so the kernel
// is laid out for HBM bandwidth, not for the tcgen05 pipeline of the large-M kernel:
//   * it reads the same prepared weight blob (codes with the nibble / byte order that gives two neighbouring
//     values per mask, scale|bias pairs transposed to [group][N]);
//   * a warp owns R groups of 8 weight rows and every eighth 128-wide slice of K; a lane loads 16 bytes of codes
//     per group and slice (32 or 16 consecutive k of one row), several slices ahead of their use;
//   * the 16 x 8 x 16 products run on mma.sync (bf16 in, f32 out) with the activation rows as A. A lane feeds the
//     k-slots of a step with its own four consecutive k, and reads the same four k of x for A: a dot product does
//     not care about the order of its terms, so no shuffle is needed to match the instruction's k layout;
//   * the eight warps' partial sums meet in shared memory; bias, SiLU and the store follow.
// Measured, the kernel moves 1.0-2.0 TB/s and its time follows the number of weights, not their bytes: the
// legacy mma.sync path (one m16n8k16 per 128 weights) and the per-weight unpack bound it, not HBM.
// Reference call sites: every nn.Linear that is applied to a conditioning vector, e.g. the AdaLayerNormZero
// linears (src/mflux/models/flux/model/flux_transformer/ada_layer_norm_zero.py:16-18) and the time/text
// embedders (time_text_embed.py:19-31); after quantization they are mlx.nn.QuantizedLinear like all others.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "host_util.cuh"
#include "qmv.cuh"

namespace mfx {
namespace qmv {

constexpr int THREADS = 256;
constexpr int WARPS = 8;

struct Params {
  const __nv_bfloat16* x;
  int64_t x_row_stride;
  int M, N, K;
  const uint32_t* codes;   // prepared codes [N][K * bits / 32]
  const uint32_t* sb;      // [K / 64][N]: bf16 scale | bf16 bias << 16
  const void* bias;
  int bias_dtype;
  int epilogue;            // MFX_EPI_NONE or MFX_EPI_SILU
  void* y;
  int y_dtype;
  int64_t y_row_stride;
};

__device__ __forceinline__ float ld_bias(const void* p, int dtype, int i) {
  if (dtype == MFX_F32) return __ldg(static_cast<const float*>(p) + i);
  if (dtype == MFX_BF16) return __bfloat162float(__ldg(static_cast<const __nv_bfloat16*>(p) + i));
  return __half2float(__ldg(static_cast<const __half*>(p) + i));
}

__device__ __forceinline__ uint32_t sub_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t fma_bf16x2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.bf16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr uint32_t MAGIC = 0x43004300u;  // bf16 pair (128.0, 128.0): OR-ing a 4-bit code gives 128 + code exactly

// Two neighbouring weights (k, k+1) of a 4-bit row: pair index i of a prepared word.
__device__ __forceinline__ uint32_t deq4(uint32_t w, int i, uint32_t scale2, uint32_t bias2) {
  const uint32_t v = ((w >> (4 * i)) & 0x000F000Fu) | MAGIC;
  return fma_bf16x2(sub_bf16x2(v, MAGIC), scale2, bias2);
}
// The four weights of one prepared 8-bit word (bytes e0,e2,e1,e3) as two bf16 pairs (e0,e1), (e2,e3), through
// float32: a byte under the exponent of 2^23 is the float 2^23 + code; packed f32x2 add and fma, one rounding to
// bf16 at the end (the same arithmetic as the large-M kernel's 8-bit path). sc2 / bi2: (scale, scale) and
// (bias, bias) as float32 pairs.
__device__ __forceinline__ void deq8_word(uint32_t w, uint64_t sc2, uint64_t bi2, uint32_t& b0, uint32_t& b1) {
  constexpr uint32_t TWO23 = 0x4B000000u;
  const uint64_t neg = 0xCB000000CB000000ull;  // (-2^23, -2^23)
  uint64_t v01, v23;
  asm("mov.b64 %0, {%1, %2};" : "=l"(v01) : "r"(__byte_perm(w, TWO23, 0x7440)), "r"(__byte_perm(w, TWO23, 0x7442)));
  asm("mov.b64 %0, {%1, %2};" : "=l"(v23) : "r"(__byte_perm(w, TWO23, 0x7441)), "r"(__byte_perm(w, TWO23, 0x7443)));
  asm("add.rn.f32x2 %0, %0, %1;" : "+l"(v01) : "l"(neg));
  asm("add.rn.f32x2 %0, %0, %1;" : "+l"(v23) : "l"(neg));
  asm("fma.rn.f32x2 %0, %0, %1, %2;" : "+l"(v01) : "l"(sc2), "l"(bi2));
  asm("fma.rn.f32x2 %0, %0, %1, %2;" : "+l"(v23) : "l"(sc2), "l"(bi2));
  float a, b, c, d;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v01));
  asm("mov.b64 {%0, %1}, %2;" : "=f"(c), "=f"(d) : "l"(v23));
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  b0 = *reinterpret_cast<const uint32_t*>(&lo);
  b1 = *reinterpret_cast<const uint32_t*>(&hi);
}

// R = groups of 8 weight rows per warp (the A fragments are reused across them). BITS = 4 or 8.
template <int BITS, int R>
__global__ void __launch_bounds__(THREADS) qmv_kernel(const Params p) {
  constexpr int KPL = 128 / BITS;            // k values a lane covers per slice with one 16-byte load: 32 or 16
  constexpr int SLICE = 4 * KPL;             // k per slice: 128 (4-bit) or 64 (8-bit)
  constexpr int STEPS = KPL / 4;             // mma steps per slice: 8 or 4
  __shared__ float red[WARPS][R][32][4];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n_base = blockIdx.x * (8 * R);
  const int words_per_row = p.K * BITS / 32;
  const int slices = (p.K + SLICE - 1) / SLICE;

  float acc[R][4];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f;

  const bool row_lo = g < p.M, row_hi = g + 8 < p.M;
  const __nv_bfloat16* x_lo = p.x + static_cast<int64_t>(g) * p.x_row_stride;
  const __nv_bfloat16* x_hi = p.x + static_cast<int64_t>(g + 8) * p.x_row_stride;

  // codes of the R rows for one slice (16 bytes each); slices are loaded one iteration ahead of their use
  auto load_codes = [&](int s, uint4 (&wv)[R]) {
    const int k0 = s * SLICE + t * KPL;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int n = n_base + 8 * r + g;
      wv[r] = (s < slices && k0 < p.K && n < p.N)
                  ? __ldg(reinterpret_cast<const uint4*>(p.codes + static_cast<int64_t>(n) * words_per_row +
                                                         k0 * BITS / 32))
                  : make_uint4(0, 0, 0, 0);
    }
  };
  uint4 wnext[R];
  load_codes(warp, wnext);
  for (int s = warp; s < slices; s += WARPS) {
    const int k0 = s * SLICE + t * KPL;      // first k of this lane in the slice
    const bool live = k0 < p.K;              // ragged last slice (K is a multiple of 64, a 4-bit slice is 128):
                                             // dead lanes feed zeros, every lane still takes part in the mma
    uint4 wv[R];
#pragma unroll
    for (int r = 0; r < R; ++r) wv[r] = wnext[r];
    load_codes(s + WARPS, wnext);
    // activations of rows g and g + 8 for the same k (KPL values = KPL / 8 16-byte loads each)
    uint32_t xa[KPL / 2], xb[KPL / 2];
#pragma unroll
    for (int i = 0; i < KPL / 8; ++i) {
      const uint4 a = (live && row_lo) ? __ldg(reinterpret_cast<const uint4*>(x_lo + k0) + i) : make_uint4(0, 0, 0, 0);
      const uint4 b = (live && row_hi) ? __ldg(reinterpret_cast<const uint4*>(x_hi + k0) + i) : make_uint4(0, 0, 0, 0);
      xa[4 * i] = a.x; xa[4 * i + 1] = a.y; xa[4 * i + 2] = a.z; xa[4 * i + 3] = a.w;
      xb[4 * i] = b.x; xb[4 * i + 1] = b.y; xb[4 * i + 2] = b.z; xb[4 * i + 3] = b.w;
    }
    const int group = k0 >> 6;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int n = n_base + 8 * r + g;
      const uint32_t sbv = (live && n < p.N) ? __ldg(p.sb + static_cast<int64_t>(group) * p.N + n) : 0u;
      const uint32_t scale2 = __byte_perm(sbv, sbv, 0x1010), bias2 = __byte_perm(sbv, sbv, 0x3232);
      uint64_t sc2 = 0, bi2 = 0;
      if (BITS == 8) {   // the same scale and bias as float32 pairs
        asm("mov.b64 %0, {%1, %1};" : "=l"(sc2) : "r"(sbv << 16));
        asm("mov.b64 %0, {%1, %1};" : "=l"(bi2) : "r"(sbv & 0xFFFF0000u));
      }
      const uint32_t w[4] = {wv[r].x, wv[r].y, wv[r].z, wv[r].w};
#pragma unroll
      for (int st = 0; st < STEPS; ++st) {
        uint32_t b0, b1;
        if (BITS == 4) {
          b0 = deq4(w[st >> 1], 2 * (st & 1), scale2, bias2);
          b1 = deq4(w[st >> 1], 2 * (st & 1) + 1, scale2, bias2);
        } else {
          deq8_word(w[st], sc2, bi2, b0, b1);
        }
        mma_16816(acc[r], xa[2 * st], xb[2 * st], xa[2 * st + 1], xb[2 * st + 1], b0, b1);
      }
    }
  }

#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int i = 0; i < 4; ++i) red[warp][r][lane][i] = acc[r][i];
  __syncthreads();
  // 16 x (8 R) outputs per block; accumulator i of lane (g, t): row g + 8 * (i >> 1), column 2 t + (i & 1)
  for (int o = threadIdx.x; o < R * 128; o += THREADS) {
    const int r = o >> 7, l = (o >> 2) & 31, i = o & 3;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) v += red[w][r][l][i];
    const int m = (l >> 2) + 8 * (i >> 1);
    const int n = n_base + 8 * r + 2 * (l & 3) + (i & 1);
    if (m < p.M && n < p.N) {
      if (p.bias) v += ld_bias(p.bias, p.bias_dtype, n);
      if (p.epilogue == MFX_EPI_SILU) v = v / (1.0f + __expf(-v));
      if (p.y_dtype == MFX_F32) static_cast<float*>(p.y)[m * p.y_row_stride + n] = v;
      else static_cast<__nv_bfloat16*>(p.y)[m * p.y_row_stride + n] = __float2bfloat16_rn(v);
    }
  }
}

bool eligible(const mfx_qlinear_args& a) {
  return a.batch == 1 && a.rows <= 16 && (a.epilogue == MFX_EPI_NONE || a.epilogue == MFX_EPI_SILU);
}

int run(const mfx_qlinear_args& a, const void* prepared, size_t codes_bytes, cudaStream_t st) {
  Params p;
  p.x = static_cast<const __nv_bfloat16*>(a.x);
  p.x_row_stride = a.x_row_stride;
  p.M = static_cast<int>(a.rows);
  p.N = static_cast<int>(a.N);
  p.K = static_cast<int>(a.K);
  p.codes = static_cast<const uint32_t*>(prepared);
  p.sb = reinterpret_cast<const uint32_t*>(static_cast<const uint8_t*>(prepared) + codes_bytes);
  p.bias = a.bias;
  p.bias_dtype = a.bias_dtype;
  p.epilogue = a.epilogue;
  p.y = a.y;
  p.y_dtype = a.y_dtype;
  p.y_row_stride = a.y_row_stride;
  // 16 rows per block while that still gives every SM two blocks, else 8 rows per block (32 rows per block take 100
  // registers and leave two blocks per SM: 10-25 % slower on 9216 to 18432 rows)
  const bool wide = (a.N + 15) / 16 >= 2 * device_sm_count();
  const unsigned blocks = static_cast<unsigned>(wide ? (a.N + 15) / 16 : (a.N + 7) / 8);
  if (kernel_bits(a.bits) == 4) {
    if (wide) qmv_kernel<4, 2><<<blocks, THREADS, 0, st>>>(p);
    else qmv_kernel<4, 1><<<blocks, THREADS, 0, st>>>(p);
  } else {
    if (wide) qmv_kernel<8, 2><<<blocks, THREADS, 0, st>>>(p);
    else qmv_kernel<8, 1><<<blocks, THREADS, 0, st>>>(p);
  }
  MFX_CUDA_TRY(cudaGetLastError());
  return MFX_OK;
}

}  // namespace qmv
}  // namespace mfx
