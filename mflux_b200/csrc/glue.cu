// Bandwidth-bound glue of the transformer blocks: fused, 16-byte vectorised, warp-shuffle reduced.
//   ln_modulate   LayerNorm(affine=False) / RMSNorm(weight) over the hidden dim, then * (1 + scale) + shift
//                 (reference: flux_transformer/ada_layer_norm_zero.py:20, joint_transformer_block.py:86-87,
//                  ada_layer_norm_continuous.py:19; z_image_transformer/transformer_block.py:29-34)
//   qknorm_rope   per-head RMSNorm(128) of Q and K followed by the rotary 2x2 rotation of (even, odd)
//                 pairs, in place inside the fused q|k|v activation buffer
//                 (reference: flux_transformer/common/attention_utils.py:8-36,75-80)
//   vec_ops       conditioning-vector helpers (sum of embeddings, SiLU) and the Euler step
//                 (reference: time_text_embed.py:25-31, linear_scheduler.py:56-58)
// The norms give one 128-thread block to a row, the others one warp to a row or head; nothing here waits on
// another thread block.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "host_util.cuh"

namespace mfx {
namespace glue {

__device__ __forceinline__ float ld_scalar(const void* p, int dtype, int64_t i) {
  if (dtype == MFX_F32) return __ldg(static_cast<const float*>(p) + i);
  if (dtype == MFX_BF16) return __bfloat162float(__ldg(static_cast<const __nv_bfloat16*>(p) + i));
  return __half2float(__ldg(static_cast<const __half*>(p) + i));
}

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]) {
  if constexpr (sizeof(T) == 4) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    const float4 b = *(reinterpret_cast<const float4*>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __bfloat162float(h[i]);
  }
}
__device__ __forceinline__ void store8_bf16(__nv_bfloat16* p, const float (&v)[8]) {
  __nv_bfloat162 h[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<uint4*>(h);
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

struct NormParams {
  const void* x;
  int64_t x_row_stride, x_batch_stride;
  int rows, batch, D;
  const void* shift;  // [batch, D] or null
  const void* scale;  // [batch, D] or null
  int mod_dtype;
  int64_t mod_batch_stride;
  const void* weight;  // [D] or null (RMSNorm weight)
  int weight_dtype;
  float eps;
  int rms;  // 0 = LayerNorm (biased variance), 1 = RMSNorm
  __nv_bfloat16* y;
  int64_t y_row_stride, y_batch_stride;
};

// E consecutive elements of a f32 / bf16 / f16 array as floats; E = 4 or 8. bf16 goes as one 8- or 16-byte load.
template <int E>
__device__ __forceinline__ void load_vec(const void* p, int dtype, int64_t off, float (&o)[E]) {
  if (dtype == MFX_BF16) {
    const __nv_bfloat16* q = static_cast<const __nv_bfloat16*>(p) + off;
    if constexpr (E == 8) {
      load8<__nv_bfloat16>(q, o);
    } else {
      const uint2 raw = *reinterpret_cast<const uint2*>(q);
      const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) o[i] = __bfloat162float(h[i]);
    }
  } else if (dtype == MFX_F32) {
    const float* q = static_cast<const float*>(p) + off;
#pragma unroll
    for (int i = 0; i < E; i += 4) {
      const float4 a = *reinterpret_cast<const float4*>(q + i);
      o[i] = a.x; o[i + 1] = a.y; o[i + 2] = a.z; o[i + 3] = a.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < E; ++i) o[i] = ld_scalar(p, dtype, off + i);
  }
}
template <int E>
__device__ __forceinline__ void store_vec_bf16(__nv_bfloat16* p, const float (&v)[E]) {
  if constexpr (E == 8) {
    store8_bf16(p, v);
  } else {
    __nv_bfloat162 h[2] = {__floats2bfloat162_rn(v[0], v[1]), __floats2bfloat162_rn(v[2], v[3])};
    *reinterpret_cast<uint2*>(p) = *reinterpret_cast<uint2*>(h);
  }
}
// Sum over the 128 threads of a block; `red` is a 4-float shared array used by this call only.
__device__ __forceinline__ float block_sum_128(float v, float* red) {
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  return (red[0] + red[1]) + (red[2] + red[3]);
}

constexpr int NORM_THREADS = 128;
constexpr int NORM_MAX_D = 4096;

// One 128-thread block per row. Thread t holds the 16-byte vectors t, t+128, ... of the row in registers (at
// most 32 floats), so every warp-level load or store covers 512 contiguous bytes and enough blocks are resident
// per SM to keep HBM busy; mean and variance are two block reductions over the registers (two-pass variance).
template <typename XT>
__global__ void __launch_bounds__(NORM_THREADS) norm_modulate_kernel(const NormParams p) {
  constexpr int E = 16 / sizeof(XT);
  constexpr int MAXV = NORM_MAX_D / E / NORM_THREADS;
  __shared__ float red[2][4];
  const int t = threadIdx.x;
  const int64_t row_id = blockIdx.x;
  const int b = static_cast<int>(row_id / p.rows);
  const int r = static_cast<int>(row_id % p.rows);
  const XT* x = static_cast<const XT*>(p.x) + b * p.x_batch_stride + static_cast<int64_t>(r) * p.x_row_stride;
  __nv_bfloat16* y = p.y + b * p.y_batch_stride + static_cast<int64_t>(r) * p.y_row_stride;
  const int nvec = p.D / E;
  float v[MAXV][E];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = t + NORM_THREADS * i;
    if (c < nvec) {
      load_vec<E>(x, sizeof(XT) == 4 ? MFX_F32 : MFX_BF16, static_cast<int64_t>(c) * E, v[i]);
#pragma unroll
      for (int j = 0; j < E; ++j) sum += v[i][j];
    }
  }
  float mean = 0.f;
  if (!p.rms) mean = block_sum_128(sum, red[0]) / static_cast<float>(p.D);
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = t + NORM_THREADS * i;
    if (c < nvec) {
#pragma unroll
      for (int j = 0; j < E; ++j) {
        const float d = v[i][j] - mean;
        sq += d * d;
      }
    }
  }
  const float rstd = rsqrtf(block_sum_128(sq, red[1]) / static_cast<float>(p.D) + p.eps);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = t + NORM_THREADS * i;
    if (c < nvec) {
      float o[E], sc[E], sh[E], wt[E];
      const int64_t moff = b * p.mod_batch_stride + static_cast<int64_t>(c) * E;
      if (p.scale) load_vec<E>(p.scale, p.mod_dtype, moff, sc);
      if (p.shift) load_vec<E>(p.shift, p.mod_dtype, moff, sh);
      if (p.weight) load_vec<E>(p.weight, p.weight_dtype, static_cast<int64_t>(c) * E, wt);
#pragma unroll
      for (int j = 0; j < E; ++j) {
        float u = (v[i][j] - mean) * rstd;
        if (p.weight) u *= wt[j];
        if (p.scale) u *= 1.0f + sc[j];
        if (p.shift) u += sh[j];
        o[j] = u;
      }
      store_vec_bf16<E>(y + static_cast<int64_t>(c) * E, o);
    }
  }
}

struct PostNormParams {
  const void* y;  // [batch, rows, D] bf16 or f32
  int64_t y_row_stride, y_batch_stride;
  int rows, batch, D;
  const void* weight;  // RMSNorm weight [D]
  int weight_dtype;
  float eps;
  const void* gate;  // [batch, D] or null (null = gate of one)
  int gate_dtype;
  int64_t gate_batch_stride;
  float* residual;  // [batch, rows, D] f32, updated in place
  int64_t res_row_stride, res_batch_stride;
  // optional second stage: next_out = RMSNorm(updated residual) * next_weight * (1 + next_scale[b]) as bf16
  __nv_bfloat16* next_out;  // null = no second stage
  int64_t next_row_stride, next_batch_stride;
  const void* next_weight;  // [D]
  int next_weight_dtype;
  const void* next_scale;   // [batch, D] or null
  int next_scale_dtype;
  int64_t next_scale_batch_stride;
  float next_eps;
};

// residual[b, r, :] += gate[b, :] * RMSNorm(y[b, r, :]) * weight: the "sandwich" post-norm of the Z-Image block
// (z_image_transformer/transformer_block.py:31,35; context_block.py:18,21). The norm needs the whole output row
// of the projection, so it cannot be an epilogue of a matmul tiled along N; this pass reads y once.
// One 128-thread block per row, 4 elements per vector (8-byte loads of bf16 y, 16-byte of the f32 residual).
// With next_out the block goes on to the pre-norm of the following sub-layer on the row it just updated
// (transformer_block.py:34 after :31, and the next block's :29-30 after :35), which saves reading the stream again.
template <typename YT>
__global__ void __launch_bounds__(NORM_THREADS) norm_gate_residual_kernel(const PostNormParams p) {
  constexpr int E = 4;
  constexpr int MAXV = NORM_MAX_D / E / NORM_THREADS;
  __shared__ float red[4], red2[4];
  const int t = threadIdx.x;
  const int64_t row_id = blockIdx.x;
  const int b = static_cast<int>(row_id / p.rows);
  const int r = static_cast<int>(row_id % p.rows);
  const YT* y = static_cast<const YT*>(p.y) + b * p.y_batch_stride + static_cast<int64_t>(r) * p.y_row_stride;
  float* res = p.residual + b * p.res_batch_stride + static_cast<int64_t>(r) * p.res_row_stride;
  const int nvec = p.D / E;
  float v[MAXV][E];
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = t + NORM_THREADS * i;
    if (c < nvec) {
      load_vec<E>(y, sizeof(YT) == 4 ? MFX_F32 : MFX_BF16, static_cast<int64_t>(c) * E, v[i]);
#pragma unroll
      for (int j = 0; j < E; ++j) sq += v[i][j] * v[i][j];
    }
  }
  const float rstd = rsqrtf(block_sum_128(sq, red) / static_cast<float>(p.D) + p.eps);
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = t + NORM_THREADS * i;
    if (c < nvec) {
      float wt[E], gt[E], rs[E];
      load_vec<E>(p.weight, p.weight_dtype, static_cast<int64_t>(c) * E, wt);
      if (p.gate) load_vec<E>(p.gate, p.gate_dtype, b * p.gate_batch_stride + static_cast<int64_t>(c) * E, gt);
      load_vec<E>(res, MFX_F32, static_cast<int64_t>(c) * E, rs);
#pragma unroll
      for (int j = 0; j < E; ++j) {
        float u = v[i][j] * rstd * wt[j];
        if (p.gate) u *= gt[j];
        rs[j] += u;
        v[i][j] = rs[j];   // the updated stream stays in registers for the optional second stage
      }
      *reinterpret_cast<float4*>(res + static_cast<int64_t>(c) * E) = make_float4(rs[0], rs[1], rs[2], rs[3]);
    }
  }
  if (p.next_out == nullptr) return;   // uniform over the grid
  float sq2 = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = t + NORM_THREADS * i;
    if (c < nvec) {
#pragma unroll
      for (int j = 0; j < E; ++j) sq2 += v[i][j] * v[i][j];
    }
  }
  const float rstd2 = rsqrtf(block_sum_128(sq2, red2) / static_cast<float>(p.D) + p.next_eps);
  __nv_bfloat16* out = p.next_out + b * p.next_batch_stride + static_cast<int64_t>(r) * p.next_row_stride;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = t + NORM_THREADS * i;
    if (c < nvec) {
      float wt[E], sc[E], o[E];
      load_vec<E>(p.next_weight, p.next_weight_dtype, static_cast<int64_t>(c) * E, wt);
      if (p.next_scale)
        load_vec<E>(p.next_scale, p.next_scale_dtype, b * p.next_scale_batch_stride + static_cast<int64_t>(c) * E, sc);
#pragma unroll
      for (int j = 0; j < E; ++j) {
        float u = v[i][j] * rstd2 * wt[j];
        if (p.next_scale) u *= 1.0f + sc[j];
        o[j] = u;
      }
      store_vec_bf16<E>(out + static_cast<int64_t>(c) * E, o);
    }
  }
}

struct RopeParams {
  __nv_bfloat16* qkv;  // [batch, seq, (heads + 2 * kv_heads) * 128]: q | k | v
  int64_t row_stride, batch_stride;
  int seq, batch, heads;
  int kv_heads;             // heads of K (and V): equal to heads unless grouped-query attention
  int rope_mode;            // 0: rotate (even, odd) pairs; 1: pairs (j, j + 64), element j uses angle j / 2
  int split;                // rows < split use the *_a norm weights (text stream), the rest *_b
  const void* qw_a;         // RMSNorm weights [128]
  const void* kw_a;
  const void* qw_b;
  const void* kw_b;
  int w_dtype;
  const float* cos_sin;     // [seq, 64, 2] = (cos, sin) per rotated pair
  float eps;
};

// A warp handles ROPE_HEADS consecutive heads of one token: lanes 0-15 hold the 128 elements of a head's Q,
// lanes 16-31 those of its K, 8 consecutive elements (one 16-byte load, rotary pairs 4l..4l+3) per lane. The
// token's cos/sin and the norm weights are loaded once per warp and all heads' loads are issued before any
// arithmetic; the RMS reduction runs inside a half warp.
constexpr int ROPE_HEADS = 4;
__global__ void __launch_bounds__(256) qknorm_rope_kernel(const RopeParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int groups = (p.heads + ROPE_HEADS - 1) / ROPE_HEADS;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * 8 + warp;
  const int64_t total = static_cast<int64_t>(p.batch) * p.seq * groups;
  if (item >= total) return;
  const int h0 = static_cast<int>(item % groups) * ROPE_HEADS;
  const int64_t tok = item / groups;
  const int s = static_cast<int>(tok % p.seq);
  const int b = static_cast<int>(tok / p.seq);
  const int which = lane >> 4, l = lane & 15;
  __nv_bfloat16* base = p.qkv + b * p.batch_stride + static_cast<int64_t>(s) * p.row_stride +
                        (which * p.heads + h0) * 128 + l * 8;
  const int my_heads = which == 0 ? p.heads : p.kv_heads;   // the K half-warp idles on heads K does not have
  uint4 raw[ROPE_HEADS];
#pragma unroll
  for (int i = 0; i < ROPE_HEADS; ++i)
    raw[i] = h0 + i < my_heads ? *reinterpret_cast<const uint4*>(base + i * 128) : make_uint4(0, 0, 0, 0);
  const float4* csp = reinterpret_cast<const float4*>(p.cos_sin + (static_cast<int64_t>(s) * 64 + 4 * l) * 2);
  const float4 cs0 = __ldg(csp), cs1 = __ldg(csp + 1);
  const void* w = which == 0 ? (s < p.split ? p.qw_a : p.qw_b) : (s < p.split ? p.kw_a : p.kw_b);
  float wt[8];
  load_vec<8>(w, p.w_dtype, l * 8, wt);
#pragma unroll
  for (int i = 0; i < ROPE_HEADS; ++i) {
    if (h0 + i >= p.heads) break;
    const __nv_bfloat16* hb = reinterpret_cast<const __nv_bfloat16*>(&raw[i]);
    float x[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = __bfloat162float(hb[j]);
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += x[j] * x[j];
#pragma unroll
    for (int o = 8; o >= 1; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float r = rsqrtf(ss * (1.0f / 128.0f) + p.eps);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = x[j] * r * wt[j];
    float o[8];
    if (p.rope_mode == 0) {
      o[0] = cs0.x * x[0] - cs0.y * x[1];
      o[1] = cs0.y * x[0] + cs0.x * x[1];
      o[2] = cs0.z * x[2] - cs0.w * x[3];
      o[3] = cs0.w * x[2] + cs0.z * x[3];
      o[4] = cs1.x * x[4] - cs1.y * x[5];
      o[5] = cs1.y * x[4] + cs1.x * x[5];
      o[6] = cs1.z * x[6] - cs1.w * x[7];
      o[7] = cs1.w * x[6] + cs1.z * x[7];
    } else {
      // x * cos + rotate_half(x) * sin with rotate_half(x) = (-x[64:], x[:64]); the partner element sits 8 lanes
      // away, and element j of either half reads the angle j / 2 (angles 4l .. 4l + 3 for this lane's 8 elements)
      const float sgn = l < 8 ? -1.0f : 1.0f;
      const float cc[4] = {cs0.x, cs0.z, cs1.x, cs1.z}, sn[4] = {cs0.y, cs0.w, cs1.y, cs1.w};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float partner = __shfl_xor_sync(0xffffffffu, x[j], 8);
        o[j] = x[j] * cc[j >> 1] + sgn * partner * sn[j >> 1];
      }
    }
    if (h0 + i < my_heads) store8_bf16(base + i * 128, o);
  }
}

// y[r, :] *= act(g[r, :]) on bf16 rows of D elements (8 per thread), rows addressed by (sample, row) strides;
// act 0 = sigmoid, 1 = GELU (erf).
__global__ void __launch_bounds__(256) act_mul_kernel(__nv_bfloat16* y, int64_t y_row_stride, int64_t y_batch_stride,
                                                          const __nv_bfloat16* g, int64_t g_row_stride,
                                                          int64_t g_batch_stride, int rows, int batch, int D, int act) {
  const int vec_per_row = D / 8;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t total = static_cast<int64_t>(batch) * rows * vec_per_row;
  if (idx >= total) return;
  const int c = static_cast<int>(idx % vec_per_row) * 8;
  const int64_t tok = idx / vec_per_row;
  const int r = static_cast<int>(tok % rows);
  const int b = static_cast<int>(tok / rows);
  __nv_bfloat16* yp = y + b * y_batch_stride + static_cast<int64_t>(r) * y_row_stride + c;
  const uint4 yv = *reinterpret_cast<const uint4*>(yp);
  const uint4 gv = *reinterpret_cast<const uint4*>(g + b * g_batch_stride + static_cast<int64_t>(r) * g_row_stride + c);
  const __nv_bfloat16* yh = reinterpret_cast<const __nv_bfloat16*>(&yv);
  const __nv_bfloat16* gh = reinterpret_cast<const __nv_bfloat16*>(&gv);
  float o[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float gv_ = __bfloat162float(gh[j]);
    const float f = act == 0 ? 1.0f / (1.0f + __expf(-gv_)) : 0.5f * gv_ * (1.0f + erff(gv_ * 0.70710678118654752f));
    o[j] = __bfloat162float(yh[j]) * f;
  }
  store8_bf16(yp, o);
}

// out[i] = f(a[i] (+ b[i]) (+ c[i])), f = identity, SiLU or tanh; out dtype bf16 or f32.
__global__ void __launch_bounds__(256) vec_sum_act_kernel(const void* a, const void* b, const void* c, int in_dtype,
                                                          int act, void* out, int out_dtype, int64_t n) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = ld_scalar(a, in_dtype, i);
  if (b) v += ld_scalar(b, in_dtype, i);
  if (c) v += ld_scalar(c, in_dtype, i);
  if (act == 1) v = v / (1.0f + __expf(-v));
  else if (act == 2) v = tanhf(v);
  if (out_dtype == MFX_F32) static_cast<float*>(out)[i] = v;
  else static_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
}

// latents_out = latents + noise * dt  (flow-matching Euler step)
__global__ void __launch_bounds__(256) euler_step_kernel(const void* latents, int lat_dtype, const void* noise,
                                                         int noise_dtype, float dt, void* out, int64_t n) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = ld_scalar(latents, lat_dtype, i) + ld_scalar(noise, noise_dtype, i) * dt;
  if (lat_dtype == MFX_F32) static_cast<float*>(out)[i] = v;
  else if (lat_dtype == MFX_BF16) static_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
  else static_cast<__half*>(out)[i] = __float2half_rn(v);
}


// x[b, r, :] = residual[b, r, :] + gate[b, :] * (y[b, r, :] + bias[:]); residual/x float32 (in place allowed),
// y bf16 or f32. Used after the all-reduce of a row-split (tensor-parallel) linear, where the gated residual
// cannot be an epilogue of the matmul because the partial sums of all ranks must be added first.
__global__ void __launch_bounds__(256) gate_residual_kernel(const void* __restrict__ y, int y_dtype,
                                                            const void* __restrict__ bias, int bias_dtype,
                                                            const void* __restrict__ gate, int gate_dtype,
                                                            int64_t gate_batch_stride, const float* residual,
                                                            float* out, int64_t res_row_stride,
                                                            int64_t res_batch_stride, int64_t rows_per_batch,
                                                            int64_t D, int64_t n_vec) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;  // one 8-element vector
  if (i >= n_vec) return;
  const int64_t vec_per_row = D >> 3;
  const int64_t row = i / vec_per_row;
  const int col = static_cast<int>(i % vec_per_row) * 8;
  const int64_t b = row / rows_per_batch;
  const int64_t roff = b * res_batch_stride + (row - b * rows_per_batch) * res_row_stride + col;
  float yv[8], rv[8];
  if (y_dtype == MFX_F32) load8<float>(static_cast<const float*>(y) + i * 8, yv);
  else load8<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(y) + i * 8, yv);
  load8<float>(residual + roff, rv);
  float o[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float bv = bias ? ld_scalar(bias, bias_dtype, col + j) : 0.f;
    const float gv = ld_scalar(gate, gate_dtype, b * gate_batch_stride + col + j);
    o[j] = rv[j] + gv * (yv[j] + bv);
  }
  *reinterpret_cast<float4*>(out + roff) = make_float4(o[0], o[1], o[2], o[3]);
  *reinterpret_cast<float4*>(out + roff + 4) = make_float4(o[4], o[5], o[6], o[7]);
}

// Classifier-free-guidance combine of two noise predictions, one warp per token row of C <= 1024 channels.
// mode 0: out = n + g * (n - n_neg)                              (z_image.py:209)
// mode 1: comb = n_neg + g * (n - n_neg); out = comb * ||n|| / ||comb|| over the channel axis, eps 1e-12
//         (QwenImage.compute_guided_noise, qwen_image.py:165-174)
__global__ void __launch_bounds__(256) cfg_combine_kernel(const void* __restrict__ n, const void* __restrict__ nn,
                                                          int dtype, float g, int mode, float* __restrict__ out,
                                                          int64_t rows, int C) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 8 + warp;
  if (row >= rows) return;
  float sn = 0.f, sc = 0.f;
  for (int c = lane; c < C; c += 32) {
    const float a = ld_scalar(n, dtype, row * C + c), b = ld_scalar(nn, dtype, row * C + c);
    const float comb = mode == 0 ? a + g * (a - b) : b + g * (a - b);
    sn += a * a;
    sc += comb * comb;
  }
  float ratio = 1.f;
  if (mode == 1) ratio = sqrtf(warp_sum(sn) + 1e-12f) / sqrtf(warp_sum(sc) + 1e-12f);
  for (int c = lane; c < C; c += 32) {
    const float a = ld_scalar(n, dtype, row * C + c), b = ld_scalar(nn, dtype, row * C + c);
    const float comb = mode == 0 ? a + g * (a - b) : b + g * (a - b);
    out[row * C + c] = comb * ratio;
  }
}

}  // namespace glue
}  // namespace mfx

extern "C" {

int mfx_norm_modulate(const mfx_norm_args* a, void* stream) {
  using namespace mfx;
  using namespace mfx::glue;
  if (!a) return MFX_ERR_NULL;
  if (!a->x || !a->y) return MFX_ERR_NULL;
  if (a->rows <= 0 || a->batch <= 0 || a->D <= 0 || a->D % 8 != 0) return MFX_ERR_SHAPE;
  if (a->D > NORM_MAX_D) return MFX_ERR_TOO_LARGE;
  if (a->x_dtype != MFX_F32 && a->x_dtype != MFX_BF16) return MFX_ERR_DTYPE;
  if ((a->shift || a->scale) && !valid_dtype(a->mod_dtype)) return MFX_ERR_DTYPE;
  if (a->weight && !valid_dtype(a->weight_dtype)) return MFX_ERR_DTYPE;
  const size_t xs = dtype_size(a->x_dtype);
  if (!aligned16(a->x) || (a->x_row_stride * xs) % 16 != 0 || (a->x_batch_stride * xs) % 16 != 0 ||
      !aligned16(a->y) || (a->y_row_stride * 2) % 16 != 0 || (a->y_batch_stride * 2) % 16 != 0)
    return MFX_ERR_ALIGN;
  // bf16 and f32 vectors are read with 8- or 16-byte loads
  if (a->mod_dtype != MFX_F16 && (a->shift || a->scale) &&
      ((a->shift && !aligned16(a->shift)) || (a->scale && !aligned16(a->scale)) ||
       (a->mod_batch_stride * dtype_size(a->mod_dtype)) % 16 != 0))
    return MFX_ERR_ALIGN;
  if (a->weight && a->weight_dtype != MFX_F16 && !aligned16(a->weight)) return MFX_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  NormParams p;
  p.x = a->x;
  p.x_row_stride = a->x_row_stride;
  p.x_batch_stride = a->x_batch_stride;
  p.rows = static_cast<int>(a->rows);
  p.batch = static_cast<int>(a->batch);
  p.D = static_cast<int>(a->D);
  p.shift = a->shift;
  p.scale = a->scale;
  p.mod_dtype = a->mod_dtype;
  p.mod_batch_stride = a->mod_batch_stride;
  p.weight = a->weight;
  p.weight_dtype = a->weight_dtype;
  p.eps = a->eps;
  p.rms = a->rms;
  p.y = static_cast<__nv_bfloat16*>(a->y);
  p.y_row_stride = a->y_row_stride;
  p.y_batch_stride = a->y_batch_stride;
  const int64_t total = a->rows * a->batch;
  if (total > 0x7fffffffll) return MFX_ERR_TOO_LARGE;
  const unsigned blocks = static_cast<unsigned>(total);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a->x_dtype == MFX_F32) norm_modulate_kernel<float><<<blocks, NORM_THREADS, 0, st>>>(p);
  else norm_modulate_kernel<__nv_bfloat16><<<blocks, NORM_THREADS, 0, st>>>(p);
  MFX_CUDA_TRY(cudaGetLastError());
  return MFX_OK;
}

int mfx_qknorm_rope(void* qkv, int64_t row_stride, int64_t batch_stride, int64_t seq, int64_t batch, int heads,
                    int64_t split, const void* qw_a, const void* kw_a, const void* qw_b, const void* kw_b,
                    int w_dtype, const float* cos_sin, float eps, void* stream) {
  return mfx_qknorm_rope_gqa(qkv, row_stride, batch_stride, seq, batch, heads, heads, 0, split, qw_a, kw_a, qw_b, kw_b,
                             w_dtype, cos_sin, eps, stream);
}

int mfx_act_mul(void* y, int64_t y_row_stride, int64_t y_batch_stride, const void* gate, int64_t g_row_stride,
                int64_t g_batch_stride, int64_t rows, int64_t batch, int64_t D, int act, void* stream) {
  using namespace mfx;
  if (!y || !gate) return MFX_ERR_NULL;
  if (rows <= 0 || batch <= 0 || D <= 0 || D % 8 != 0 || act < 0 || act > 1) return MFX_ERR_SHAPE;
  if (!aligned16(y) || !aligned16(gate) || y_row_stride % 8 != 0 || y_batch_stride % 8 != 0 || g_row_stride % 8 != 0 ||
      g_batch_stride % 8 != 0)
    return MFX_ERR_ALIGN;
  if (rows > (1ll << 30) || batch > 65535) return MFX_ERR_TOO_LARGE;
  if (int rc = check_arch()) return rc;
  const int64_t total = rows * batch * (D / 8);
  glue::act_mul_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<__nv_bfloat16*>(y), y_row_stride, y_batch_stride, static_cast<const __nv_bfloat16*>(gate),
      g_row_stride, g_batch_stride, static_cast<int>(rows), static_cast<int>(batch), static_cast<int>(D), act);
  MFX_CUDA_TRY(cudaGetLastError());
  return MFX_OK;
}

int mfx_qknorm_rope_gqa(void* qkv, int64_t row_stride, int64_t batch_stride, int64_t seq, int64_t batch, int heads,
                        int kv_heads, int rope_mode, int64_t split, const void* qw_a, const void* kw_a, const void* qw_b,
                        const void* kw_b, int w_dtype, const float* cos_sin, float eps, void* stream) {
  using namespace mfx;
  using namespace mfx::glue;
  if (!qkv || !qw_a || !kw_a || !qw_b || !kw_b || !cos_sin) return MFX_ERR_NULL;
  if (seq <= 0 || batch <= 0 || heads <= 0 || kv_heads <= 0 || kv_heads > heads || split < 0 || rope_mode < 0 ||
      rope_mode > 1)
    return MFX_ERR_SHAPE;
  if (!valid_dtype(w_dtype)) return MFX_ERR_DTYPE;
  if (!aligned16(qkv) || row_stride % 8 != 0 || batch_stride % 8 != 0 || !aligned16(cos_sin) ||
      (w_dtype != MFX_F16 && (!aligned16(qw_a) || !aligned16(kw_a) || !aligned16(qw_b) || !aligned16(kw_b))))
    return MFX_ERR_ALIGN;
  if (row_stride < (heads + 2ll * kv_heads) * 128) return MFX_ERR_SHAPE;
  if (int rc = check_arch()) return rc;
  RopeParams p;
  p.qkv = static_cast<__nv_bfloat16*>(qkv);
  p.row_stride = row_stride;
  p.batch_stride = batch_stride;
  p.seq = static_cast<int>(seq);
  p.batch = static_cast<int>(batch);
  p.heads = heads;
  p.kv_heads = kv_heads;
  p.rope_mode = rope_mode;
  p.split = static_cast<int>(split);
  p.qw_a = qw_a;
  p.kw_a = kw_a;
  p.qw_b = qw_b;
  p.kw_b = kw_b;
  p.w_dtype = w_dtype;
  p.cos_sin = cos_sin;
  p.eps = eps;
  const int64_t total = seq * batch * ((heads + glue::ROPE_HEADS - 1) / glue::ROPE_HEADS);
  qknorm_rope_kernel<<<static_cast<unsigned>((total + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  MFX_CUDA_TRY(cudaGetLastError());
  return MFX_OK;
}

int mfx_vec_sum_act(const void* a, const void* b, const void* c, int in_dtype, int act, void* out, int out_dtype,
                    int64_t n, void* stream) {
  using namespace mfx;
  if (!a || !out) return MFX_ERR_NULL;
  if (n <= 0 || act < 0 || act > 2) return MFX_ERR_SHAPE;
  if (!valid_dtype(in_dtype) || (out_dtype != MFX_F32 && out_dtype != MFX_BF16)) return MFX_ERR_DTYPE;
  if (int rc = check_arch()) return rc;
  glue::vec_sum_act_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      a, b, c, in_dtype, act, out, out_dtype, n);
  MFX_CUDA_TRY(cudaGetLastError());
  return MFX_OK;
}

int mfx_euler_step(const void* latents, int lat_dtype, const void* noise, int noise_dtype, float dt, void* out,
                   int64_t n, void* stream) {
  using namespace mfx;
  if (!latents || !noise || !out) return MFX_ERR_NULL;
  if (n <= 0) return MFX_ERR_SHAPE;
  if (!valid_dtype(lat_dtype) || !valid_dtype(noise_dtype)) return MFX_ERR_DTYPE;
  if (int rc = check_arch()) return rc;
  glue::euler_step_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      latents, lat_dtype, noise, noise_dtype, dt, out, n);
  MFX_CUDA_TRY(cudaGetLastError());
  return MFX_OK;
}

int mfx_gate_residual(const void* y, int y_dtype, const void* bias, int bias_dtype, const void* gate, int gate_dtype,
                      int64_t gate_batch_stride, const float* residual, float* out, int64_t res_row_stride,
                      int64_t res_batch_stride, int64_t batch, int64_t rows, int64_t D, void* stream) {
  using namespace mfx;
  if (!y || !gate || !residual || !out) return MFX_ERR_NULL;
  if (batch <= 0 || rows <= 0 || D <= 0 || D % 8 != 0) return MFX_ERR_SHAPE;
  if ((y_dtype != MFX_F32 && y_dtype != MFX_BF16) || !valid_dtype(gate_dtype) || (bias && !valid_dtype(bias_dtype)))
    return MFX_ERR_DTYPE;
  if (!aligned16(y) || !aligned16(residual) || !aligned16(out) || res_row_stride % 4 != 0 || res_batch_stride % 4 != 0)
    return MFX_ERR_ALIGN;
  if (res_row_stride < D) return MFX_ERR_SHAPE;
  if (int rc = check_arch()) return rc;
  const int64_t n_vec = batch * rows * D / 8;
  glue::gate_residual_kernel<<<static_cast<unsigned>((n_vec + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      y, y_dtype, bias, bias_dtype, gate, gate_dtype, gate_batch_stride, residual, out, res_row_stride, res_batch_stride, rows,
      D, n_vec);
  MFX_CUDA_TRY(cudaGetLastError());
  return MFX_OK;
}

int mfx_post_pre_norm(const mfx_post_pre_norm_args* a, void* stream) {
  using namespace mfx;
  using namespace mfx::glue;
  if (!a || !a->y || !a->weight || !a->residual) return MFX_ERR_NULL;
  if (a->rows <= 0 || a->batch <= 0 || a->D <= 0 || a->D % 8 != 0) return MFX_ERR_SHAPE;
  if (a->D > NORM_MAX_D) return MFX_ERR_TOO_LARGE;
  if ((a->y_dtype != MFX_F32 && a->y_dtype != MFX_BF16) || !valid_dtype(a->weight_dtype) ||
      (a->gate && !valid_dtype(a->gate_dtype)))
    return MFX_ERR_DTYPE;
  const size_t ys = dtype_size(a->y_dtype);
  if (!aligned16(a->y) || (a->y_row_stride * ys) % 16 != 0 || (a->y_batch_stride * ys) % 16 != 0 ||
      !aligned16(a->residual) || (a->res_row_stride * 4) % 16 != 0 || (a->res_batch_stride * 4) % 16 != 0)
    return MFX_ERR_ALIGN;
  if (a->weight_dtype != MFX_F16 && !aligned16(a->weight)) return MFX_ERR_ALIGN;
  if (a->gate && a->gate_dtype != MFX_F16 &&
      (!aligned16(a->gate) || (a->gate_batch_stride * dtype_size(a->gate_dtype)) % 16 != 0))
    return MFX_ERR_ALIGN;
  if (a->next_out) {
    if (!a->next_weight) return MFX_ERR_NULL;
    if (!valid_dtype(a->next_weight_dtype) || (a->next_scale && !valid_dtype(a->next_scale_dtype))) return MFX_ERR_DTYPE;
    if (!aligned16(a->next_out) || (a->next_row_stride * 2) % 16 != 0 || (a->next_batch_stride * 2) % 16 != 0)
      return MFX_ERR_ALIGN;
    if (a->next_weight_dtype != MFX_F16 && !aligned16(a->next_weight)) return MFX_ERR_ALIGN;
    if (a->next_scale && a->next_scale_dtype != MFX_F16 &&
        (!aligned16(a->next_scale) || (a->next_scale_batch_stride * dtype_size(a->next_scale_dtype)) % 16 != 0))
      return MFX_ERR_ALIGN;
  }
  if (int rc = check_arch()) return rc;
  PostNormParams p;
  p.y = a->y;
  p.y_row_stride = a->y_row_stride;
  p.y_batch_stride = a->y_batch_stride;
  p.rows = static_cast<int>(a->rows);
  p.batch = static_cast<int>(a->batch);
  p.D = static_cast<int>(a->D);
  p.weight = a->weight;
  p.weight_dtype = a->weight_dtype;
  p.eps = a->eps;
  p.gate = a->gate;
  p.gate_dtype = a->gate_dtype;
  p.gate_batch_stride = a->gate_batch_stride;
  p.residual = a->residual;
  p.res_row_stride = a->res_row_stride;
  p.res_batch_stride = a->res_batch_stride;
  p.next_out = static_cast<__nv_bfloat16*>(a->next_out);
  p.next_row_stride = a->next_row_stride;
  p.next_batch_stride = a->next_batch_stride;
  p.next_weight = a->next_weight;
  p.next_weight_dtype = a->next_weight_dtype;
  p.next_scale = a->next_scale;
  p.next_scale_dtype = a->next_scale_dtype;
  p.next_scale_batch_stride = a->next_scale_batch_stride;
  p.next_eps = a->next_eps;
  if (a->rows * a->batch > 0x7fffffffll) return MFX_ERR_TOO_LARGE;
  const unsigned blocks = static_cast<unsigned>(a->rows * a->batch);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a->y_dtype == MFX_F32) norm_gate_residual_kernel<float><<<blocks, NORM_THREADS, 0, st>>>(p);
  else norm_gate_residual_kernel<__nv_bfloat16><<<blocks, NORM_THREADS, 0, st>>>(p);
  MFX_CUDA_TRY(cudaGetLastError());
  return MFX_OK;
}

int mfx_norm_gate_residual(const void* y, int y_dtype, int64_t y_row_stride, int64_t y_batch_stride, int64_t rows,
                           int64_t batch, int64_t D, const void* weight, int weight_dtype, float eps,
                           const void* gate, int gate_dtype, int64_t gate_batch_stride, float* residual,
                           int64_t res_row_stride, int64_t res_batch_stride, void* stream) {
  mfx_post_pre_norm_args a;
  memset(&a, 0, sizeof(a));
  a.y = y;
  a.y_dtype = y_dtype;
  a.y_row_stride = y_row_stride;
  a.y_batch_stride = y_batch_stride;
  a.rows = rows;
  a.batch = batch;
  a.D = D;
  a.weight = weight;
  a.weight_dtype = weight_dtype;
  a.eps = eps;
  a.gate = gate;
  a.gate_dtype = gate_dtype;
  a.gate_batch_stride = gate_batch_stride;
  a.residual = residual;
  a.res_row_stride = res_row_stride;
  a.res_batch_stride = res_batch_stride;
  return mfx_post_pre_norm(&a, stream);
}

int mfx_cfg_combine(const void* noise, const void* noise_negative, int dtype, float guidance, int mode, float* out,
                    int64_t rows, int64_t channels, void* stream) {
  using namespace mfx;
  if (!noise || !noise_negative || !out) return MFX_ERR_NULL;
  if (rows <= 0 || channels <= 0 || channels > 1024 || (mode != 0 && mode != 1)) return MFX_ERR_SHAPE;
  if (!valid_dtype(dtype)) return MFX_ERR_DTYPE;
  if (int rc = check_arch()) return rc;
  glue::cfg_combine_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      noise, noise_negative, dtype, guidance, mode, out, rows, static_cast<int>(channels));
  MFX_CUDA_TRY(cudaGetLastError());
  return MFX_OK;
}

}  // extern "C"
