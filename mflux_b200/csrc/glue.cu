// Bandwidth-bound glue of the transformer blocks: fused, 16-byte vectorised, warp-shuffle reduced.
//   ln_modulate   LayerNorm(affine=False) / RMSNorm(weight) over the hidden dim, then * (1 + scale) + shift
//                 (reference: flux_transformer/ada_layer_norm_zero.py:20, joint_transformer_block.py:86-87,
//                  ada_layer_norm_continuous.py:19; z_image_transformer/transformer_block.py:29-34)
//   qknorm_rope   per-head RMSNorm(128) of Q and K followed by the rotary 2x2 rotation of (even, odd)
//                 pairs, in place inside the fused q|k|v activation buffer
//                 (reference: flux_transformer/common/attention_utils.py:8-36,75-80)
//   vec_ops       conditioning-vector helpers (sum of embeddings, SiLU) and the Euler step
//                 (reference: time_text_embed.py:25-31, linear_scheduler.py:56-58)
// One warp owns one row; nothing here waits on another thread block.
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

// MAXV = number of 8-element vectors a lane may hold: D <= 32 * 8 * MAXV.
template <typename XT, int MAXV>
__global__ void __launch_bounds__(128) norm_modulate_kernel(const NormParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row_id = static_cast<int64_t>(blockIdx.x) * 4 + warp;
  if (row_id >= static_cast<int64_t>(p.rows) * p.batch) return;
  const int b = static_cast<int>(row_id / p.rows);
  const int r = static_cast<int>(row_id % p.rows);
  const XT* x = static_cast<const XT*>(p.x) + b * p.x_batch_stride + static_cast<int64_t>(r) * p.x_row_stride;
  __nv_bfloat16* y = p.y + b * p.y_batch_stride + static_cast<int64_t>(r) * p.y_row_stride;
  const int nvec = p.D >> 3;
  float v[MAXV][8];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec) {
      load8<XT>(x + c * 8, v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) sum += v[i][j];
    }
  }
  float mean = 0.f;
  if (!p.rms) mean = warp_sum(sum) / static_cast<float>(p.D);
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = v[i][j] - mean;
        sq += d * d;
      }
    }
  }
  const float rstd = rsqrtf(warp_sum(sq) / static_cast<float>(p.D) + p.eps);
  // shift / scale / weight are read as 16-byte vectors when their dtype is bf16 (the usual case)
  const bool vec_mod = p.mod_dtype == MFX_BF16;
  const bool vec_w = p.weight_dtype == MFX_BF16;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec) {
      float o[8], sc[8], sh[8], wt[8];
      const int64_t moff = b * p.mod_batch_stride + c * 8;
      if (p.scale) {
        if (vec_mod) load8<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(p.scale) + moff, sc);
        else
#pragma unroll
          for (int j = 0; j < 8; ++j) sc[j] = ld_scalar(p.scale, p.mod_dtype, moff + j);
      }
      if (p.shift) {
        if (vec_mod) load8<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(p.shift) + moff, sh);
        else
#pragma unroll
          for (int j = 0; j < 8; ++j) sh[j] = ld_scalar(p.shift, p.mod_dtype, moff + j);
      }
      if (p.weight) {
        if (vec_w) load8<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(p.weight) + c * 8, wt);
        else
#pragma unroll
          for (int j = 0; j < 8; ++j) wt[j] = ld_scalar(p.weight, p.weight_dtype, c * 8 + j);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float t = (v[i][j] - mean) * rstd;
        if (p.weight) t *= wt[j];
        if (p.scale) t *= 1.0f + sc[j];
        if (p.shift) t += sh[j];
        o[j] = t;
      }
      store8_bf16(y + c * 8, o);
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
};

// residual[b, r, :] += gate[b, :] * RMSNorm(y[b, r, :]) * weight: the "sandwich" post-norm of the Z-Image block
// (z_image_transformer/transformer_block.py:31,35; context_block.py:18,21). The norm needs the whole output row
// of the projection, so it cannot be an epilogue of a matmul tiled along N; this pass reads y once.
template <typename YT, int MAXV>
__global__ void __launch_bounds__(128) norm_gate_residual_kernel(const PostNormParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row_id = static_cast<int64_t>(blockIdx.x) * 4 + warp;
  if (row_id >= static_cast<int64_t>(p.rows) * p.batch) return;
  const int b = static_cast<int>(row_id / p.rows);
  const int r = static_cast<int>(row_id % p.rows);
  const YT* y = static_cast<const YT*>(p.y) + b * p.y_batch_stride + static_cast<int64_t>(r) * p.y_row_stride;
  float* res = p.residual + b * p.res_batch_stride + static_cast<int64_t>(r) * p.res_row_stride;
  const int nvec = p.D >> 3;
  float v[MAXV][8];
  float sq = 0.f;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec) {
      load8<YT>(y + c * 8, v[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) sq += v[i][j] * v[i][j];
    }
  }
  const float rstd = rsqrtf(warp_sum(sq) / static_cast<float>(p.D) + p.eps);
  const bool vec_w = p.weight_dtype == MFX_BF16;
  const bool vec_g = p.gate_dtype == MFX_BF16;
#pragma unroll
  for (int i = 0; i < MAXV; ++i) {
    const int c = lane + 32 * i;
    if (c < nvec) {
      float wt[8], gt[8], rs[8];
      if (vec_w) load8<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(p.weight) + c * 8, wt);
      else
#pragma unroll
        for (int j = 0; j < 8; ++j) wt[j] = ld_scalar(p.weight, p.weight_dtype, c * 8 + j);
      if (p.gate) {
        const int64_t goff = b * p.gate_batch_stride + c * 8;
        if (vec_g) load8<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(p.gate) + goff, gt);
        else
#pragma unroll
          for (int j = 0; j < 8; ++j) gt[j] = ld_scalar(p.gate, p.gate_dtype, goff + j);
      }
      load8<float>(res + c * 8, rs);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float t = v[i][j] * rstd * wt[j];
        if (p.gate) t *= gt[j];
        rs[j] += t;
      }
      *reinterpret_cast<float4*>(res + c * 8) = make_float4(rs[0], rs[1], rs[2], rs[3]);
      *reinterpret_cast<float4*>(res + c * 8 + 4) = make_float4(rs[4], rs[5], rs[6], rs[7]);
    }
  }
}

struct RopeParams {
  __nv_bfloat16* qkv;  // [batch, seq, 3 * heads * 128]: q | k | v
  int64_t row_stride, batch_stride;
  int seq, batch, heads;
  int split;                // rows < split use the *_a norm weights (text stream), the rest *_b
  const void* qw_a;         // RMSNorm weights [128]
  const void* kw_a;
  const void* qw_b;
  const void* kw_b;
  int w_dtype;
  const float* cos_sin;     // [seq, 64, 2] = (cos, sin) per rotated pair
  float eps;
};

// One warp per (token, head): lane l holds elements 4l..4l+3 of Q and of K, i.e. rotary pairs 2l and 2l+1.
__global__ void __launch_bounds__(256) qknorm_rope_kernel(const RopeParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * 8 + warp;
  const int64_t total = static_cast<int64_t>(p.batch) * p.seq * p.heads;
  if (item >= total) return;
  const int h = static_cast<int>(item % p.heads);
  const int64_t tok = item / p.heads;
  const int s = static_cast<int>(tok % p.seq);
  const int b = static_cast<int>(tok / p.seq);
  __nv_bfloat16* row = p.qkv + b * p.batch_stride + static_cast<int64_t>(s) * p.row_stride;
  const float4 cs = __ldg(reinterpret_cast<const float4*>(p.cos_sin + (static_cast<int64_t>(s) * 64 + 2 * lane) * 2));
  const void* qw = s < p.split ? p.qw_a : p.qw_b;
  const void* kw = s < p.split ? p.kw_a : p.kw_b;
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    __nv_bfloat16* ptr = row + (which * p.heads + h) * 128 + lane * 4;
    const void* w = which == 0 ? qw : kw;
    const uint2 raw = *reinterpret_cast<const uint2*>(ptr);
    const __nv_bfloat16* hb = reinterpret_cast<const __nv_bfloat16*>(&raw);
    float x[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) x[j] = __bfloat162float(hb[j]);
    const float ss = warp_sum(x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3]);
    const float r = rsqrtf(ss * (1.0f / 128.0f) + p.eps);
#pragma unroll
    for (int j = 0; j < 4; ++j) x[j] = x[j] * r * ld_scalar(w, p.w_dtype, lane * 4 + j);
    float o[4];
    o[0] = cs.x * x[0] - cs.y * x[1];
    o[1] = cs.y * x[0] + cs.x * x[1];
    o[2] = cs.z * x[2] - cs.w * x[3];
    o[3] = cs.w * x[2] + cs.z * x[3];
    __nv_bfloat162 out2[2] = {__floats2bfloat162_rn(o[0], o[1]), __floats2bfloat162_rn(o[2], o[3])};
    *reinterpret_cast<uint2*>(ptr) = *reinterpret_cast<uint2*>(out2);
  }
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
                                                            float* out, int64_t rows_per_batch, int64_t D,
                                                            int64_t n_vec) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;  // one 8-element vector
  if (i >= n_vec) return;
  const int64_t vec_per_row = D >> 3;
  const int64_t row = i / vec_per_row;
  const int col = static_cast<int>(i % vec_per_row) * 8;
  const int64_t b = row / rows_per_batch;
  float yv[8], rv[8];
  if (y_dtype == MFX_F32) load8<float>(static_cast<const float*>(y) + i * 8, yv);
  else load8<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(y) + i * 8, yv);
  load8<float>(residual + i * 8, rv);
  float o[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float bv = bias ? ld_scalar(bias, bias_dtype, col + j) : 0.f;
    const float gv = ld_scalar(gate, gate_dtype, b * gate_batch_stride + col + j);
    o[j] = rv[j] + gv * (yv[j] + bv);
  }
  *reinterpret_cast<float4*>(out + i * 8) = make_float4(o[0], o[1], o[2], o[3]);
  *reinterpret_cast<float4*>(out + i * 8 + 4) = make_float4(o[4], o[5], o[6], o[7]);
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
  if (a->D > 32 * 8 * 16) return MFX_ERR_TOO_LARGE;
  if (a->x_dtype != MFX_F32 && a->x_dtype != MFX_BF16) return MFX_ERR_DTYPE;
  if ((a->shift || a->scale) && !valid_dtype(a->mod_dtype)) return MFX_ERR_DTYPE;
  if (a->weight && !valid_dtype(a->weight_dtype)) return MFX_ERR_DTYPE;
  const size_t xs = dtype_size(a->x_dtype);
  if (!aligned16(a->x) || (a->x_row_stride * xs) % 16 != 0 || (a->x_batch_stride * xs) % 16 != 0 ||
      !aligned16(a->y) || (a->y_row_stride * 2) % 16 != 0 || (a->y_batch_stride * 2) % 16 != 0)
    return MFX_ERR_ALIGN;
  if (a->mod_dtype == MFX_BF16 && (a->shift || a->scale) &&
      ((a->shift && !aligned16(a->shift)) || (a->scale && !aligned16(a->scale)) || (a->mod_batch_stride * 2) % 16 != 0))
    return MFX_ERR_ALIGN;
  if (a->weight && a->weight_dtype == MFX_BF16 && !aligned16(a->weight)) return MFX_ERR_ALIGN;
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
  const unsigned blocks = static_cast<unsigned>((total + 3) / 4);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int nvec_lane = static_cast<int>((a->D / 8 + 31) / 32);
  if (a->x_dtype == MFX_F32) {
    if (nvec_lane <= 12) norm_modulate_kernel<float, 12><<<blocks, 128, 0, st>>>(p);
    else norm_modulate_kernel<float, 16><<<blocks, 128, 0, st>>>(p);
  } else {
    if (nvec_lane <= 12) norm_modulate_kernel<__nv_bfloat16, 12><<<blocks, 128, 0, st>>>(p);
    else norm_modulate_kernel<__nv_bfloat16, 16><<<blocks, 128, 0, st>>>(p);
  }
  MFX_CUDA_TRY(cudaGetLastError());
  return MFX_OK;
}

int mfx_qknorm_rope(void* qkv, int64_t row_stride, int64_t batch_stride, int64_t seq, int64_t batch, int heads,
                    int64_t split, const void* qw_a, const void* kw_a, const void* qw_b, const void* kw_b,
                    int w_dtype, const float* cos_sin, float eps, void* stream) {
  using namespace mfx;
  using namespace mfx::glue;
  if (!qkv || !qw_a || !kw_a || !qw_b || !kw_b || !cos_sin) return MFX_ERR_NULL;
  if (seq <= 0 || batch <= 0 || heads <= 0 || split < 0) return MFX_ERR_SHAPE;
  if (!valid_dtype(w_dtype)) return MFX_ERR_DTYPE;
  if ((reinterpret_cast<uintptr_t>(qkv) & 7u) || row_stride % 4 != 0 || batch_stride % 4 != 0 || !aligned16(cos_sin))
    return MFX_ERR_ALIGN;
  if (row_stride < 3ll * heads * 128) return MFX_ERR_SHAPE;
  if (int rc = check_arch()) return rc;
  RopeParams p;
  p.qkv = static_cast<__nv_bfloat16*>(qkv);
  p.row_stride = row_stride;
  p.batch_stride = batch_stride;
  p.seq = static_cast<int>(seq);
  p.batch = static_cast<int>(batch);
  p.heads = heads;
  p.split = static_cast<int>(split);
  p.qw_a = qw_a;
  p.kw_a = kw_a;
  p.qw_b = qw_b;
  p.kw_b = kw_b;
  p.w_dtype = w_dtype;
  p.cos_sin = cos_sin;
  p.eps = eps;
  const int64_t total = seq * batch * heads;
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
                      int64_t gate_batch_stride, const float* residual, float* out, int64_t batch, int64_t rows,
                      int64_t D, void* stream) {
  using namespace mfx;
  if (!y || !gate || !residual || !out) return MFX_ERR_NULL;
  if (batch <= 0 || rows <= 0 || D <= 0 || D % 8 != 0) return MFX_ERR_SHAPE;
  if ((y_dtype != MFX_F32 && y_dtype != MFX_BF16) || !valid_dtype(gate_dtype) || (bias && !valid_dtype(bias_dtype)))
    return MFX_ERR_DTYPE;
  if (!aligned16(y) || !aligned16(residual) || !aligned16(out)) return MFX_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  const int64_t n_vec = batch * rows * D / 8;
  glue::gate_residual_kernel<<<static_cast<unsigned>((n_vec + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      y, y_dtype, bias, bias_dtype, gate, gate_dtype, gate_batch_stride, residual, out, rows, D, n_vec);
  MFX_CUDA_TRY(cudaGetLastError());
  return MFX_OK;
}

int mfx_norm_gate_residual(const void* y, int y_dtype, int64_t y_row_stride, int64_t y_batch_stride, int64_t rows,
                           int64_t batch, int64_t D, const void* weight, int weight_dtype, float eps,
                           const void* gate, int gate_dtype, int64_t gate_batch_stride, float* residual,
                           int64_t res_row_stride, int64_t res_batch_stride, void* stream) {
  using namespace mfx;
  using namespace mfx::glue;
  if (!y || !weight || !residual) return MFX_ERR_NULL;
  if (rows <= 0 || batch <= 0 || D <= 0 || D % 8 != 0) return MFX_ERR_SHAPE;
  if (D > 32 * 8 * 16) return MFX_ERR_TOO_LARGE;
  if ((y_dtype != MFX_F32 && y_dtype != MFX_BF16) || !valid_dtype(weight_dtype) || (gate && !valid_dtype(gate_dtype)))
    return MFX_ERR_DTYPE;
  const size_t ys = dtype_size(y_dtype);
  if (!aligned16(y) || (y_row_stride * ys) % 16 != 0 || (y_batch_stride * ys) % 16 != 0 || !aligned16(residual) ||
      (res_row_stride * 4) % 16 != 0 || (res_batch_stride * 4) % 16 != 0)
    return MFX_ERR_ALIGN;
  if (weight_dtype == MFX_BF16 && !aligned16(weight)) return MFX_ERR_ALIGN;
  if (gate && gate_dtype == MFX_BF16 && (!aligned16(gate) || (gate_batch_stride * 2) % 16 != 0)) return MFX_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  PostNormParams p;
  p.y = y;
  p.y_row_stride = y_row_stride;
  p.y_batch_stride = y_batch_stride;
  p.rows = static_cast<int>(rows);
  p.batch = static_cast<int>(batch);
  p.D = static_cast<int>(D);
  p.weight = weight;
  p.weight_dtype = weight_dtype;
  p.eps = eps;
  p.gate = gate;
  p.gate_dtype = gate_dtype;
  p.gate_batch_stride = gate_batch_stride;
  p.residual = residual;
  p.res_row_stride = res_row_stride;
  p.res_batch_stride = res_batch_stride;
  const unsigned blocks = static_cast<unsigned>((rows * batch + 3) / 4);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int nvec_lane = static_cast<int>((D / 8 + 31) / 32);
  if (y_dtype == MFX_F32) {
    if (nvec_lane <= 12) norm_gate_residual_kernel<float, 12><<<blocks, 128, 0, st>>>(p);
    else norm_gate_residual_kernel<float, 16><<<blocks, 128, 0, st>>>(p);
  } else {
    if (nvec_lane <= 12) norm_gate_residual_kernel<__nv_bfloat16, 12><<<blocks, 128, 0, st>>>(p);
    else norm_gate_residual_kernel<__nv_bfloat16, 16><<<blocks, 128, 0, st>>>(p);
  }
  MFX_CUDA_TRY(cudaGetLastError());
  return MFX_OK;
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
