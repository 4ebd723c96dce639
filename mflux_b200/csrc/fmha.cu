// Non-causal flash attention for head dimension 128 on tcgen05 (sm_100a).
//
// Replaces mx.fast.scaled_dot_product_attention(q, k, v, scale) as called by the reference's
// AttentionUtils.compute_attention (src/mflux/models/flux/model/flux_transformer/common/attention_utils.py:48-52).
//
// One CTA = one (sample, head, 128-query tile); two CTAs share an SM so that the softmax of one overlaps
// the tensor-core work of the other. 192 threads:
//   warp 0     TMA producer: Q once, then K and V tiles of 128 keys (128-byte swizzle, two 64-wide halves of d)
//   warp 1     allocates 256 TMEM columns, issues tcgen05.mma:
//                S[128 q x 128 keys] = Q K^T            (both operands from shared memory, K-major)
//                O[128 q x 128 d]   += P V              (P bf16 from tensor memory, V MN-major from shared memory)
//   warps 2-5  softmax: tcgen05.ld S (thread = query row), running max kept stale until it would grow by
//              more than 2^8 (then O and the row sum are rescaled), exp2, P -> tcgen05.st over the S columns,
//              finally O / rowsum -> global
// All waits are bounded.
#include <cuda_bf16.h>

#include "host_util.cuh"
#include "ptx.cuh"

namespace mfx {
namespace fmha {

constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr int HD = 128;
constexpr int NUM_THREADS = 192;
constexpr int TILE_BYTES = 128 * HD * 2;  // 32 KiB: [128 rows][128 d] bf16 as two 16 KiB halves of d
constexpr int HALF_BYTES = TILE_BYTES / 2;
constexpr uint32_t TMEM_COLS = 256;
constexpr uint32_t COL_S = 0;    // S fp32 [0,128); P bf16 pairs reuse [0,64)
constexpr uint32_t COL_O = 128;  // O fp32 [128,256)

constexpr int OFF_Q = 0;
constexpr int OFF_K = OFF_Q + TILE_BYTES;
constexpr int OFF_V = OFF_K + TILE_BYTES;
constexpr int OFF_BAR = OFF_V + TILE_BYTES;
constexpr int NUM_BARS = 9;
constexpr int OFF_TMEM = OFF_BAR + NUM_BARS * 8;
constexpr int DYN_BYTES = OFF_TMEM + 16 + 1024;

struct Params {
  int seq, batch, heads;
  float scale_log2;  // scale * log2(e)
  __nv_bfloat16* out;
  int64_t out_row_stride, out_batch_stride;
};

// Shared-memory descriptor of an MN-major operand stored as [K rows][64 MN elements = 128 B] with the
// 128-byte swizzle: 8-row K groups 1024 B apart (stride byte offset), 64-element MN chunks `mn_chunk_bytes`
// apart (leading byte offset).
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(uint32_t saddr, uint32_t mn_chunk_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(mn_chunk_bytes >> 4) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(NUM_THREADS, 2)
fmha_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
            const __grid_constant__ CUtensorMap tmap_v, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t q_s = smem_base + OFF_Q, k_s = smem_base + OFF_K, v_s = smem_base + OFF_V;
  const uint32_t bar0 = smem_base + OFF_BAR;
  const uint32_t q_full = bar0, k_full = bar0 + 8, v_full = bar0 + 16, k_empty = bar0 + 24, v_empty = bar0 + 32,
                 s_full = bar0 + 40, p_full = bar0 + 48, o_full = bar0 + 56;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + OFF_TMEM);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * BQ;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int n_tiles = (p.seq + BKV - 1) / BKV;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(k_full, 1);
    mbar_init(v_full, 1);
    mbar_init(k_empty, 1);
    mbar_init(v_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(p_full, 4);
    mbar_init(o_full, 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(smem_base + OFF_TMEM, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_arrive_expect_tx(q_full, TILE_BYTES);
      tma_load_4d(q_s, &tmap_q, q_full, 0, h, q0, b);
      tma_load_4d(q_s + HALF_BYTES, &tmap_q, q_full, 64, h, q0, b);
    }
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const uint32_t ph = static_cast<uint32_t>(j & 1);
      if (!mbar_wait(k_empty, ph ^ 1u, DEV_TIMEOUT_ATTN)) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(k_full, TILE_BYTES);
        tma_load_4d(k_s, &tmap_k, k_full, 0, h, j * BKV, b);
        tma_load_4d(k_s + HALF_BYTES, &tmap_k, k_full, 64, h, j * BKV, b);
      }
      if (!mbar_wait(v_empty, ph ^ 1u, DEV_TIMEOUT_ATTN)) break;
      if (lane == 0) {
        mbar_arrive_expect_tx(v_full, TILE_BYTES);
        tma_load_4d(v_s, &tmap_v, v_full, 0, h, j * BKV, b);
        tma_load_4d(v_s + HALF_BYTES, &tmap_v, v_full, 64, h, j * BKV, b);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    constexpr uint32_t IDESC_S = make_idesc(FMT_BF16, FMT_BF16, BQ, BKV);       // K-major x K-major
    constexpr uint32_t IDESC_O = make_idesc_b_mn(FMT_BF16, FMT_BF16, BQ, HD);   // P (TMEM) x V (MN-major)
    bool ok = mbar_wait(q_full, 0, DEV_TIMEOUT_ATTN);
    for (int j = 0; j < n_tiles && ok; ++j) {
      const uint32_t ph = static_cast<uint32_t>(j & 1);
      if (!mbar_wait(k_full, ph, DEV_TIMEOUT_ATTN)) break;
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int i = 0; i < HD / 16; ++i) {
          const uint32_t off = (i >> 2) * HALF_BYTES + (i & 3) * 32;  // half of d, then 32 B per 16 d
          umma_f16_ss(tmem_base + COL_S, smem_desc_sw128(q_s + off), smem_desc_sw128(k_s + off), IDESC_S,
                      i != 0 ? 1u : 0u);
        }
        umma_commit(s_full);
        umma_commit(k_empty);
      }
      __syncwarp();
      if (!mbar_wait(p_full, ph, DEV_TIMEOUT_ATTN) || !mbar_wait(v_full, ph, DEV_TIMEOUT_ATTN)) break;
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int i = 0; i < BKV / 16; ++i) {
          // A: 16 keys of P = 8 TMEM columns; B: 16 key rows of V = 2048 B further, d halves 16 KiB apart
          umma_f16_ts(tmem_base + COL_O, tmem_base + COL_S + 8 * i, smem_desc_sw128_mn(v_s + i * 2048, HALF_BYTES),
                      IDESC_O, (j | i) != 0 ? 1u : 0u);
        }
        umma_commit(v_empty);
        if (j == n_tiles - 1) umma_commit(o_full);
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------ softmax + output (thread = query row)
    const int qd = warp & 3;  // TMEM lane quarter
    const int row = qd * 32 + lane;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(qd * 32) << 16);
    float m_ref = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const uint32_t ph = static_cast<uint32_t>(j & 1);
      if (!mbar_wait(s_full, ph, DEV_TIMEOUT_ATTN)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int keys_here = min(BKV, p.seq - j * BKV);
      const bool tail = keys_here < BKV;  // only the last tile of a ragged sequence needs key masking
      // pass 1: row maximum of this tile
      float m_tile = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t s[32];
        tmem_ld_32x32(t_row + COL_S + c * 32, s);
        tmem_ld_wait();
        if (!tail) {
          float m0 = __uint_as_float(s[0]), m1 = __uint_as_float(s[1]);
#pragma unroll
          for (int i = 2; i < 32; i += 2) {
            m0 = fmaxf(m0, __uint_as_float(s[i]));
            m1 = fmaxf(m1, __uint_as_float(s[i + 1]));
          }
          m_tile = fmaxf(m_tile, fmaxf(m0, m1));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i < keys_here) m_tile = fmaxf(m_tile, __uint_as_float(s[i]));
        }
      }
      m_tile *= p.scale_log2;
      // grow the reference maximum only when it would change the exponent range by more than 2^8
      const bool grow = m_tile > m_ref + 8.0f;
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = fmaxf(m_ref, m_tile);
        const float alpha = (m_ref == -INFINITY) ? 0.f : ex2(m_ref - m_new);
        l_sum *= alpha;
        if (j > 0) {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(t_row + COL_O + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(t_row + COL_O + c * 32, o);
          }
          tmem_st_wait();
        }
        m_ref = m_new;
      }
      // pass 2: probabilities, packed to bf16 pairs over the columns S no longer needs
      float l0 = 0.f, l1 = 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t s[32];
        tmem_ld_32x32(t_row + COL_S + c * 32, s);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float p0 = ex2(fmaf(__uint_as_float(s[2 * i]), p.scale_log2, -m_ref));
          float p1 = ex2(fmaf(__uint_as_float(s[2 * i + 1]), p.scale_log2, -m_ref));
          if (tail) {
            if (c * 32 + 2 * i >= keys_here) p0 = 0.f;
            if (c * 32 + 2 * i + 1 >= keys_here) p1 = 0.f;
          }
          l0 += p0;
          l1 += p1;
          const __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
          pk[i] = *reinterpret_cast<const uint32_t*>(&hh);
        }
        tmem_st_32x16(t_row + COL_S + c * 16, pk);
      }
      l_sum += l0 + l1;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok && mbar_wait(o_full, 0, DEV_TIMEOUT_ATTN)) {
      tc_fence_after();
      const float inv = 1.0f / l_sum;
      const int q = q0 + row;
      __nv_bfloat16* dst = p.out + b * p.out_batch_stride + static_cast<int64_t>(q) * p.out_row_stride + h * HD;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(t_row + COL_O + c * 32, o);
        tmem_ld_wait();
        if (q < p.seq) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            __nv_bfloat162 hh[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
              hh[i] = __floats2bfloat162_rn(__uint_as_float(o[g * 8 + 2 * i]) * inv,
                                            __uint_as_float(o[g * 8 + 2 * i + 1]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + g * 8) = *reinterpret_cast<uint4*>(hh);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

MFX_DEFINE_STATUS_READER(read_status)

}  // namespace fmha
}  // namespace mfx

extern "C" {

int mfx_fmha(const void* q, const void* k, const void* v, int64_t qkv_row_stride, int64_t qkv_batch_stride,
             int64_t seq, int64_t batch, int heads, float scale, void* out, int64_t out_row_stride,
             int64_t out_batch_stride, void* stream) {
  using namespace mfx;
  using namespace mfx::fmha;
  if (!q || !k || !v || !out) return MFX_ERR_NULL;
  if (seq <= 0 || batch <= 0 || heads <= 0) return MFX_ERR_SHAPE;
  if (seq > (1 << 24) || batch > 65535 || heads > 65535) return MFX_ERR_TOO_LARGE;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out) || (qkv_row_stride * 2) % 16 != 0 ||
      (qkv_batch_stride * 2) % 16 != 0 || (out_row_stride * 2) % 16 != 0 || (out_batch_stride * 2) % 16 != 0)
    return MFX_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  CUtensorMap tq, tk, tv;
  const uint64_t dims[4] = {HD, static_cast<uint64_t>(heads), static_cast<uint64_t>(seq),
                            static_cast<uint64_t>(batch)};
  const uint64_t bstride = batch > 1 ? static_cast<uint64_t>(qkv_batch_stride) * 2
                                     : static_cast<uint64_t>(qkv_row_stride) * 2 * seq;
  const uint64_t strides[3] = {HD * 2, static_cast<uint64_t>(qkv_row_stride) * 2, bstride};
  const uint32_t box[4] = {64, 1, 128, 1};
  const void* ptrs[3] = {q, k, v};
  CUtensorMap* maps[3] = {&tq, &tk, &tv};
  for (int i = 0; i < 3; ++i)
    if (int rc = encode_tmap(maps[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, ptrs[i], dims, strides, box,
                             CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  Params p;
  p.seq = static_cast<int>(seq);
  p.batch = static_cast<int>(batch);
  p.heads = heads;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out_row_stride = out_row_stride;
  p.out_batch_stride = out_batch_stride;
  static bool configured = false;
  static int configured_dev = -1;
  int dev = 0;
  MFX_CUDA_TRY(cudaGetDevice(&dev));
  if (!configured || configured_dev != dev) {
    MFX_CUDA_TRY(cudaFuncSetAttribute(fmha_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DYN_BYTES));
    configured = true;
    configured_dev = dev;
  }
  dim3 grid(static_cast<unsigned>((seq + BQ - 1) / BQ), static_cast<unsigned>(heads), static_cast<unsigned>(batch));
  fmha_kernel<<<grid, NUM_THREADS, DYN_BYTES, static_cast<cudaStream_t>(stream)>>>(tq, tk, tv, p);
  MFX_CUDA_TRY(cudaGetLastError());
  return MFX_OK;
}

}  // extern "C"
