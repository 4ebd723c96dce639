// Non-causal flash attention for head dimension 128 on tcgen05 (sm_100a).
//
// Replaces mx.fast.scaled_dot_product_attention(q, k, v, scale) as called by the reference's
// AttentionUtils.compute_attention (src/mflux/models/flux/model/flux_transformer/common/attention_utils.py:48-52),
// optionally with a per-key additive bias, keys / values of their own length and fewer key / value heads than
// query heads (the entry points at the end of the file say which reference call each shape replaces).
//
// Two kernels, chosen per call by use_pingpong(): sdpa_pair_kernel (this comment) and sdpa_pingpong_kernel (namespace
// pp below: two query tiles per CTA, one CTA per SM, for long sequences on grids that fill their last wave).
//
// sdpa_pair_kernel: one CTA = one (sample, head, 128-query tile); two CTAs share an SM. Keys go in tiles of 64 and the score tile
// S is double-buffered in tensor memory, so S of tile j+1 is computed while the softmax of tile j runs and the
// softmax warps never wait for a matmul in steady state. 384 threads:
//   warp 0     TMA producer: Q once, then K tiles of 64 keys into two stages (128-byte swizzle, two 64-wide
//              halves of d); warp 10 does the same for V
//   warp 1     allocates 256 TMEM columns (S0 | S1 | O) and issues S(t) = Q K(t)^T (both operands from shared
//              memory, K-major) into buffer t & 1 once P(t-2) V(t-2), which read that buffer, has completed
//   warp 11    issues O += P(j) V(j) (P bf16 from tensor memory, V MN-major from shared memory). Two issuing warps
//              because tcgen05.mma issue blocks while the pipe is busy: with one warp the waits and commits of one
//              kind of product delayed the other by a third of the tile time
//   warps 2-9  softmax, two warps per 32-row quarter of the tile, each owning 32 of the 64 key columns
//              (thread = query row): one tcgen05.ld of its S columns into registers, row maximum exchanged
//              with the partner warp through shared memory, running max kept stale until it would grow by
//              more than 2^8 (then O and the row sums are rescaled), exp2 (three quarters on the special-function
//              unit, one quarter as a cubic on the FMA pipe), P -> tcgen05.st over the warp's own S columns,
//              finally O / rowsum -> global (each warp its 64 columns of d)
// All waits are bounded.
#include <cuda_bf16.h>

#include <cstdlib>

#include "host_util.cuh"
#include "ptx.cuh"

namespace mfx {
namespace attn {

constexpr int BQ = 128;
constexpr int PARTS = 2;                     // softmax warps per 32-row quarter, each owning 32 key columns.
                                             // 4 (128-key tiles, all 512 TMEM columns, one CTA per SM) also works
                                             // and measured 8 % slower: nothing hides a CTA's prologue and epilogue
constexpr int BKV = 32 * PARTS;              // keys per tile
constexpr int HD = 128;
constexpr int NUM_SOFTMAX_WARPS = 4 * PARTS;
constexpr int V_PRODUCER_WARP = 2 + NUM_SOFTMAX_WARPS;
constexpr int PV_ISSUER_WARP = V_PRODUCER_WARP + 1;   // warp 1 issues S = Q K^T, this one O += P V
constexpr int NUM_THREADS = (PV_ISSUER_WARP + 1) * 32;
constexpr int CTAS_PER_SM = PARTS == 2 ? 2 : 1;
constexpr int OC = HD / PARTS;               // columns of O a softmax warp rescales and writes out
constexpr int Q_BYTES = BQ * HD * 2;        // 32 KiB: [128 rows][128 d] bf16 as two 16 KiB halves of d
constexpr int Q_HALF = Q_BYTES / 2;
constexpr int KV_BYTES = BKV * HD * 2;      // [BKV keys][128 d] as two halves of d (16 KiB for 64 keys)
constexpr int KV_HALF = KV_BYTES / 2;
constexpr uint32_t TMEM_COLS = 2 * BKV + HD <= 256 ? 256 : 512;
constexpr uint32_t COL_S = 0;    // two S buffers of BKV fp32 columns; P (bf16 pairs) of a warp's 32 keys goes over
                                 // the first 16 of the 32 S columns that warp owns
constexpr uint32_t COL_O = 2 * BKV;  // O fp32, 128 columns after the two S buffers

constexpr int OFF_Q = 0;
constexpr int OFF_K = OFF_Q + Q_BYTES;          // 2 stages
constexpr int OFF_V = OFF_K + 2 * KV_BYTES;     // 2 stages
constexpr int OFF_BAR = OFF_V + 2 * KV_BYTES;
constexpr int NUM_BARS = 14;
constexpr int OFF_TMEM = OFF_BAR + NUM_BARS * 8;
constexpr int OFF_XCH = OFF_TMEM + 16;                // float [2 parities][4 quarters][2 halves][32 rows]
constexpr int XCH_FLOATS = 4 * PARTS * 32;        // one value per softmax thread
constexpr int XCH_BYTES = 2 * XCH_FLOATS * 4;     // two buffers by tile parity
constexpr int DYN_BYTES = OFF_XCH + XCH_BYTES + 1024;

struct Params {
  int seq, batch, heads;   // seq = number of queries
  int seq_kv;              // number of keys / values (>= 1; equals seq for self-attention)
  int kv_rep;              // query heads per key/value head (1 unless grouped-query attention)
  float scale_log2;  // scale * log2(e)
  const float* key_bias;        // optional additive bias per (sample, key), added to the scaled scores
  int64_t bias_batch_stride;
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

// Packed pairs of floats in one 64-bit register: sm_100 executes add/fma on both halves in one instruction.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// max(m, all 32 values) with two independent chains of 3-input max.
__device__ __forceinline__ float max_chunk(const uint32_t (&s)[32], float m) {
  float a = m, b = __uint_as_float(s[0]);
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    a = max3(a, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
    b = max3(b, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
  }
  return fmaxf(a, b);
}

// 2^x for a pair on the FMA and integer pipes instead of the special-function unit: n = rint(x) by the
// magic-number add, 2^(x-n) by a cubic fitted on [-0.5, 0.5] (max relative error 7.5e-5, far below the bf16
// rounding the result gets), n added into the exponent field. x is clamped at -126 to keep the exponent in range.
__device__ __forceinline__ void exp2_poly2(uint64_t x2, float& p0, float& p1) {
  float x0, x1;
  unpack2(x2, x0, x1);
  x2 = pack2(fmaxf(x0, -126.f), fmaxf(x1, -126.f));
  const uint64_t magic = pack2(12582912.f, 12582912.f), nmagic = pack2(-12582912.f, -12582912.f);
  const uint64_t t2 = add2(x2, magic);
  const uint64_t n2 = add2(t2, nmagic);
  const uint64_t f2 = fma2(n2, pack2(-1.f, -1.f), x2);
  uint64_t r2 = fma2(f2, pack2(0.0551716685f, 0.0551716685f), pack2(0.2426111251f, 0.2426111251f));
  r2 = fma2(r2, f2, pack2(0.6932609677f, 0.6932609677f));
  r2 = fma2(r2, f2, pack2(0.9999280572f, 0.9999280572f));
  float t0, t1, r0, r1;
  unpack2(t2, t0, t1);
  unpack2(r2, r0, r1);
  p0 = __uint_as_float(__float_as_uint(r0) + (__float_as_uint(t0) << 23));
  p1 = __uint_as_float(__float_as_uint(r1) + (__float_as_uint(t1) << 23));
}

// Pairs (by index within a 32-column chunk) whose exponential runs on the FMA pipe; the rest use ex2 on the
// special-function unit. One pair in four balances the two pipes against the tensor pipe's time per tile.
constexpr uint32_t POLY_PAIRS = 0x8888u;

// p = 2^(s * scale - m) for 32 scores, bf16 pairs into pk, float sums into lsum2.
template <uint32_t POLY = POLY_PAIRS>
__device__ __forceinline__ void exp_chunk(const uint32_t (&s)[32], uint64_t scale2, uint64_t negm2, uint64_t& lsum2,
                                          uint32_t (&pk)[16]) {
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint64_t x2 = fma2(pack2(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1])), scale2, negm2);
    float p0, p1;
    if ((POLY >> i) & 1u) {
      exp2_poly2(x2, p0, p1);
    } else {
      float x0, x1;
      unpack2(x2, x0, x1);
      p0 = ex2(x0);
      p1 = ex2(x1);
    }
    lsum2 = add2(lsum2, pack2(p0, p1));
    const __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
    pk[i] = *reinterpret_cast<const uint32_t*>(&hh);
  }
}

// HAS_BIAS adds a per-key additive bias (a key-padding mask) to the scaled scores before the row maximum; the
// variant without it is the plain kernel, instruction for instruction.
template <bool HAS_BIAS>
__global__ void __launch_bounds__(NUM_THREADS, CTAS_PER_SM)
sdpa_pair_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
            const __grid_constant__ CUtensorMap tmap_v, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t q_s = smem_base + OFF_Q, k_s = smem_base + OFF_K, v_s = smem_base + OFF_V;
  const uint32_t bar0 = smem_base + OFF_BAR;
  // per-stage barriers are pairs: index + 8 * stage
  const uint32_t q_full = bar0, o_full = bar0 + 8, k_full = bar0 + 16, v_full = bar0 + 32,
                 v_empty = bar0 + 64, s_full = bar0 + 80, p_full = bar0 + 96;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + OFF_TMEM);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * BQ;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int n_tiles = (p.seq_kv + BKV - 1) / BKV;
  const int hk = h / p.kv_rep;   // key/value head of this query head

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(o_full, 1);
#pragma unroll
    for (int st = 0; st < 2; ++st) {
      mbar_init(k_full + 8 * st, 1);
      mbar_init(v_full + 8 * st, 1);
      mbar_init(v_empty + 8 * st, 1);
      mbar_init(s_full + 8 * st, 1);
      mbar_init(p_full + 8 * st, NUM_SOFTMAX_WARPS);
    }
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
    if (elect_one()) {
      mbar_arrive_expect_tx(q_full, Q_BYTES);
      tma_load_4d(q_s, &tmap_q, q_full, 0, h, q0, b);
      tma_load_4d(q_s + Q_HALF, &tmap_q, q_full, 64, h, q0, b);
    }
    // K stream (the V stream has its own warp): a K stage frees as soon as S of that tile is done, a V stage only
    // after the tile's P V product, and K of the next tiles must not wait behind V
    for (int j = 0; j < n_tiles; ++j) {
      const int st = j & 1;
      const uint32_t ph = static_cast<uint32_t>((j >> 1) & 1);
      // the stage is free once S of the tile that used it (j - 2) is complete: that is what s_full signals
      if (j >= 2 && !mbar_wait(s_full + 8 * st, ph ^ 1u, DEV_TIMEOUT_ATTN)) break;
      if (elect_one()) {
        mbar_arrive_expect_tx(k_full + 8 * st, KV_BYTES);
        tma_load_4d(k_s + st * KV_BYTES, &tmap_k, k_full + 8 * st, 0, hk, j * BKV, b);
        tma_load_4d(k_s + st * KV_BYTES + KV_HALF, &tmap_k, k_full + 8 * st, 64, hk, j * BKV, b);
      }
      __syncwarp();
    }
  } else if (warp == V_PRODUCER_WARP) {
    for (int j = 0; j < n_tiles; ++j) {
      const int st = j & 1;
      const uint32_t ph = static_cast<uint32_t>((j >> 1) & 1);
      if (!mbar_wait(v_empty + 8 * st, ph ^ 1u, DEV_TIMEOUT_ATTN)) break;
      if (elect_one()) {
        mbar_arrive_expect_tx(v_full + 8 * st, KV_BYTES);
        tma_load_4d(v_s + st * KV_BYTES, &tmap_v, v_full + 8 * st, 0, hk, j * BKV, b);
        tma_load_4d(v_s + st * KV_BYTES + KV_HALF, &tmap_v, v_full + 8 * st, 64, hk, j * BKV, b);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ issuer of S(t) = Q K(t)^T into S buffer t & 1
    // Two issuing warps, so that the barrier waits and commits of one kind of product do not hold up the other.
    // S(t) overwrites the buffer that held P(t-2): it waits for the completion of P(t-2) V(t-2), which the other
    // issuer commits to v_empty.
    constexpr uint32_t IDESC_S = make_idesc(FMT_BF16, FMT_BF16, BQ, BKV);       // K-major x K-major
    bool ok = mbar_wait(q_full, 0, DEV_TIMEOUT_ATTN);
    for (int t = 0; t < n_tiles && ok; ++t) {
      const int st = t & 1;
      const uint32_t ph = static_cast<uint32_t>((t >> 1) & 1);
      if (!mbar_wait(k_full + 8 * st, ph, DEV_TIMEOUT_ATTN)) break;
      if (t >= 2 && !mbar_wait(v_empty + 8 * st, ph ^ 1u, DEV_TIMEOUT_ATTN)) break;
      tc_fence_after();
      if (elect_one()) {
        // descriptors of the tiles' first bytes; a step adds its byte offset >> 4 to the start-address field
        const uint64_t q_desc = smem_desc_sw128(q_s), k_desc = smem_desc_sw128(k_s + st * KV_BYTES);
#pragma unroll
        for (int i = 0; i < HD / 16; ++i) {
          // half of d, then 32 B per 16 d inside the 128-byte rows
          const uint32_t qoff = (i >> 2) * Q_HALF + (i & 3) * 32, koff = (i >> 2) * KV_HALF + (i & 3) * 32;
          umma_f16_ss(tmem_base + COL_S + BKV * st, q_desc + (qoff >> 4), k_desc + (koff >> 4), IDESC_S,
                      i != 0 ? 1u : 0u);
        }
        umma_commit(s_full + 8 * st);
      }
      __syncwarp();
    }
  } else if (warp == PV_ISSUER_WARP) {
    // ------------------------------------------------------------ issuer of O += P(j) V(j)
    constexpr uint32_t IDESC_O = make_idesc_b_mn(FMT_BF16, FMT_BF16, BQ, HD);   // P (TMEM) x V (MN-major)
    for (int j = 0; j < n_tiles; ++j) {
      const int st = j & 1;
      const uint32_t ph = static_cast<uint32_t>((j >> 1) & 1);
      if (!mbar_wait(p_full + 8 * st, ph, DEV_TIMEOUT_ATTN) || !mbar_wait(v_full + 8 * st, ph, DEV_TIMEOUT_ATTN))
        break;
      tc_fence_after();
      if (elect_one()) {
        const uint64_t v_desc = smem_desc_sw128_mn(v_s + st * KV_BYTES, KV_HALF);
#pragma unroll
        for (int i = 0; i < BKV / 16; ++i) {
          // A: 16 keys of P = 8 TMEM columns (the 32 keys of softmax part p at columns 32 p .. 32 p + 15 of the
          // buffer); B: 16 key rows of V = 2048 B further, d halves KV_HALF apart
          umma_f16_ts(tmem_base + COL_O, tmem_base + COL_S + BKV * st + (i >> 1) * 32 + 8 * (i & 1),
                      v_desc + (i * 2048 >> 4), IDESC_O, (j | i) != 0 ? 1u : 0u);
        }
        umma_commit(v_empty + 8 * st);
        if (j == n_tiles - 1) umma_commit(o_full);
      }
      __syncwarp();
    }
  } else if (warp >= 2 && warp < V_PRODUCER_WARP) {
    // ------------------------------------------------------------ softmax + output (thread = query row)
    const int qd = warp & 3;          // TMEM lane quarter this warp may access
    const int pt = (warp - 2) >> 2;   // which 32 of the tile's key columns (and which OC columns of d at the end)
    const int row = qd * 32 + lane;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(qd * 32) << 16);
    const uint32_t t_o = t_row + COL_O + pt * OC;   // own O columns
    float* xch = reinterpret_cast<float*>(smem_gen + OFF_XCH);
    const int xch_row = qd * PARTS * 32 + lane;   // + 32 * part
    float m_ref = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int st = j & 1;
      const uint32_t ph = static_cast<uint32_t>((j >> 1) & 1);
      if (!mbar_wait(s_full + 8 * st, ph, DEV_TIMEOUT_ATTN)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_s = t_row + COL_S + BKV * st + 32 * pt;   // own S columns; own P goes over the first 16
      const int keys_here = min(BKV, p.seq_kv - j * BKV) - pt * 32;  // valid keys among this warp's 32 columns
      const bool tail = keys_here < 32;  // only the last tile of a ragged sequence needs key masking
      uint32_t sA[32];
      tmem_ld_32x32(t_s, sA);
      tmem_ld_fence(sA);
      if constexpr (HAS_BIAS) {
        // scores become s * scale * log2(e) + bias * log2(e) here; everything after works on them with scale 1.
        // All threads of the warp read the same 32 bias values (one transaction per load).
        constexpr float LOG2E = 1.4426950408889634f;
        const int k0 = j * BKV + pt * 32;
        const float* bp = p.key_bias + b * p.bias_batch_stride + k0;
        if (!tail) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 bv = __ldg(reinterpret_cast<const float4*>(bp) + i);
            sA[4 * i + 0] = __float_as_uint(fmaf(__uint_as_float(sA[4 * i + 0]), p.scale_log2, bv.x * LOG2E));
            sA[4 * i + 1] = __float_as_uint(fmaf(__uint_as_float(sA[4 * i + 1]), p.scale_log2, bv.y * LOG2E));
            sA[4 * i + 2] = __float_as_uint(fmaf(__uint_as_float(sA[4 * i + 2]), p.scale_log2, bv.z * LOG2E));
            sA[4 * i + 3] = __float_as_uint(fmaf(__uint_as_float(sA[4 * i + 3]), p.scale_log2, bv.w * LOG2E));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float bv = i < keys_here ? __ldg(bp + i) : 0.f;
            sA[i] = __float_as_uint(fmaf(__uint_as_float(sA[i]), p.scale_log2, bv * LOG2E));
          }
        }
      }
      const float sc = HAS_BIAS ? 1.0f : p.scale_log2;
      float m_mine;
      if (!tail) {
        m_mine = max_chunk(sA, -INFINITY);
      } else {
        m_mine = -INFINITY;
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (i < keys_here) m_mine = fmaxf(m_mine, __uint_as_float(sA[i]));
      }
      // the partner warp holds the other 32 columns of the same rows: swap maxima (two buffers by tile parity;
      // the barrier per tile keeps the two warps at most one tile apart)
      xch[st * XCH_FLOATS + xch_row + 32 * pt] = m_mine;
      named_bar_sync(1 + qd, 32 * PARTS);
      float m_all = m_mine;
#pragma unroll
      for (int o = 0; o < PARTS; ++o) m_all = fmaxf(m_all, xch[st * XCH_FLOATS + xch_row + 32 * o]);
      const float m_tile = m_all * sc;
      // grow the reference maximum only when it would change the exponent range by more than 2^8; both warps
      // of a quarter see the same maxima and take the same branch, each rescaling its own half of O
      const bool grow = m_tile > m_ref + 8.0f;
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = fmaxf(m_ref, m_tile);
        const float alpha = (m_ref == -INFINITY) ? 0.f : ex2(m_ref - m_new);
        l_sum *= alpha;
        if (j > 0) {
          // O still receives P(j-1) V(j-1): wait until that product has finished (its commit frees the V stage)
          if (!mbar_wait(v_empty + 8 * (st ^ 1), static_cast<uint32_t>(((j - 1) >> 1) & 1), DEV_TIMEOUT_ATTN)) {
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < OC / 16; ++c) {
            uint32_t o[16];
            tmem_ld_32x16(t_o + c * 16, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x16(t_o + c * 16, o);
          }
          tmem_st_wait();
        }
        m_ref = m_new;
      }
      // probabilities from the registers, packed to bf16 pairs over this warp's own (already read) S columns
      uint64_t l2 = pack2(0.f, 0.f);
      uint32_t pk[16];
      if (!tail) {
        exp_chunk(sA, pack2(sc, sc), pack2(-m_ref, -m_ref), l2, pk);
      } else {
        float l0 = 0.f, l1 = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float p0 = ex2(fmaf(__uint_as_float(sA[2 * i]), sc, -m_ref));
          float p1 = ex2(fmaf(__uint_as_float(sA[2 * i + 1]), sc, -m_ref));
          if (2 * i >= keys_here) p0 = 0.f;
          if (2 * i + 1 >= keys_here) p1 = 0.f;
          l0 += p0;
          l1 += p1;
          const __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
          pk[i] = *reinterpret_cast<const uint32_t*>(&hh);
        }
        l2 = pack2(l0, l1);
      }
      tmem_st_32x16(t_s, pk);
      float l0, l1;
      unpack2(l2, l0, l1);
      l_sum += l0 + l1;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full + 8 * st);
    }
    if (ok && mbar_wait(o_full, 0, DEV_TIMEOUT_ATTN)) {
      tc_fence_after();
      // total row sum = this warp's part + the partner's
      const int ph = n_tiles & 1;
      xch[ph * XCH_FLOATS + xch_row + 32 * pt] = l_sum;
      named_bar_sync(1 + qd, 32 * PARTS);
      float l_all = 0.f;
#pragma unroll
      for (int o = 0; o < PARTS; ++o) l_all += xch[ph * XCH_FLOATS + xch_row + 32 * o];
      const float inv = 1.0f / l_all;
      const int q = q0 + row;
      __nv_bfloat16* dst = p.out + b * p.out_batch_stride + static_cast<int64_t>(q) * p.out_row_stride + h * HD +
                           pt * OC;
#pragma unroll 1
      for (int c = 0; c < OC / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(t_o + c * 32, o);
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


// ------------------------------------------------------------------------------------------------------------
// Ping-pong variant: one CTA per SM works on two 128-query tiles of the same (sample, head) against the same
// stream of 128-key tiles. Tensor memory holds S0 | S1 | O0 | O1 (4 x 128 columns). The products are issued in the
// order P0(j) V(j), S0(j+1) = Q0 K(j+1)^T, P1(j) V(j), S1(j+1): while the softmax of one query tile runs, the
// tensor pipe works for the other, and because the pipe executes one thread's products in order, S_t(j+1) may
// overwrite the columns P_t(j) occupied without a wait. 576 threads:
//   warps 0-15 softmax: warp = 8 * tile + 4 * half + quarter. Two threads per query row, one per 64-key half of
//              the tile: scores of the half in registers, row maximum swapped with the partner through shared
//              memory, stale running maximum, exponentials split between the special-function unit and an
//              FMA-pipe cubic, P as bf16 pairs over the first 32 columns of the thread's own S half, the rare
//              rescale of O and the final O / rowsum -> global (each thread 64 columns of d). Four softmax warps
//              per scheduler: one warp alone issues an instruction every third clock.
//   warp 16    TMA producer: both Q tiles and K(0) once, then the pairs {V(j), K(j+1)} through two 64 KiB slots
//              (one barrier wait per pair on the issuing side; K(0) borrows the K half of slot 1)
//   warp 17    allocates the 512 columns and issues every product
namespace pp {

constexpr int BK = 128;                       // keys per tile
constexpr int NUM_SM_WARPS = 16;
constexpr int PRODUCER_WARP = NUM_SM_WARPS, ISSUER_WARP = NUM_SM_WARPS + 1;
constexpr int NT = (ISSUER_WARP + 1) * 32;
constexpr int SLOTS = 2;                      // ring slots of 64 KiB: V(j) and K(j+1) travel together
#ifndef MFX_PP_POLY
#define MFX_PP_POLY 0x8888u
#endif
constexpr uint32_t PP_POLY = MFX_PP_POLY;   // pairs of a 32-key chunk whose exponential runs on the FMA pipe
constexpr int TILE_BYTES = 128 * HD * 2;      // 32 KiB, two 16 KiB halves of d, for a Q tile and for a K or V tile
constexpr int TILE_HALF = TILE_BYTES / 2;
constexpr uint32_t COL_S0 = 0, COL_O0 = 256;  // + 128 for the second query tile
constexpr int OFF_Q2 = 0;
constexpr int OFF_KV = OFF_Q2 + 2 * TILE_BYTES;
constexpr int OFF_BAR2 = OFF_KV + SLOTS * 2 * TILE_BYTES;
constexpr int NUM_BARS2 = 1 + 2 * SLOTS + 7;
constexpr int OFF_TMEM2 = OFF_BAR2 + NUM_BARS2 * 8;
constexpr int OFF_XCH2 = (OFF_TMEM2 + 16 + 15) / 16 * 16;   // float [2 parities][2 tiles][4 quarters][2 halves][32 rows]
constexpr int XCH2_FLOATS = 2 * 4 * 2 * 32;
constexpr int DYN_BYTES2 = OFF_XCH2 + 2 * XCH2_FLOATS * 4 + 1024;
static_assert(DYN_BYTES2 <= 227 * 1024, "shared memory of the ping-pong kernel");

// scores -> s * scale * log2(e) + bias * log2(e) for one 32-key chunk starting at key k0 (keys < `valid` exist)
__device__ __forceinline__ void add_bias_chunk(uint32_t (&s)[32], const float* bp, int valid, float scale_log2) {
  constexpr float LOG2E = 1.4426950408889634f;
  if (valid >= 32) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4 bv = __ldg(reinterpret_cast<const float4*>(bp) + i);
      s[4 * i + 0] = __float_as_uint(fmaf(__uint_as_float(s[4 * i + 0]), scale_log2, bv.x * LOG2E));
      s[4 * i + 1] = __float_as_uint(fmaf(__uint_as_float(s[4 * i + 1]), scale_log2, bv.y * LOG2E));
      s[4 * i + 2] = __float_as_uint(fmaf(__uint_as_float(s[4 * i + 2]), scale_log2, bv.z * LOG2E));
      s[4 * i + 3] = __float_as_uint(fmaf(__uint_as_float(s[4 * i + 3]), scale_log2, bv.w * LOG2E));
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float bv = i < valid ? __ldg(bp + i) : 0.f;
      s[i] = __float_as_uint(fmaf(__uint_as_float(s[i]), scale_log2, bv * LOG2E));
    }
  }
}

// keys past the end of the sequence get a score of -inf (weight 0)
__device__ __forceinline__ void mask_chunk(uint32_t (&s)[32], int valid) {
#pragma unroll
  for (int i = 0; i < 32; ++i)
    if (i >= valid) s[i] = __float_as_uint(-INFINITY);
}

template <bool HAS_BIAS>
__global__ void __launch_bounds__(NT, 1)
sdpa_pingpong_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t q_s = smem_base + OFF_Q2, kv_s = smem_base + OFF_KV;
  const uint32_t bar0 = smem_base + OFF_BAR2;
  const uint32_t q_full = bar0, kv_full = bar0 + 8, kv_empty = kv_full + 8 * SLOTS, s_full = kv_empty + 8 * SLOTS,
                 p_first = s_full + 16, p_full = p_first + 16, o_full = p_full + 16;   // s_full, p_first, p_full: per query tile
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + OFF_TMEM2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * (2 * BQ);
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  const int n_tiles = (p.seq_kv + BK - 1) / BK;
  const int hk = h / p.kv_rep;   // key/value head of this query head
  const bool two = q0 + BQ < p.seq;   // the last block of a sequence may hold one query tile only

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
#pragma unroll
    for (int i = 0; i < SLOTS; ++i) {
      mbar_init(kv_full + 8 * i, 1);
      mbar_init(kv_empty + 8 * i, 1);
    }
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      mbar_init(s_full + 8 * t, 1);
      mbar_init(p_first + 8 * t, 8);
      mbar_init(p_full + 8 * t, 8);
    }
    mbar_init(o_full, 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == ISSUER_WARP) {
    tmem_alloc(smem_base + OFF_TMEM2, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == PRODUCER_WARP) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      mbar_arrive_expect_tx(q_full, (two ? 2 : 1) * TILE_BYTES);
      for (int t = 0; t < (two ? 2 : 1); ++t) {
        tma_load_4d(q_s + t * TILE_BYTES, &tmap_q, q_full, 0, h, q0 + t * BQ, b);
        tma_load_4d(q_s + t * TILE_BYTES + TILE_HALF, &tmap_q, q_full, 64, h, q0 + t * BQ, b);
      }
    }
    __syncwarp();
    // K(0) into the K half of slot 1, then pair j = {V(j), K(j+1)} into slot j & 1. Slot 1 therefore completes
    // one phase more than slot 0 at the same pair index.
    if (elect_one()) {
      mbar_arrive_expect_tx(kv_full + 8, TILE_BYTES);
      tma_load_4d(kv_s + 3 * TILE_BYTES, &tmap_k, kv_full + 8, 0, hk, 0, b);
      tma_load_4d(kv_s + 3 * TILE_BYTES + TILE_HALF, &tmap_k, kv_full + 8, 64, hk, 0, b);
    }
    __syncwarp();
    for (int j = 0; j < n_tiles; ++j) {
      const int slot = j & 1;
      const int use = (j >> 1) + slot;          // how often the slot was filled before
      if (use >= 1 && !mbar_wait(kv_empty + 8 * slot, static_cast<uint32_t>((use - 1) & 1), DEV_TIMEOUT_ATTN)) break;
      if (elect_one()) {
        const bool more = j + 1 < n_tiles;
        const uint32_t dst = kv_s + slot * 2 * TILE_BYTES;
        mbar_arrive_expect_tx(kv_full + 8 * slot, (more ? 2 : 1) * TILE_BYTES);
        tma_load_4d(dst, &tmap_v, kv_full + 8 * slot, 0, hk, j * BK, b);
        tma_load_4d(dst + TILE_HALF, &tmap_v, kv_full + 8 * slot, 64, hk, j * BK, b);
        if (more) {
          tma_load_4d(dst + TILE_BYTES, &tmap_k, kv_full + 8 * slot, 0, hk, (j + 1) * BK, b);
          tma_load_4d(dst + TILE_BYTES + TILE_HALF, &tmap_k, kv_full + 8 * slot, 64, hk, (j + 1) * BK, b);
        }
      }
      __syncwarp();
    }
  } else if (warp == ISSUER_WARP) {
    // ------------------------------------------------------------ issuer of every product
    // Order P0(j) V(j), S0(j+1), P1(j) V(j), S1(j+1). The commit after S_t(j+1) also covers P_t(j) V(j): a softmax
    // warp that sees S_t(j+1) may rescale O_t. P V starts once the first 32 keys of both halves of P are stored.
    // The whole warp runs the loop and its waits; elect_one() picks the issuing thread per block of products.
    // (A region guarded by `lane == 0` is divergent code to the compiler: operands are then built in vector
    // registers and moved to uniform registers one product at a time, and that instruction chain starves behind
    // the softmax warps of the same scheduler: 90-110 clocks per product instead of 64.)
    constexpr uint32_t IDESC_S = make_idesc(FMT_BF16, FMT_BF16, BQ, BK);        // K-major x K-major
    constexpr uint32_t IDESC_O = make_idesc_b_mn(FMT_BF16, FMT_BF16, BQ, HD);   // P (TMEM) x V (MN-major)
    // Descriptors of the tiles' first bytes; a step inside a tile adds its byte offset >> 4 to the start-address
    // field (no carry out of it: every tile lies inside the 256 KiB the field spans), one add per operand instead
    // of rebuilding the descriptor for every product.
    const uint64_t q_desc0 = smem_desc_sw128(q_s), q_desc1 = smem_desc_sw128(q_s + TILE_BYTES);
    // S_t = Q_t K^T (called by the elected thread)
    auto issue_s = [&](int t, uint64_t k_desc) {
      const uint64_t q_desc = t ? q_desc1 : q_desc0;
#pragma unroll
      for (int i = 0; i < HD / 16; ++i) {
        const uint32_t off = ((i >> 2) * TILE_HALF + (i & 3) * 32) >> 4;   // half of d, then 32 B per 16 d
        umma_f16_ss(tmem_base + COL_S0 + 128 * t, q_desc + off, k_desc + off, IDESC_S, i != 0 ? 1u : 0u);
      }
      umma_commit(s_full + 8 * t);
    };
    // One part of P_t(j) V(j) (called by the elected thread). A = 16 keys of P = 8 columns of bf16 pairs (each
    // 64-key half of P lies over the first 32 columns of its own half of S); B = 16 key rows of V, 2048 B per 16
    // keys, d halves TILE_HALF apart. Part 0 = the first 32 keys of either half (what every softmax thread stores
    // first).
    auto issue_pv_part = [&](int t, int part, uint64_t v_desc, bool first_tile) {
#pragma unroll
      for (int ii = 0; ii < BK / 32; ++ii) {
        const int i = (ii >> 1) * 4 + part * 2 + (ii & 1);   // 16-key groups 0,1,4,5 or 2,3,6,7
        umma_f16_ts(tmem_base + COL_O0 + 128 * t, tmem_base + COL_S0 + 128 * t + 64 * (i >> 2) + 8 * (i & 3),
                    v_desc + (i * 2048 >> 4), IDESC_O, (first_tile && part == 0 && ii == 0) ? 0u : 1u);
      }
    };
    bool ok = mbar_wait(q_full, 0, DEV_TIMEOUT_ATTN) && mbar_wait(kv_full + 8, 0, DEV_TIMEOUT_ATTN);
    if (ok) {
      tc_fence_after();
      if (elect_one()) {
        issue_s(0, smem_desc_sw128(kv_s + 3 * TILE_BYTES));
        if (two) issue_s(1, smem_desc_sw128(kv_s + 3 * TILE_BYTES));
        umma_commit(kv_empty + 8);
      }
      __syncwarp();
    }
    for (int j = 0; j < n_tiles && ok; ++j) {
      const uint32_t ph = static_cast<uint32_t>(j & 1);
      const bool more = j + 1 < n_tiles;
      const int slot = j & 1;
      // every scalar step here costs the issuing warp 25-170 clocks while the pipe holds ~300 clocks of queued
      // products: one barrier per operand pair, one elected region per wait
      if (!mbar_wait_ready(kv_full + 8 * slot, static_cast<uint32_t>(((j >> 1) + slot) & 1), DEV_TIMEOUT_ATTN)) break;
      const uint64_t vaddr = smem_desc_sw128_mn(kv_s + slot * 2 * TILE_BYTES, TILE_HALF);
      const uint64_t kaddr = smem_desc_sw128(kv_s + slot * 2 * TILE_BYTES + TILE_BYTES);
      if (!mbar_wait_ready(p_first, ph, DEV_TIMEOUT_ATTN)) break;
      tc_fence_after();
      if (elect_one()) issue_pv_part(0, 0, vaddr, j == 0);
      __syncwarp();   // the other lanes must not poll the next barrier in between the elected lane's products
      if (!mbar_wait(p_full, ph, DEV_TIMEOUT_ATTN)) break;
      tc_fence_after();
      if (elect_one()) {
        issue_pv_part(0, 1, vaddr, false);
        if (more) issue_s(0, kaddr);
        if (!two) umma_commit(more ? kv_empty + 8 * slot : o_full);
      }
      __syncwarp();
      if (two) {
        if (!mbar_wait_ready(p_first + 8, ph, DEV_TIMEOUT_ATTN)) break;
        tc_fence_after();
        if (elect_one()) issue_pv_part(1, 0, vaddr, j == 0);
        __syncwarp();
        if (!mbar_wait(p_full + 8, ph, DEV_TIMEOUT_ATTN)) break;
        tc_fence_after();
        if (elect_one()) {
          issue_pv_part(1, 1, vaddr, false);
          if (more) issue_s(1, kaddr);
          umma_commit(more ? kv_empty + 8 * slot : o_full);
        }
        __syncwarp();
      }
    }
  } else if (warp < 8 || two) {
    // ------------------------------------------------------------ softmax + output (two threads per query row)
    const int t = warp >> 3;          // query tile
    const int hf = (warp >> 2) & 1;   // which 64 of the tile's 128 keys (and which 64 columns of d at the end)
    const int qd = warp & 3;          // TMEM lane quarter this warp may access
    const int row = qd * 32 + lane;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(qd * 32) << 16);
    const uint32_t t_s = t_row + COL_S0 + 128 * t + 64 * hf;   // own S columns; own P goes over the first 32
    const uint32_t t_o = t_row + COL_O0 + 128 * t + 64 * hf;   // own O columns
    const uint32_t my_s_full = s_full + 8 * t, my_p_first = p_first + 8 * t, my_p_full = p_full + 8 * t;
    float* xch = reinterpret_cast<float*>(smem_gen + OFF_XCH2);
    const int xch_mine = ((t * 4 + qd) * 2 + hf) * 32 + lane, xch_other = ((t * 4 + qd) * 2 + (hf ^ 1)) * 32 + lane;
    const uint32_t pair_bar = 1 + t * 4 + qd;   // named barrier of the two warps that share these rows
    const float sc = HAS_BIAS ? 1.0f : p.scale_log2;
    float m_ref = -INFINITY, l_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      if (!mbar_wait(my_s_full, static_cast<uint32_t>(j & 1), DEV_TIMEOUT_ATTN)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t sa[32], sb[32];
      tmem_ld_32x32(t_s, sa);
      tmem_ld_32x32(t_s + 32, sb);
      tmem_ld_fence(sa);
      tmem_ld_fence(sb);
      const int keys_here = p.seq_kv - j * BK - 64 * hf;   // >= 64 except on the last tile of a ragged sequence
      if constexpr (HAS_BIAS) {
        const float* bp = p.key_bias + b * p.bias_batch_stride + j * BK + 64 * hf;
        add_bias_chunk(sa, bp, keys_here, p.scale_log2);
        add_bias_chunk(sb, bp + 32, keys_here - 32, p.scale_log2);
      }
      if (keys_here < 64) {
        mask_chunk(sa, keys_here);
        mask_chunk(sb, keys_here - 32);
      }
      const float m_mine = fmaxf(max_chunk(sa, -INFINITY), max_chunk(sb, -INFINITY));
      // the partner warp holds the other 64 keys of the same rows: swap maxima (two buffers by tile parity; the
      // barrier per tile keeps the two warps at most one tile apart)
      float* x = xch + (j & 1) * XCH2_FLOATS;
      x[xch_mine] = m_mine;
      named_bar_sync(pair_bar, 64);
      const float m_tile = fmaxf(m_mine, x[xch_other]) * sc;
      // grow the reference maximum only when it would change the exponent range by more than 2^8; both warps of
      // a row see the same maxima and take the same branch, each rescaling its own half of O
      const bool grow = m_tile > m_ref + 8.0f;
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = fmaxf(m_ref, m_tile);
        const float alpha = (m_ref == -INFINITY) ? 0.f : ex2(m_ref - m_new);
        l_sum *= alpha;
        if (j > 0) {
          // P(j-1) V(j-1) has finished: the commit that announced S(j) was issued after it by the same thread
#pragma unroll 1
          for (int c = 0; c < 64 / 16; ++c) {
            uint32_t o[16];
            tmem_ld_32x16(t_o + c * 16, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x16(t_o + c * 16, o);
          }
          tmem_st_wait();
        }
        m_ref = m_new;
      }
      const uint64_t scale2 = pack2(sc, sc), negm2 = pack2(-m_ref, -m_ref);
      uint64_t la = pack2(0.f, 0.f), lb = pack2(0.f, 0.f);
      uint32_t pk[16];
      exp_chunk<PP_POLY>(sa, scale2, negm2, la, pk);
      tmem_st_32x16(t_s, pk);
      // P V can start on the first 32 keys of both halves
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(my_p_first);
      exp_chunk<PP_POLY>(sb, scale2, negm2, lb, pk);
      tmem_st_32x16(t_s + 16, pk);
      float l0, l1;
      unpack2(add2(la, lb), l0, l1);
      l_sum += l0 + l1;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(my_p_full);
    }
    if (ok && mbar_wait(o_full, 0, DEV_TIMEOUT_ATTN)) {
      tc_fence_after();
      // total row sum = this thread's half + the partner's
      float* x = xch + (n_tiles & 1) * XCH2_FLOATS;
      x[xch_mine] = l_sum;
      named_bar_sync(pair_bar, 64);
      const float inv = 1.0f / (l_sum + x[xch_other]);
      const int q = q0 + t * BQ + row;
      __nv_bfloat16* dst = p.out + b * p.out_batch_stride + static_cast<int64_t>(q) * p.out_row_stride + h * HD +
                           64 * hf;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(t_o + c * 32, o);
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
  if (warp == ISSUER_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace pp

MFX_DEFINE_STATUS_READER(read_status)

}  // namespace attn
}  // namespace mfx

namespace mfx {
namespace attn {

// Which kernel serves a call. The ping-pong kernel (two query tiles per CTA, one CTA per SM) is the faster main
// loop (1245-1270 against 1150-1170 TFLOP/s at 16 x 24 heads x 4608 tokens), but its work items are twice as
// large: it is chosen from 1024 keys on, and only if the last wave of CTAs leaves at most 7 % of the SMs' time
// unused (2 x 24 heads x 7145 tokens is 9.08 waves of 148 = 91 %: 1091 against 1158 TFLOP/s, the other kernel wins).
// MFX_FMHA_KERNEL=pingpong | pair overrides the choice.
static bool use_pingpong(int64_t seq, int64_t seq_kv, int64_t batch, int heads) {
  const char* e = getenv("MFX_FMHA_KERNEL");
  if (e && e[0] == 'p' && e[1] == 'i') return true;
  if (e && e[0] == 'p' && e[1] == 'a') return false;
  if (seq_kv < 1024) return false;
  const int64_t ctas = (seq + 2 * BQ - 1) / (2 * BQ) * heads * batch;
  const int64_t sms = device_sm_count();
  const int64_t waves = (ctas + sms - 1) / sms;
  return ctas * 100 >= waves * sms * 93;
}

// Arguments of one attention call (the C entry points fill it).
struct Call {
  const void *q, *k, *v;
  int64_t q_row_stride, q_batch_stride, kv_row_stride, kv_batch_stride;   // elements
  int64_t seq, seq_kv, batch;
  int heads, kv_heads;
  float scale;
  const float* key_bias;
  int64_t bias_batch_stride;
  void* out;
  int64_t out_row_stride, out_batch_stride;
};

int run(const Call& c, cudaStream_t stream) {
  const void *q = c.q, *k = c.k, *v = c.v;
  void* out = c.out;
  const int64_t seq = c.seq, seq_kv = c.seq_kv, batch = c.batch;
  const int heads = c.heads;
  const float* key_bias = c.key_bias;
  const int64_t bias_batch_stride = c.bias_batch_stride, out_row_stride = c.out_row_stride,
                out_batch_stride = c.out_batch_stride;
  if (!q || !k || !v || !out) return MFX_ERR_NULL;
  if (seq <= 0 || seq_kv <= 0 || batch <= 0 || heads <= 0 || c.kv_heads <= 0 || heads % c.kv_heads != 0)
    return MFX_ERR_SHAPE;
  if (seq > (1 << 24) || seq_kv > (1 << 24) || batch > 65535 || heads > 65535) return MFX_ERR_TOO_LARGE;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out) || (c.q_row_stride * 2) % 16 != 0 ||
      (c.q_batch_stride * 2) % 16 != 0 || (c.kv_row_stride * 2) % 16 != 0 || (c.kv_batch_stride * 2) % 16 != 0 ||
      (out_row_stride * 2) % 16 != 0 || (out_batch_stride * 2) % 16 != 0)
    return MFX_ERR_ALIGN;
  if (key_bias) {
    // the kernel reads the bias of 32 consecutive keys as eight 16-byte vectors
    if (!aligned16(key_bias) || (batch > 1 && (bias_batch_stride * 4) % 16 != 0)) return MFX_ERR_ALIGN;
    if (batch > 1 && bias_batch_stride < seq_kv) return MFX_ERR_SHAPE;
  }
  if (int rc = check_arch()) return rc;
  CUtensorMap tq, tk, tv;
  const uint64_t dims_q[4] = {HD, static_cast<uint64_t>(heads), static_cast<uint64_t>(seq),
                              static_cast<uint64_t>(batch)};
  const uint64_t dims_kv[4] = {HD, static_cast<uint64_t>(c.kv_heads), static_cast<uint64_t>(seq_kv),
                               static_cast<uint64_t>(batch)};
  const uint64_t strides_q[3] = {HD * 2, static_cast<uint64_t>(c.q_row_stride) * 2,
                                 batch > 1 ? static_cast<uint64_t>(c.q_batch_stride) * 2
                                           : static_cast<uint64_t>(c.q_row_stride) * 2 * seq};
  const uint64_t strides_kv[3] = {HD * 2, static_cast<uint64_t>(c.kv_row_stride) * 2,
                                  batch > 1 ? static_cast<uint64_t>(c.kv_batch_stride) * 2
                                            : static_cast<uint64_t>(c.kv_row_stride) * 2 * seq_kv};
  const bool pingpong = use_pingpong(seq, seq_kv, batch, heads);
  const uint32_t box_q[4] = {64, 1, BQ, 1}, box_kv[4] = {64, 1, static_cast<uint32_t>(pingpong ? pp::BK : BKV), 1};
  const void* ptrs[3] = {q, k, v};
  CUtensorMap* maps[3] = {&tq, &tk, &tv};
  for (int i = 0; i < 3; ++i)
    if (int rc = encode_tmap(maps[i], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, ptrs[i], i == 0 ? dims_q : dims_kv,
                             i == 0 ? strides_q : strides_kv, i == 0 ? box_q : box_kv, CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  const float scale = c.scale;
  Params p;
  p.seq = static_cast<int>(seq);
  p.seq_kv = static_cast<int>(seq_kv);
  p.kv_rep = heads / c.kv_heads;
  p.batch = static_cast<int>(batch);
  p.heads = heads;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.key_bias = key_bias;
  p.bias_batch_stride = batch > 1 ? bias_batch_stride : 0;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.out_row_stride = out_row_stride;
  p.out_batch_stride = out_batch_stride;
  if (pingpong) {
    dim3 grid(static_cast<unsigned>((seq + 2 * BQ - 1) / (2 * BQ)), static_cast<unsigned>(heads),
              static_cast<unsigned>(batch));
    if (key_bias) {
      static SmemConfigured configured;
      if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(pp::sdpa_pingpong_kernel<true>),
                                       pp::DYN_BYTES2, configured))
        return rc;
      pp::sdpa_pingpong_kernel<true><<<grid, pp::NT, pp::DYN_BYTES2, stream>>>(tq, tk, tv, p);
    } else {
      static SmemConfigured configured;
      if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(pp::sdpa_pingpong_kernel<false>),
                                       pp::DYN_BYTES2, configured))
        return rc;
      pp::sdpa_pingpong_kernel<false><<<grid, pp::NT, pp::DYN_BYTES2, stream>>>(tq, tk, tv, p);
    }
    MFX_CUDA_TRY(cudaGetLastError());
    return MFX_OK;
  }
  dim3 grid(static_cast<unsigned>((seq + BQ - 1) / BQ), static_cast<unsigned>(heads), static_cast<unsigned>(batch));
  if (key_bias) {
    static SmemConfigured configured;
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(sdpa_pair_kernel<true>), DYN_BYTES, configured))
      return rc;
    sdpa_pair_kernel<true><<<grid, NUM_THREADS, DYN_BYTES, stream>>>(tq, tk, tv, p);
  } else {
    static SmemConfigured configured;
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(sdpa_pair_kernel<false>), DYN_BYTES, configured))
      return rc;
    sdpa_pair_kernel<false><<<grid, NUM_THREADS, DYN_BYTES, stream>>>(tq, tk, tv, p);
  }
  MFX_CUDA_TRY(cudaGetLastError());
  return MFX_OK;
}

}  // namespace attn
}  // namespace mfx

extern "C" {

int mfx_fmha(const void* q, const void* k, const void* v, int64_t qkv_row_stride, int64_t qkv_batch_stride,
             int64_t seq, int64_t batch, int heads, float scale, void* out, int64_t out_row_stride,
             int64_t out_batch_stride, void* stream) {
  const mfx::attn::Call c{q, k, v, qkv_row_stride, qkv_batch_stride, qkv_row_stride, qkv_batch_stride, seq, seq, batch,
                          heads, heads, scale, nullptr, 0, out, out_row_stride, out_batch_stride};
  return mfx::attn::run(c, static_cast<cudaStream_t>(stream));
}

int mfx_fmha_bias(const void* q, const void* k, const void* v, int64_t qkv_row_stride, int64_t qkv_batch_stride,
                  int64_t seq, int64_t batch, int heads, float scale, const float* key_bias,
                  int64_t bias_batch_stride, void* out, int64_t out_row_stride, int64_t out_batch_stride,
                  void* stream) {
  if (!key_bias) return MFX_ERR_NULL;
  const mfx::attn::Call c{q, k, v, qkv_row_stride, qkv_batch_stride, qkv_row_stride, qkv_batch_stride, seq, seq, batch,
                          heads, heads, scale, key_bias, bias_batch_stride, out, out_row_stride, out_batch_stride};
  return mfx::attn::run(c, static_cast<cudaStream_t>(stream));
}

int mfx_fmha_ex(const mfx_fmha_args* a, void* stream) {
  if (!a) return MFX_ERR_NULL;
  const mfx::attn::Call c{a->q, a->k, a->v, a->q_row_stride, a->q_batch_stride, a->kv_row_stride, a->kv_batch_stride,
                          a->seq_q, a->seq_kv, a->batch, a->heads, a->kv_heads, a->scale, a->key_bias,
                          a->bias_batch_stride, a->out, a->out_row_stride, a->out_batch_stride};
  return mfx::attn::run(c, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
