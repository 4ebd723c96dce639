// Quantized linear layer  Y[M,N] = X[M,K] . dequant(Wq[N,K])^T + bias  for large M (tensor-core bound).
//
// Replaces mlx.nn.QuantizedLinear.__call__ -> mx.quantized_matmul(x, w, scales, biases, transpose=True,
// group_size=64, bits) for every nn.Linear of the transformer blocks of the reference
// (e.g. src/mflux/models/flux/model/flux_transformer/joint_attention.py:14-21, feed_forward.py:8-9).
//
// Two CTAs on neighbouring SMs form a pair (cluster of 2, tcgen05 cta_group::2) and share one 256 x 256
// output tile: each CTA loads the 128 activation rows of its half (A operand) and dequantizes 128 of the 256
// weight rows (its half of the B operand); one MMA of the pair reads both halves. Per flop that halves the
// dequantization work and the weight-operand shared-memory traffic of a single-CTA 128 x 256 tile, which is
// what bounded it. A pipeline stage carries two quantization groups (128 k-values) because the issuing thread
// loses a few hundred cycles around every wait + commit. Persistent, warp-specialised, per CTA:
//   warp 0      TMA producer: per stage its X tile [128 x 128 k] bf16 as two 128-byte-swizzled slabs (counted
//               on the leader's barrier), the packed codes of its 128 weight rows and their (scale, bias) pairs
//   warp 1      allocates TMEM; in the leader CTA issues tcgen05.mma.cta_group::2 (M=256, N=256, K=16)
//   warps 4-7   epilogue: tcgen05.ld -> bias / activation / gated residual -> global, overlapped with the
//               main loop of the next tile (two 256-column TMEM accumulators)
//   warps 8-15  dequantizers: codes (smem) -> bf16 -> B operand tile in the swizzled K-major layout. 4-bit codes
//               by the bf16 exponent-magic (128 + code) and one bf16 fma with the group's scale and bias; 8-bit
//               codes by the float32 magic (2^23 + code) and packed f32x2 add + fma, rounded to bf16 at the end
// Barriers that both CTAs feed live in the leader; MMA completion is multicast to both CTAs. All mbarrier
// waits are bounded.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <mutex>
#include <stdlib.h>
#include <string.h>

#include "host_util.cuh"
#include "ptx.cuh"
#include "qmm_common.cuh"
#include "qmm_t.cuh"
#include "qmv.cuh"

namespace mfx {
namespace qmm {

constexpr int BM = 128;       // activation rows per CTA (256 per pair)
constexpr int BN = 256;       // weight rows (output columns) per pair tile
constexpr int BN_HALF = 128;  // weight rows each CTA dequantizes
constexpr int BK = 64;        // one quantization group
constexpr int GPS = 2;        // quantization groups per pipeline stage
constexpr int FIXED_WARPS = 8;  // producer, MMA, 2 spare, 4 epilogue
constexpr int FIRST_DQ_WARP = 8;
constexpr int FIRST_EPI_WARP = 4;
constexpr int X_TILE_BYTES = BM * BK * 2;        // 16 KiB per group
constexpr int WD_TILE_BYTES = BN_HALF * BK * 2;  // 16 KiB per group
constexpr int SB_TILE_BYTES = BN_HALF * 4;       // one bf16 (scale, bias) pair per weight row
constexpr uint32_t TMEM_COLS = 512;

struct Params {
  int rows, batch, N, K;
  int tiles_m_per_sample, tiles_m, tiles_n, total_tiles;
  int band_n;  // n-tiles per band of the tile order (see tile_coords)
  // Low-rank extension: after the K / 64 quantized groups every tile runs num_ext more stages whose B operand is a
  // dense bf16 matrix lb [N, r] (read through the codes' staging buffer and copied instead of dequantized) and whose
  // A operand is t [batch, rows, r]; ext_r is the rank rounded up to 16. num_ext == 0: plain quantized matmul.
  int num_ext, ext_r;
  const void* bias;
  int bias_dtype;
  int epilogue;
  const void* gate;
  int gate_dtype;
  int64_t gate_batch_stride;
  const void* residual;
  int64_t res_row_stride, res_batch_stride;
  void* y;
  int64_t y_row_stride, y_batch_stride;
  // MFX_EPI_PEER_SCATTER: partial rows go to slot [sc_rank] of the rank that owns them (see include/mfx.h)
  int sc_world, sc_rank;
  int64_t sc_rows_per_rank, sc_row_offset;
  __nv_bfloat16* sc_dst[MFX_TP_MAX_WORLD];
  int* sc_flags[MFX_TP_MAX_WORLD];
  int* sc_done;
};

// ST = stages of the TMA ring, SD = stages of the dequantized-weight ring; one stage = GPS groups.
// STG = bytes of the epilogue's staging buffer (tensor-parallel scatter only).
template <int BITS, int ST, int SD, int STG = 0>
struct Smem {
  static constexpr int WQ_TILE_BYTES = BN_HALF * BK * BITS / 8;
  static constexpr int X_STAGE = GPS * X_TILE_BYTES;
  static constexpr int WD_STAGE = GPS * WD_TILE_BYTES;
  static constexpr int WQ_STAGE = GPS * WQ_TILE_BYTES;
  static constexpr int SB_STAGE = GPS * SB_TILE_BYTES;
  static constexpr int OFF_X = 0;
  static constexpr int OFF_WD = OFF_X + ST * X_STAGE;
  static constexpr int OFF_WQ = OFF_WD + SD * WD_STAGE;
  static constexpr int OFF_SB = OFF_WQ + ST * WQ_STAGE;
  static constexpr int OFF_VEC = OFF_SB + ST * SB_STAGE;  // bias[2][256] + gate[2][256] floats
  static constexpr int OFF_STAGE = OFF_VEC + 4 * BN * 4;
  static constexpr int OFF_BAR = OFF_STAGE + STG;
  static constexpr int NUM_BARS = 4 * ST + 2 * SD + 4;
  static constexpr int OFF_TMEM = OFF_BAR + NUM_BARS * 8;
  static constexpr int TOTAL = OFF_TMEM + 16;
  static constexpr int DYN_BYTES = TOTAL + 1024;  // slack for manual 1024-byte alignment
};

// Tile order. The weight rows are cut into bands of band_n n-tiles whose packed codes, scales and biases fit in
// L2 together; inside a band the tiles run m-tile by m-tile with the n-tile index fastest. The pairs that run at
// the same time then share one or two activation tiles (read from HBM once per band) and sweep a band of weights
// that stays in L2, instead of each streaming its own activation tile from HBM once per n-tile.
__device__ __forceinline__ void tile_coords(const Params& p, int tile, int& tm, int& tn) {
  const int per_band = p.tiles_m * p.band_n;
  const int band = tile / per_band;
  const int r = tile - band * per_band;
  const int n_first = band * p.band_n;
  const int width = min(p.band_n, p.tiles_n - n_first);
  tm = r / width;
  tn = n_first + r - tm * width;
}

// EXT compiles the low-rank extension stages in; without it the loops below are the plain quantized matmul.
template <int BITS, uint32_t WF, int ST, int SD, typename OUT, int EPI, int NUM_DQ_WARPS, bool EXT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__((FIXED_WARPS + NUM_DQ_WARPS) * 32, 1)
qmm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
           const __grid_constant__ CUtensorMap tmap_sb, const __grid_constant__ CUtensorMap tmap_t,
           const __grid_constant__ CUtensorMap tmap_lb, const Params p) {
  // The scatter epilogue stages 32 rows x SCATTER_ROW bytes per epilogue warp to turn "thread = row" into stores
  // of whole 128-byte (64-byte for 8-bit codes, where shared memory is tighter) row segments.
  constexpr int SCATTER_ROW = BITS == 4 ? 128 : 64;
  using L = Smem<BITS, ST, SD, EPI == MFX_EPI_PEER_SCATTER ? 4 * 32 * SCATTER_ROW : 0>;
  // With as many TMA stages as dequantized-weight stages the two rings advance in lockstep and one "stage
  // consumed" barrier serves both: the commit after a stage's MMAs frees its activation tile and its B tile, and
  // the stage's packed codes were read before its B tile was written, so they are free by then too. That is one
  // tcgen05.commit and eight dequantizer arrivals less per stage.
  constexpr bool UNIFIED = (ST == SD);
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t x_s = smem_base + L::OFF_X;
  const uint32_t wd_s = smem_base + L::OFF_WD;
  const uint32_t wq_s = smem_base + L::OFF_WQ;
  const uint32_t sb_s = smem_base + L::OFF_SB;
  float* vec_s = reinterpret_cast<float*>(smem_gen + L::OFF_VEC);
  const uint32_t bar0 = smem_base + L::OFF_BAR;
  auto w_full = [&](int s) { return bar0 + 8u * s; };              // local: codes + pairs landed
  auto x_full = [&](int s) { return bar0 + 8u * (ST + s); };       // leader: X tiles of both CTAs landed
  auto t_empty = [&](int s) { return bar0 + 8u * (2 * ST + s); };  // local: TMA stage may be refilled
  constexpr int B0 = 3 * ST;
  auto d_full = [&](int s) { return bar0 + 8u * (B0 + s); };             // leader: B halves of both CTAs written
  auto d_empty = [&](int s) {                                              // local: B stage consumed
    return UNIFIED ? bar0 + 8u * (2 * ST + s) : bar0 + 8u * (B0 + SD + s);   // (== t_empty when unified)
  };
  auto acc_full = [&](int s) { return bar0 + 8u * (B0 + 2 * SD + s); };  // local
  auto acc_empty = [&](int s) { return bar0 + 8u * (B0 + 2 * SD + 2 + s); };  // leader
  auto c_empty = [&](int s) { return bar0 + 8u * (B0 + 2 * SD + 4 + s); };    // local: codes of the stage were read
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::OFF_TMEM);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = p.K / BK;
  const int num_st = (num_kb + GPS - 1) / GPS;  // a ragged last stage reads TMA zero fill for its missing group
  // An extension stage moves as many bytes through the codes' staging buffer as a quantized one: per group
  // 128 rows x EXT_KG dense bf16 values, 16 (4-bit codes) or 32 (8-bit codes) k-values of the low-rank term.
  constexpr int EXT_KG = 4 * BITS;
  const int num_all = EXT ? num_st + p.num_ext : num_st;
  const uint32_t rank = cluster_ctarank();      // 0 = leader of the pair
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < ST; ++s) {
      mbar_init(w_full(s), 1);
      mbar_init(x_full(s), 1);                  // the leader's expect_tx covers both CTAs' X tiles
      mbar_init(t_empty(s), 1);              // MMA commit: the activation tile (and, unified, the B tile) is free
      mbar_init(c_empty(s), NUM_DQ_WARPS);   // every local dequantizer warp has read the stage's codes
    }
    for (int s = 0; s < SD; ++s) {
      mbar_init(d_full(s), 2 * NUM_DQ_WARPS);   // the dequantizer warps of both CTAs
      if (!UNIFIED) mbar_init(d_empty(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(acc_full(s), 1);
      mbar_init(acc_empty(s), 8);               // 4 epilogue warps in each CTA
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmap_x);
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_sb);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_base + L::OFF_TMEM, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anyone signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer of the activation tiles
    // The activation tile of a stage is free only once the stage's MMAs are done, the packed codes as soon as the
    // dequantizers have read them. Two producers with their own barriers let the codes (warp 2) run ahead of the
    // activations, so that dequantizing stage s+1, s+2 overlaps the flight time of activation tile s instead of
    // following it: with both on one barrier the chain TMA -> dequantize -> MMA -> commit bounded a stage.
    int st = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int tile = pair; tile < p.total_tiles && ok; tile += num_pairs) {
      int tm, tn;
      tile_coords(p, tile, tm, tn);
      const int b = tm / p.tiles_m_per_sample;
      const int r0 = (tm % p.tiles_m_per_sample) * (2 * BM) + static_cast<int>(rank) * BM;
      for (int s = 0; s < num_all; ++s) {
        if (!mbar_wait(t_empty(st), ph ^ 1u, DEV_TIMEOUT_TMA_EMPTY)) {
          ok = false;
          break;
        }
        if (lane == 0) {
          if (rank == 0) mbar_arrive_expect_tx(x_full(st), 2 * L::X_STAGE);
          if (!EXT || s < num_st) {
#pragma unroll
            for (int g = 0; g < GPS; ++g)   // beyond K on a ragged last stage: the loads return zeros
              tma_load_3d_pair(x_s + st * L::X_STAGE + g * X_TILE_BYTES, &tmap_x, x_full(st), (s * GPS + g) * BK, r0,
                               b);
          } else {
            // extension stage: the activation tile comes from t, whose first EXT_KG columns the tensor cores read
#pragma unroll
            for (int g = 0; g < GPS; ++g)
              tma_load_3d_pair(x_s + st * L::X_STAGE + g * X_TILE_BYTES, &tmap_t, x_full(st),
                               ((s - num_st) * GPS + g) * EXT_KG, r0, b);
          }
        }
        __syncwarp();
        if (++st == ST) {
          st = 0;
          ph ^= 1u;
        }
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------ TMA producer of the packed weights
    int st = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int tile = pair; tile < p.total_tiles && ok; tile += num_pairs) {
      int tm, tn;
      tile_coords(p, tile, tm, tn);
      const int n0 = tn * BN + static_cast<int>(rank) * BN_HALF;
      for (int s = 0; s < num_all; ++s) {
        if (!mbar_wait(c_empty(st), ph ^ 1u, DEV_TIMEOUT_TMA_EMPTY)) {
          ok = false;
          break;
        }
        if (lane == 0) {
          mbar_arrive_expect_tx(w_full(st), L::WQ_STAGE + L::SB_STAGE);
          if (!EXT || s < num_st) {
#pragma unroll
            for (int g = 0; g < GPS; ++g) {
              const int kb = s * GPS + g;
              tma_load_2d(wq_s + st * L::WQ_STAGE + g * L::WQ_TILE_BYTES, &tmap_w, w_full(st),
                          kb * (BK * BITS / 32), n0);
              tma_load_2d(sb_s + st * L::SB_STAGE + g * SB_TILE_BYTES, &tmap_sb, w_full(st), n0, kb);
            }
          } else {
            // Extension stage: the same byte counts on the same barrier. The dense tile lands where the codes
            // would; the (scale, bias) load reads past the last group (zero fill, unused).
#pragma unroll
            for (int g = 0; g < GPS; ++g) {
              const int k0 = ((s - num_st) * GPS + g) * EXT_KG;
              tma_load_2d(wq_s + st * L::WQ_STAGE + g * L::WQ_TILE_BYTES, &tmap_lb, w_full(st), k0, n0);
              tma_load_2d(sb_s + st * L::SB_STAGE + g * SB_TILE_BYTES, &tmap_sb, w_full(st), n0, num_kb + g);
            }
          }
        }
        __syncwarp();
        if (++st == ST) {
          st = 0;
          ph ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (rank == 0) {
      constexpr uint32_t IDESC = make_idesc(FMT_BF16, WF, 2 * BM, BN);  // M = 256 over the pair, N = 256
      int st = 0, sd = 0;
      uint32_t ph_t = 0, ph_d = 0;
      bool ok = true;
      int it = 0;
      for (int tile = pair; tile < p.total_tiles && ok; tile += num_pairs, ++it) {
        const int a = it & 1;
        const uint32_t aph = (it >> 1) & 1;
        if (!mbar_wait(acc_empty(a), aph ^ 1u, DEV_TIMEOUT_ACC_EMPTY)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + a * BN;
        for (int s = 0; s < num_all; ++s) {
          if (!mbar_wait(x_full(st), ph_t, DEV_TIMEOUT_TMA_FULL) || !mbar_wait(d_full(sd), ph_d, DEV_TIMEOUT_DQ_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          if (lane == 0) {
            if (!EXT || s < num_st) {
#pragma unroll
              for (int g = 0; g < GPS; ++g) {
                const uint64_t adesc = smem_desc_sw128(x_s + st * L::X_STAGE + g * X_TILE_BYTES);
                const uint64_t bdesc = smem_desc_sw128(wd_s + sd * L::WD_STAGE + g * WD_TILE_BYTES);
#pragma unroll
                for (int k4 = 0; k4 < BK / 16; ++k4) {
                  // +32 bytes (>>4 = 2) per 16-element K step inside the 128-byte swizzle atom
                  umma_f16_ss_pair(d_tmem, adesc + 2 * k4, bdesc + 2 * k4, IDESC, (s | g | k4) != 0 ? 1u : 0u);
                }
              }
            } else {
              // extension stage: only the first EXT_KG k-values of each group's tiles carry data, and only up
              // to the rank (the tile always starts with a quantized stage, so these always accumulate)
#pragma unroll
              for (int g = 0; g < GPS; ++g) {
                const uint64_t adesc = smem_desc_sw128(x_s + st * L::X_STAGE + g * X_TILE_BYTES);
                const uint64_t bdesc = smem_desc_sw128(wd_s + sd * L::WD_STAGE + g * WD_TILE_BYTES);
                const int k0 = ((s - num_st) * GPS + g) * EXT_KG;
#pragma unroll
                for (int k4 = 0; k4 < EXT_KG / 16; ++k4) {
                  if (k0 + 16 * k4 < p.ext_r) umma_f16_ss_pair(d_tmem, adesc + 2 * k4, bdesc + 2 * k4, IDESC, 1u);
                }
              }
            }
            umma_commit_pair(t_empty(st));
            if (!UNIFIED) umma_commit_pair(d_empty(sd));
            if (s == num_all - 1) umma_commit_pair(acc_full(a));
          }
          __syncwarp();
          if (++st == ST) {
            st = 0;
            ph_t ^= 1u;
          }
          if (++sd == SD) {
            sd = 0;
            ph_d ^= 1u;
          }
        }
      }
    }
  } else if (warp >= FIRST_DQ_WARP) {
    // ------------------------------------------------------------ dequantizers
    // Every warp serves one quantization group of the stage: with 8 warps four warps per group and one thread
    // per weight row (16 warps would give eight per group and half a row per thread).
    constexpr int WPG = NUM_DQ_WARPS / GPS;        // warps per group
    constexpr int SPLIT = WPG / 4;                 // threads per weight row: 1 or 2
    const int dq = warp - FIRST_DQ_WARP;
    const int grp = dq / WPG;
    const int row = ((dq % WPG) / SPLIT) * 32 + lane;  // row of this CTA's 128-row weight tile
    const int part = dq % SPLIT;                       // which part of the row's 64 k-values
    constexpr int ROW_BYTES = BK * BITS / 8;           // packed bytes per row per group
    constexpr int RD_CHUNKS = ROW_BYTES / 16;          // 16-byte chunks per row: 2 (4 bits) or 4 (8 bits)
    constexpr int MY_CHUNKS = RD_CHUNKS / SPLIT;       // packed chunks this thread reads
    constexpr int MY_OUT = 8 / SPLIT;                  // 16-byte output chunks this thread writes
    // The packed tile is loaded with the TMA swizzle whose span equals one row (32 B for 4 bits,
    // 64 B for 8 bits): 16-byte chunk c of row r sits at chunk c ^ ((r*ROW_BYTES >> 7) & mask), which
    // spreads the per-row reads of a quarter-warp over all banks. Offsets are per-thread constants.
    const uint32_t rd_sw = (static_cast<uint32_t>(row * ROW_BYTES) >> 7) & (RD_CHUNKS - 1);
    const uint8_t* rd_base = smem_gen + L::OFF_WQ + grp * L::WQ_TILE_BYTES + row * ROW_BYTES;
    uint32_t rd_off[MY_CHUNKS];
#pragma unroll
    for (int h = 0; h < MY_CHUNKS; ++h) rd_off[h] = (static_cast<uint32_t>(part * MY_CHUNKS + h) ^ rd_sw) << 4;
    // B operand tile: 128-byte rows, 16-byte chunk c of row r at chunk c ^ (r & 7)
    uint8_t* wr_base = smem_gen + L::OFF_WD + grp * WD_TILE_BYTES + row * 128;
    uint32_t wr_off[MY_OUT];
#pragma unroll
    for (int c = 0; c < MY_OUT; ++c)
      wr_off[c] = (static_cast<uint32_t>(part * MY_OUT + c) ^ static_cast<uint32_t>(row & 7)) << 4;
    const uint32_t* sb_base = reinterpret_cast<const uint32_t*>(smem_gen + L::OFF_SB + grp * SB_TILE_BYTES) + row;
    int st = 0, sd = 0;
    uint32_t ph_t = 0, ph_d = 0;
    bool ok = true;
    for (int tile = pair; tile < p.total_tiles && ok; tile += num_pairs) {
      for (int s = 0; s < num_all; ++s) {
        if (!mbar_wait(d_empty(sd), ph_d ^ 1u, DEV_TIMEOUT_DQ_EMPTY) ||
            !mbar_wait(w_full(st), ph_t, DEV_TIMEOUT_TMA_FULL)) {
          ok = false;
          break;
        }
        if (EXT && s >= num_st) {
          // extension stage: the staged bytes are bf16 values already; chunk c of the row goes to chunk c of the
          // B tile row (the tensor cores read no further than EXT_KG k-values of these stages)
          const uint8_t* esrc = rd_base + st * L::WQ_STAGE;
          uint8_t* edst = wr_base + sd * L::WD_STAGE;
#pragma unroll
          for (int h = 0; h < MY_CHUNKS; ++h) {
            const uint32_t c = static_cast<uint32_t>(part * MY_CHUNKS + h);
            *reinterpret_cast<uint4*>(edst + ((c ^ static_cast<uint32_t>(row & 7)) << 4)) =
                *reinterpret_cast<const uint4*>(esrc + rd_off[h]);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            mbar_arrive_leader(d_full(sd));
            mbar_arrive(c_empty(st));
          }
          if (++st == ST) {
            st = 0;
            ph_t ^= 1u;
          }
          if (++sd == SD) {
            sd = 0;
            ph_d ^= 1u;
          }
          continue;
        }
        const uint32_t sbv = sb_base[st * (L::SB_STAGE / 4)];
        const uint32_t s2 = __byte_perm(sbv, sbv, 0x1010);  // (scale, scale)
        const uint32_t b2 = __byte_perm(sbv, sbv, 0x3232);  // (bias, bias)
        const uint8_t* src = rd_base + st * L::WQ_STAGE;
        uint8_t* dst = wr_base + sd * L::WD_STAGE;
#pragma unroll
        for (int h = 0; h < MY_CHUNKS; ++h) {
          const uint4 pk = *reinterpret_cast<const uint4*>(src + rd_off[h]);
          if (BITS == 4) {  // 4 words x 8 codes -> 4 output chunks
            const uint32_t wds[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
            for (int j = 0; j < 4; ++j)
              *reinterpret_cast<uint4*>(dst + wr_off[h * 4 + j]) = dequant_w4(wds[j], s2, b2);
          } else {          // 4 words x 4 codes -> 2 output chunks
            const uint32_t sf = sbv << 16, bf = sbv & 0xFFFF0000u;   // scale and bias as float32 bit patterns
            uint64_t sc2, bi2;
            asm("mov.b64 %0, {%1, %1};" : "=l"(sc2) : "r"(sf));
            asm("mov.b64 %0, {%1, %1};" : "=l"(bi2) : "r"(bf));
            const uint2 lo0 = dequant_w8_f32(pk.x, sc2, bi2);
            const uint2 hi0 = dequant_w8_f32(pk.y, sc2, bi2);
            const uint2 lo1 = dequant_w8_f32(pk.z, sc2, bi2);
            const uint2 hi1 = dequant_w8_f32(pk.w, sc2, bi2);
            *reinterpret_cast<uint4*>(dst + wr_off[2 * h]) = make_uint4(lo0.x, lo0.y, hi0.x, hi0.y);
            *reinterpret_cast<uint4*>(dst + wr_off[2 * h + 1]) = make_uint4(lo1.x, lo1.y, hi1.x, hi1.y);
          }
        }
        fence_proxy_async_smem();  // make these generic-proxy writes visible to the tensor cores of the pair
        __syncwarp();
        if (lane == 0) {
          mbar_arrive_leader(d_full(sd));
          mbar_arrive(c_empty(st));
        }
        if (++st == ST) {
          st = 0;
          ph_t ^= 1u;
        }
        if (++sd == SD) {
          sd = 0;
          ph_d ^= 1u;
        }
      }
    }
  } else if (warp >= FIRST_EPI_WARP) {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;            // TMEM lane quarter this warp may read
    const int et = threadIdx.x - FIRST_EPI_WARP * 32;  // 0..127
    const int row = q * 32 + lane;
    bool ok = true;
    int it = 0;
    for (int tile = pair; tile < p.total_tiles && ok; tile += num_pairs, ++it) {
      const int a = it & 1;
      const uint32_t aph = (it >> 1) & 1;
      int tm, tn;
      tile_coords(p, tile, tm, tn);
      const int b = tm / p.tiles_m_per_sample;
      const int r = (tm % p.tiles_m_per_sample) * (2 * BM) + static_cast<int>(rank) * BM + row;
      const int n0 = tn * BN;
      float* bias_s = vec_s + a * BN;
      float* gate_s = vec_s + 2 * BN + a * BN;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int c = et + 128 * h;
        const int n = n0 + c;
        bias_s[c] = (p.bias != nullptr && n < p.N) ? load_scalar(p.bias, p.bias_dtype, n) : 0.f;
        if (EPI == MFX_EPI_GATE_RESIDUAL)
          gate_s[c] = (n < p.N) ? load_scalar(p.gate, p.gate_dtype, b * p.gate_batch_stride + n) : 0.f;
      }
      named_bar_sync(1, 128);
      if (!mbar_wait_sleep(acc_full(a), aph, DEV_TIMEOUT_ACC_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const bool row_ok = r < p.rows;
      // SwiGLU writes one value per (gate, up) column pair: output column n/2
      OUT* yrow = static_cast<OUT*>(p.y) + b * p.y_batch_stride + static_cast<int64_t>(r) * p.y_row_stride +
                  (EPI == MFX_EPI_SWIGLU ? n0 / 2 : n0);
      const OUT* rrow = nullptr;
      if (EPI == MFX_EPI_GATE_RESIDUAL)
        rrow = static_cast<const OUT*>(p.residual) + b * p.res_batch_stride +
               static_cast<int64_t>(r) * p.res_row_stride + n0;
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + a * BN;
      if constexpr (EPI == MFX_EPI_PEER_SCATTER) {
        // Partial rows go to slot [sc_rank] of the rank that owns each row, over NVLink, where only stores of whole
        // lines run at full rate (measured: 32-byte pieces of 32 different rows per instruction 280 GB/s, whole
        // lines 655 GB/s). So: thread = row writes its packed bf16 values into a swizzled staging tile, then the
        // warp stores the tile SCATTER_ROW bytes of a row at a time (lane = 16-byte piece, 32 / PIECES rows per
        // instruction).
        constexpr int PIECES = SCATTER_ROW / 16;
        constexpr int ROWS_PER_ST = 32 / PIECES;
        constexpr int CHUNKS = SCATTER_ROW / 64;   // 32-column accumulator chunks per staged row
        uint8_t* stg = smem_gen + L::OFF_STAGE + q * (32 * SCATTER_ROW);
        const int piece = lane % PIECES, rsub = lane / PIECES;
        __nv_bfloat16* drow[PIECES];
#pragma unroll
        for (int i = 0; i < PIECES; ++i) {
          const int rr = rsub + ROWS_PER_ST * i;
          const int rg = r - lane + rr;   // row of the sample this lane stores in pass i
          drow[i] = nullptr;
          if (rg < p.rows) {
            const int64_t tj = p.sc_row_offset + rg;   // row of the joint sequence
            const int64_t owner = tj / p.sc_rows_per_rank;
            const int64_t local = tj - owner * p.sc_rows_per_rank;
            drow[i] = p.sc_dst[owner] +
                      ((static_cast<int64_t>(p.sc_rank) * p.batch + b) * p.sc_rows_per_rank + local) * p.N + n0;
          }
        }
#pragma unroll 1
        for (int round = 0; round < BN / (32 * CHUNKS); ++round) {
          if (n0 + round * 32 * CHUNKS >= p.N) break;
#pragma unroll
          for (int h = 0; h < CHUNKS; ++h) {
            uint32_t acc[32];
            tmem_ld_32x32(t_addr + (round * CHUNKS + h) * 32, acc);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              __nv_bfloat162 hh[4];
#pragma unroll
              for (int e = 0; e < 4; ++e)
                hh[e] = __floats2bfloat162_rn(__uint_as_float(acc[8 * j + 2 * e]), __uint_as_float(acc[8 * j + 2 * e + 1]));
              const int idx = h * 4 + j;
              *reinterpret_cast<uint4*>(stg + lane * SCATTER_ROW + ((idx ^ (lane & (PIECES - 1))) << 4)) =
                  *reinterpret_cast<uint4*>(hh);
            }
          }
          __syncwarp();
          const int col = round * 32 * CHUNKS + piece * 8;
#pragma unroll
          for (int i = 0; i < PIECES; ++i) {
            const int rr = rsub + ROWS_PER_ST * i;
            const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * SCATTER_ROW + ((piece ^ (rr & (PIECES - 1))) << 4));
            if (drow[i] != nullptr && n0 + col < p.N) *reinterpret_cast<uint4*>(drow[i] + col) = v;
          }
          __syncwarp();
        }
      } else
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t acc[32];
        tmem_ld_32x32(t_addr + c * 32, acc);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int g8 = 0; g8 < 4; ++g8) {
            const int col = c * 32 + g8 * 8;
            if (n0 + col >= p.N) break;
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(acc[g8 * 8 + j]) + bias_s[col + j];
            if (EPI == MFX_EPI_GELU_ERF) {
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = gelu_erf(v[j]);
            } else if (EPI == MFX_EPI_GELU_TANH) {
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = gelu_tanh(v[j]);
            } else if (EPI == MFX_EPI_SILU) {
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = silu(v[j]);
            } else if (EPI == MFX_EPI_GATE_RESIDUAL) {
              float rs[8];
              if constexpr (sizeof(OUT) == 4) {
                // the float32 residual stream is read once and written once per launch and is larger than L2:
                // streaming loads / stores keep it from evicting the activation tiles the other n-tiles re-read
                const float4 r0 = __ldcs(reinterpret_cast<const float4*>(rrow + col));
                const float4 r1 = __ldcs(reinterpret_cast<const float4*>(rrow + col + 4));
                rs[0] = r0.x; rs[1] = r0.y; rs[2] = r0.z; rs[3] = r0.w;
                rs[4] = r1.x; rs[5] = r1.y; rs[6] = r1.z; rs[7] = r1.w;
              } else {
                const uint4 raw = *reinterpret_cast<const uint4*>(rrow + col);
                const __nv_bfloat16* hb = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
                for (int j = 0; j < 8; ++j) rs[j] = __bfloat162float(hb[j]);
              }
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = rs[j] + gate_s[col + j] * v[j];
            }
            if constexpr (EPI == MFX_EPI_SWIGLU) {
              float o[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) o[j] = silu(v[2 * j]) * v[2 * j + 1];
              if constexpr (sizeof(OUT) == 4) {
                *reinterpret_cast<float4*>(yrow + col / 2) = make_float4(o[0], o[1], o[2], o[3]);
              } else {
                __nv_bfloat162 h[2];
                h[0] = __floats2bfloat162_rn(o[0], o[1]);
                h[1] = __floats2bfloat162_rn(o[2], o[3]);
                *reinterpret_cast<uint2*>(yrow + col / 2) = *reinterpret_cast<uint2*>(h);
              }
            } else if constexpr (sizeof(OUT) == 4) {
              if constexpr (EPI == MFX_EPI_GATE_RESIDUAL) {
                __stcs(reinterpret_cast<float4*>(yrow + col), make_float4(v[0], v[1], v[2], v[3]));
                __stcs(reinterpret_cast<float4*>(yrow + col + 4), make_float4(v[4], v[5], v[6], v[7]));
              } else {
                *reinterpret_cast<float4*>(yrow + col) = make_float4(v[0], v[1], v[2], v[3]);
                *reinterpret_cast<float4*>(yrow + col + 4) = make_float4(v[4], v[5], v[6], v[7]);
              }
            } else {
              __nv_bfloat162 h[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
              *reinterpret_cast<uint4*>(yrow + col) = *reinterpret_cast<uint4*>(h);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_leader(acc_empty(a));
    }
    if (EPI == MFX_EPI_PEER_SCATTER) {
      // every thread's peer stores are ordered before this CTA's arrival; the last CTA of the grid tells the owners
      __threadfence_system();
      named_bar_sync(1, 128);
      if (threadIdx.x == FIRST_EPI_WARP * 32) {
        const int done = atomicAdd(p.sc_done, 1);
        if (done == static_cast<int>(gridDim.x) - 1) {
          *p.sc_done = 0;
          __threadfence_system();
          for (int r = 0; r < p.sc_world; ++r)
            asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p.sc_flags[r]), "r"(1) : "memory");
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer may still be reading this CTA's shared/tensor memory until here
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

MFX_DEFINE_STATUS_READER(read_status)

template <int BITS, uint32_t WF, int ST, int SD, typename OUT, int EPI, bool EXT>
int launch_epi(const CUtensorMap& tx, const CUtensorMap& tw, const CUtensorMap& tsb, const CUtensorMap& tt,
               const CUtensorMap& tlb, const Params& p, int grid, cudaStream_t st) {
  using L = Smem<BITS, ST, SD, EPI == MFX_EPI_PEER_SCATTER ? 4 * 32 * (BITS == 4 ? 128 : 64) : 0>;
  // eight dequantizer warps keep up with the tensor pipe for both widths (8-bit codes go through packed float32
  // arithmetic, five instructions per pair) and draw less power than sixteen
  constexpr int NDQ = 8;
  constexpr int NUM_THREADS = (FIXED_WARPS + NDQ) * 32;
  auto kern = qmm_kernel<BITS, WF, ST, SD, OUT, EPI, NDQ, EXT>;
  static SmemConfigured configured;  // one record per instantiation of the kernel
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), L::DYN_BYTES, configured)) return rc;
  kern<<<grid, NUM_THREADS, L::DYN_BYTES, st>>>(tx, tw, tsb, tt, tlb, p);
  MFX_CUDA_TRY(cudaGetLastError());
  return MFX_OK;
}

template <int BITS, uint32_t WF, int ST, int SD, typename OUT, bool EXT>
int launch_ext(const CUtensorMap& tx, const CUtensorMap& tw, const CUtensorMap& tsb, const CUtensorMap& tt,
           const CUtensorMap& tlb, const Params& p, int grid, cudaStream_t st) {
  switch (p.epilogue) {
    case MFX_EPI_GELU_ERF: return launch_epi<BITS, WF, ST, SD, OUT, MFX_EPI_GELU_ERF, EXT>(tx, tw, tsb, tt, tlb, p, grid, st);
    case MFX_EPI_GELU_TANH: return launch_epi<BITS, WF, ST, SD, OUT, MFX_EPI_GELU_TANH, EXT>(tx, tw, tsb, tt, tlb, p, grid, st);
    case MFX_EPI_GATE_RESIDUAL: return launch_epi<BITS, WF, ST, SD, OUT, MFX_EPI_GATE_RESIDUAL, EXT>(tx, tw, tsb, tt, tlb, p, grid, st);
    case MFX_EPI_SILU: return launch_epi<BITS, WF, ST, SD, OUT, MFX_EPI_SILU, EXT>(tx, tw, tsb, tt, tlb, p, grid, st);
    case MFX_EPI_SWIGLU: return launch_epi<BITS, WF, ST, SD, OUT, MFX_EPI_SWIGLU, EXT>(tx, tw, tsb, tt, tlb, p, grid, st);
    case MFX_EPI_PEER_SCATTER:
      if constexpr (sizeof(OUT) == 2 && !EXT)
        return launch_epi<BITS, WF, ST, SD, OUT, MFX_EPI_PEER_SCATTER, EXT>(tx, tw, tsb, tt, tlb, p, grid, st);
      else
        return MFX_ERR_DTYPE;
    default: return launch_epi<BITS, WF, ST, SD, OUT, MFX_EPI_NONE, EXT>(tx, tw, tsb, tt, tlb, p, grid, st);
  }
}

template <int BITS, uint32_t WF, int ST, int SD, typename OUT>
int launch(const CUtensorMap& tx, const CUtensorMap& tw, const CUtensorMap& tsb, const CUtensorMap& tt,
           const CUtensorMap& tlb, const Params& p, int grid, cudaStream_t st) {
  return p.num_ext > 0 ? launch_ext<BITS, WF, ST, SD, OUT, true>(tx, tw, tsb, tt, tlb, p, grid, st)
                       : launch_ext<BITS, WF, ST, SD, OUT, false>(tx, tw, tsb, tt, tlb, p, grid, st);
}

// sb[g * N + n] = bf16(scales[n, g]) | bf16(biases[n, g]) << 16
__global__ void __launch_bounds__(256) pack_scales_kernel(const void* __restrict__ scales,
                                                          const void* __restrict__ biases, int sb_dtype, int N,
                                                          int G, uint32_t* __restrict__ packed) {
  __shared__ uint32_t tile[32][33];
  const int n0 = blockIdx.x * 32, g0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int n = n0 + ty + 8 * i, g = g0 + tx;  // reads run along g (contiguous in [N, G])
    uint32_t v = 0;
    if (n < N && g < G) {
      const int64_t idx = static_cast<int64_t>(n) * G + g;
      const __nv_bfloat16 sv = __float2bfloat16_rn(load_scalar(scales, sb_dtype, idx));
      const __nv_bfloat16 bv = __float2bfloat16_rn(load_scalar(biases, sb_dtype, idx));
      v = static_cast<uint32_t>(__bfloat16_as_ushort(sv)) | (static_cast<uint32_t>(__bfloat16_as_ushort(bv)) << 16);
    }
    tile[ty + 8 * i][tx] = v;
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int g = g0 + ty + 8 * i, n = n0 + tx;  // writes run along n (contiguous in [G, N])
    if (n < N && g < G) packed[static_cast<int64_t>(g) * N + n] = tile[tx][ty + 8 * i];
  }
}

// Interleave the codes of every uint32: 4 bits -> nibbles e0,e2,e4,e6,e1,e3,e5,e7; 8 bits -> bytes e0,e2,e1,e3.
template <int BITS>
__global__ void __launch_bounds__(256) interleave_codes_kernel(const uint4* __restrict__ in, uint4* __restrict__ out,
                                                               int64_t n_vec) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  const uint4 v = __ldg(in + i);
  uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t q = w[j];
    if (BITS == 4) {
      uint32_t r = 0;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int pos = (e & 1) ? 4 + (e >> 1) : (e >> 1);
        r |= ((q >> (4 * e)) & 0xFu) << (4 * pos);
      }
      w[j] = r;
    } else {
      w[j] = __byte_perm(q, 0u, 0x3120);
    }
  }
  out[i] = make_uint4(w[0], w[1], w[2], w[3]);
}

// Codes of SRC_BITS (3, 5 or 6) bits, packed as a little-end-first bit stream, widened to the kernel's 4- or 8-bit
// codes and interleaved like interleave_codes_kernel does. One thread writes 16 bytes: 32 (4-bit) or 16 (8-bit)
// codes, whose source is 12, 10 or 12 bytes of the stream.
template <int SRC_BITS>
__global__ void __launch_bounds__(256) widen_codes_kernel(const uint8_t* __restrict__ in, uint4* __restrict__ out,
                                                          int64_t n_vec) {
  constexpr int KB = SRC_BITS <= 4 ? 4 : 8;
  constexpr int CODES = 128 / KB;                 // codes per 16-byte vector
  constexpr int SRC_BYTES = CODES * SRC_BITS / 8;
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  const uint8_t* src = in + i * SRC_BYTES;
  uint32_t w[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    // the 8 (or 4) codes of output word j start at bit j * (32 / KB) * SRC_BITS of this thread's stream
    constexpr int PER_WORD = 32 / KB;
    const int bit0 = j * PER_WORD * SRC_BITS;
    unsigned long long stream = 0;
#pragma unroll
    for (int b = 0; b < (PER_WORD * SRC_BITS + 7) / 8 + 1; ++b) {
      const int byte = bit0 / 8 + b;
      if (byte < SRC_BYTES) stream |= static_cast<unsigned long long>(__ldg(src + byte)) << (8 * b);
    }
    stream >>= (bit0 & 7);
    uint32_t r = 0;
#pragma unroll
    for (int e = 0; e < PER_WORD; ++e) {
      const uint32_t code = static_cast<uint32_t>(stream >> (SRC_BITS * e)) & ((1u << SRC_BITS) - 1u);
      int pos;
      if (KB == 4) pos = (e & 1) ? 4 + (e >> 1) : (e >> 1);   // nibbles e0,e2,e4,e6,e1,e3,e5,e7
      else pos = (e == 1) ? 2 : (e == 2) ? 1 : e;             // bytes e0,e2,e1,e3
      r |= code << (KB * pos);
    }
    w[j] = r;
  }
  out[i] = make_uint4(w[0], w[1], w[2], w[3]);
}

size_t codes_bytes_padded(int64_t N, int64_t K, int bits) {
  const size_t raw = static_cast<size_t>(N) * static_cast<size_t>(K) * kernel_bits(bits) / 8;
  return (raw + 255) & ~static_cast<size_t>(255);
}

size_t prepared_bytes(int64_t N, int64_t K, int bits, int group_size) {
  if (N <= 0 || K <= 0 || group_size != 64 || K % 64 != 0 || !valid_bits(bits)) return 0;
  return codes_bytes_padded(N, K, bits) + static_cast<size_t>(N) * static_cast<size_t>(K / 64) * 4;
}

int prepare(const uint32_t* wq, const void* scales, const void* biases, int sb_dtype, int64_t N, int64_t K,
            int bits, int group_size, void* prepared, size_t bytes, cudaStream_t st) {
  if (!wq || !scales || !biases || !prepared) return MFX_ERR_NULL;
  if (!valid_bits(bits) || group_size != 64) return MFX_ERR_UNSUPPORTED_BITS;
  if (N <= 0 || K <= 0 || K % 64 != 0) return MFX_ERR_SHAPE;
  if (N > (1 << 30) || K > (1 << 30)) return MFX_ERR_TOO_LARGE;
  if (!valid_dtype(sb_dtype)) return MFX_ERR_DTYPE;
  if (bytes < prepared_bytes(N, K, bits, group_size)) return MFX_ERR_SHAPE;
  if (!aligned16(wq) || (reinterpret_cast<uintptr_t>(prepared) & 255u) != 0) return MFX_ERR_ALIGN;
  if (int rc = check_arch()) return rc;
  // K % 64 == 0 makes every row a whole number of 16-byte vectors of kernel-width codes
  const int64_t n_vec = N * K * kernel_bits(bits) / 8 / 16;
  const unsigned blocks = static_cast<unsigned>((n_vec + 255) / 256);
  uint4* dst = static_cast<uint4*>(prepared);
  const uint8_t* stream = reinterpret_cast<const uint8_t*>(wq);
  switch (bits) {
    case 4: interleave_codes_kernel<4><<<blocks, 256, 0, st>>>(reinterpret_cast<const uint4*>(wq), dst, n_vec); break;
    case 8: interleave_codes_kernel<8><<<blocks, 256, 0, st>>>(reinterpret_cast<const uint4*>(wq), dst, n_vec); break;
    case 3: widen_codes_kernel<3><<<blocks, 256, 0, st>>>(stream, dst, n_vec); break;
    case 5: widen_codes_kernel<5><<<blocks, 256, 0, st>>>(stream, dst, n_vec); break;
    default: widen_codes_kernel<6><<<blocks, 256, 0, st>>>(stream, dst, n_vec); break;
  }
  MFX_CUDA_TRY(cudaGetLastError());
  const int G = static_cast<int>(K / 64);
  uint32_t* sb = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(prepared) + codes_bytes_padded(N, K, bits));
  dim3 grid(static_cast<unsigned>((N + 31) / 32), static_cast<unsigned>((G + 31) / 32));
  pack_scales_kernel<<<grid, 256, 0, st>>>(scales, biases, sb_dtype, static_cast<int>(N), G, sb);
  MFX_CUDA_TRY(cudaGetLastError());
  return MFX_OK;
}

// The kernel of qmm_t.cu (weights as the tensor-memory operand) is the slower of the two on every shape measured
// (about 1050 against 1300 TFLOP/s on the single-linear configuration); it serves the tensor-parallel scatter
// epilogue, whose stores it can issue as contiguous runs along the output row, and, for side-by-side timing, every
// call without a low-rank term when the environment says MFX_QMM_KERNEL=tmem.
static bool tmem_operand_kernel() {
  static const bool on = [] {
    const char* v = getenv("MFX_QMM_KERNEL");
    return v && strcmp(v, "tmem") == 0;
  }();
  return on;
}

int run(const mfx_qlinear_args& a, cudaStream_t st) {
  const bool scatter = a.epilogue == MFX_EPI_PEER_SCATTER;
  if (!a.x || (!a.y && !scatter)) return MFX_ERR_NULL;
  if (!valid_bits(a.bits) || a.group_size != 64) return MFX_ERR_UNSUPPORTED_BITS;
  const int kb = kernel_bits(a.bits);   // width of the prepared codes: 4 (from 3 or 4) or 8 (from 5, 6 or 8)
  if (a.rows <= 0 || a.batch <= 0 || a.N <= 0 || a.K <= 0) return MFX_ERR_SHAPE;
  if (a.K % 64 != 0 || a.N % 8 != 0) return MFX_ERR_SHAPE;
  if (a.rows > (1 << 30) || a.N > (1 << 30) || a.K > (1 << 30) || a.batch > (1 << 20)) return MFX_ERR_TOO_LARGE;
  if (a.bias && !valid_dtype(a.bias_dtype)) return MFX_ERR_DTYPE;
  if (!scatter && a.y_dtype != MFX_BF16 && a.y_dtype != MFX_F32) return MFX_ERR_DTYPE;
  if (a.epilogue < MFX_EPI_NONE || a.epilogue > MFX_EPI_PEER_SCATTER) return MFX_ERR_SHAPE;
  if (scatter) {
    const mfx_tp_scatter* sc = a.scatter;
    if (!sc || !sc->done_counter) return MFX_ERR_NULL;
    if (sc->world < 1 || sc->world > MFX_TP_MAX_WORLD || sc->rank < 0 || sc->rank >= sc->world) return MFX_ERR_SHAPE;
    if (sc->rows_per_rank <= 0 || sc->row_offset < 0 || sc->D != a.N) return MFX_ERR_SHAPE;
    if (sc->row_offset + a.rows > sc->rows_per_rank * sc->world) return MFX_ERR_SHAPE;
    for (int r = 0; r < sc->world; ++r)
      if (!sc->dst[r] || !sc->flags[r]) return MFX_ERR_NULL;
    if (a.lora_r > 0 || a.N % 16 != 0) return MFX_ERR_SHAPE;   // no low-rank term; 32-byte stores of 16 columns
  }
  if (a.epilogue == MFX_EPI_SWIGLU && a.N % 16 != 0) return MFX_ERR_SHAPE;
  const void* prepared = a.prepared;
  if (!prepared) {
    if (!a.wq || !a.scales || !a.biases || !a.workspace) return MFX_ERR_NULL;
    if (a.workspace_bytes < prepared_bytes(a.N, a.K, a.bits, a.group_size)) return MFX_ERR_SHAPE;
  } else if ((reinterpret_cast<uintptr_t>(prepared) & 255u) != 0) {
    return MFX_ERR_ALIGN;
  }
  if (a.epilogue == MFX_EPI_GATE_RESIDUAL) {
    if (!a.gate || !a.residual) return MFX_ERR_NULL;
    if (!valid_dtype(a.gate_dtype)) return MFX_ERR_DTYPE;
    const size_t es = dtype_size(a.y_dtype);
    if (!aligned16(a.residual) || (a.res_row_stride * es) % 16 != 0 || (a.res_batch_stride * es) % 16 != 0)
      return MFX_ERR_ALIGN;
  }
  {
    const size_t es = dtype_size(a.y_dtype);
    if (!scatter && (!aligned16(a.y) || (a.y_row_stride * es) % 16 != 0 || (a.y_batch_stride * es) % 16 != 0))
      return MFX_ERR_ALIGN;
    if (!aligned16(a.x) || (a.x_row_stride * 2) % 16 != 0 || (a.x_batch_stride * 2) % 16 != 0) return MFX_ERR_ALIGN;
  }
  const bool low_rank = a.lora_r > 0;
  if (a.lora_r < 0) return MFX_ERR_SHAPE;
  if (low_rank) {
    if (!a.lora_t || !a.lora_b) return MFX_ERR_NULL;
    if (a.lora_ld <= 0 || a.lora_ld % 64 != 0 || a.lora_r > a.lora_ld || a.lora_ld > 1024) return MFX_ERR_SHAPE;
    if (!aligned16(a.lora_t) || !aligned16(a.lora_b) || (a.lora_t_row_stride * 2) % 16 != 0 ||
        (a.lora_t_batch_stride * 2) % 16 != 0 || a.lora_t_row_stride < a.lora_ld)
      return MFX_ERR_ALIGN;
  }
  if (int rc = check_arch()) return rc;
  if (!prepared) {
    if (int rc = prepare(a.wq, a.scales, a.biases, a.sb_dtype, a.N, a.K, a.bits, a.group_size, a.workspace,
                         a.workspace_bytes, st))
      return rc;
    prepared = a.workspace;
  }
  if (!low_rank && !scatter && qmv::eligible(a)) return qmv::run(a, prepared, codes_bytes_padded(a.N, a.K, a.bits), st);
  if (!low_rank && tmem_operand_kernel()) return qmmt::run(a, prepared, codes_bytes_padded(a.N, a.K, a.bits), st);
  const void* codes = prepared;
  const void* sb_packed = static_cast<const uint8_t*>(prepared) + codes_bytes_padded(a.N, a.K, a.bits);

  CUtensorMap tx, tw, tsb, tt, tlb;
  {
    const uint64_t dims[3] = {static_cast<uint64_t>(a.K), static_cast<uint64_t>(a.rows),
                              static_cast<uint64_t>(a.batch)};
    // a single sample may carry a zero batch stride; the tensor map still wants a valid (>0) one
    const uint64_t bstride = a.batch > 1 ? static_cast<uint64_t>(a.x_batch_stride) * 2
                                         : static_cast<uint64_t>(a.x_row_stride) * 2 * a.rows;
    const uint64_t strides[2] = {static_cast<uint64_t>(a.x_row_stride) * 2, bstride};
    const uint32_t box[3] = {BK, BM, 1};
    if (int rc = encode_tmap(&tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a.x, dims, strides, box,
                             CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  {
    const uint64_t words_per_row = static_cast<uint64_t>(a.K) * kb / 32;
    const uint64_t dims[2] = {words_per_row, static_cast<uint64_t>(a.N)};
    const uint64_t strides[1] = {words_per_row * 4};
    const uint32_t box[2] = {static_cast<uint32_t>(BK * kb / 32), BN_HALF};  // each CTA of a pair: 128 weight rows
    if (int rc = encode_tmap(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, codes, dims, strides, box,
                             kb == 4 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_64B))
      return rc;
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(a.N), static_cast<uint64_t>(a.K / 64)};
    const uint64_t strides[1] = {static_cast<uint64_t>(a.N) * 4};
    const uint32_t box[2] = {BN_HALF, 1};
    if (int rc = encode_tmap(&tsb, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, sb_packed, dims, strides, box,
                             CU_TENSOR_MAP_SWIZZLE_NONE))
      return rc;
  }
  if (low_rank) {
    const uint64_t dims[3] = {static_cast<uint64_t>(a.lora_ld), static_cast<uint64_t>(a.rows),
                              static_cast<uint64_t>(a.batch)};
    const uint64_t bstride = a.batch > 1 ? static_cast<uint64_t>(a.lora_t_batch_stride) * 2
                                         : static_cast<uint64_t>(a.lora_t_row_stride) * 2 * a.rows;
    const uint64_t strides[2] = {static_cast<uint64_t>(a.lora_t_row_stride) * 2, bstride};
    const uint32_t box[3] = {BK, BM, 1};
    if (int rc = encode_tmap(&tt, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a.lora_t, dims, strides, box,
                             CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
    // the dense tile takes the place of the packed codes in shared memory: same bytes per row (32 or 64), same swizzle
    const uint64_t bdims[2] = {static_cast<uint64_t>(a.lora_ld), static_cast<uint64_t>(a.N)};
    const uint64_t bstrides[1] = {static_cast<uint64_t>(a.lora_ld) * 2};
    const uint32_t bbox[2] = {static_cast<uint32_t>(4 * kb), BN_HALF};
    if (int rc = encode_tmap(&tlb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.lora_b, bdims, bstrides, bbox,
                             kb == 4 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_64B))
      return rc;
  } else {
    tt = tx;   // never read: the kernel runs no extension stage
    tlb = tw;
  }
  Params p;
  p.ext_r = low_rank ? static_cast<int>((a.lora_r + 15) / 16 * 16) : 0;
  p.num_ext = low_rank ? (p.ext_r + GPS * 4 * kb - 1) / (GPS * 4 * kb) : 0;
  p.rows = static_cast<int>(a.rows);
  p.batch = static_cast<int>(a.batch);
  p.N = static_cast<int>(a.N);
  p.K = static_cast<int>(a.K);
  p.tiles_m_per_sample = static_cast<int>((a.rows + 2 * BM - 1) / (2 * BM));  // a pair covers 256 activation rows
  p.tiles_m = p.tiles_m_per_sample * p.batch;
  p.tiles_n = static_cast<int>((a.N + BN - 1) / BN);
  const int64_t total = static_cast<int64_t>(p.tiles_m) * p.tiles_n;
  if (total > (1ll << 30)) return MFX_ERR_TOO_LARGE;
  p.total_tiles = static_cast<int>(total);
  {
    // bands of weight rows that stay L2-resident while every activation tile passes over them: 32 MB leaves room
    // for the activation and output tiles in flight even if each die's half of the L2 keeps its own copy
    const int64_t n_tile_bytes = static_cast<int64_t>(BN) * (a.K * kb / 8 + a.K / 64 * 4);
    const int64_t bands = (n_tile_bytes * p.tiles_n + (32ll << 20) - 1) / (32ll << 20);
    p.band_n = static_cast<int>((p.tiles_n + bands - 1) / bands);
    if (p.band_n < 1) p.band_n = 1;
  }
  p.bias = a.bias;
  p.bias_dtype = a.bias_dtype;
  p.epilogue = a.epilogue;
  p.gate = a.gate;
  p.gate_dtype = a.gate_dtype;
  p.gate_batch_stride = a.gate_batch_stride;
  p.residual = a.residual;
  p.res_row_stride = a.res_row_stride;
  p.res_batch_stride = a.res_batch_stride;
  p.y = a.y;
  p.y_row_stride = a.y_row_stride;
  p.y_batch_stride = a.y_batch_stride;
  p.sc_world = 0;
  if (scatter) {
    const mfx_tp_scatter& sc = *a.scatter;
    p.sc_world = sc.world;
    p.sc_rank = sc.rank;
    p.sc_rows_per_rank = sc.rows_per_rank;
    p.sc_row_offset = sc.row_offset;
    for (int r = 0; r < sc.world; ++r) {
      p.sc_dst[r] = static_cast<__nv_bfloat16*>(sc.dst[r]);
      p.sc_flags[r] = sc.flags[r];
    }
    p.sc_done = sc.done_counter;
  }
  const int pairs = device_sm_count() / 2;
  const bool f32_out = a.y_dtype == MFX_F32 && !scatter;
  const int grid = 2 * (p.total_tiles < pairs ? p.total_tiles : pairs);
  const bool f32 = f32_out;
  if (kb == 4) {
    // the scatter epilogue's staging tile takes the room of the third dequantized-weight stage
    if (scatter) return launch<4, FMT_BF16, 3, 2, __nv_bfloat16>(tx, tw, tsb, tt, tlb, p, grid, st);
    return f32 ? launch<4, FMT_BF16, 3, 3, float>(tx, tw, tsb, tt, tlb, p, grid, st)
               : launch<4, FMT_BF16, 3, 3, __nv_bfloat16>(tx, tw, tsb, tt, tlb, p, grid, st);
  }
  return f32 ? launch<8, FMT_BF16, 3, 2, float>(tx, tw, tsb, tt, tlb, p, grid, st)
             : launch<8, FMT_BF16, 3, 2, __nv_bfloat16>(tx, tw, tsb, tt, tlb, p, grid, st);
}

// ---------------------------------------------------------------- allocation-free variant
// Scratch for mfx_qlinear_static_scratch: the prepared form of ONE weight. It is part of the library image,
// so every GPU that loads the library carries these bytes until the process exits. In host code the name
// below is only a handle: the device address is obtained per device with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[MFX_STATIC_SCRATCH_BYTES];

// Device address of g_static_scratch on the current device (looked up once per device).
int static_scratch_address(void** out) {
  static std::mutex mu;
  static void* cached[64];
  int dev = 0;
  MFX_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return MFX_ERR_TOO_LARGE;
  std::lock_guard<std::mutex> lk(mu);
  if (cached[dev] == nullptr) {
    void* ptr = nullptr;
    MFX_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_scratch));
    if (ptr == nullptr) {
      set_cuda_error_text("cudaGetSymbolAddress returned a null address for the static scratch");
      return MFX_ERR_CUDA;
    }
    cached[dev] = ptr;
  }
  *out = cached[dev];
  return MFX_OK;
}

}  // namespace qmm
}  // namespace mfx

extern "C" {

int mfx_qlinear_ex(const mfx_qlinear_args* args, void* stream) {
  if (!args) return MFX_ERR_NULL;
  return mfx::qmm::run(*args, static_cast<cudaStream_t>(stream));
}

size_t mfx_qlinear_prepared_bytes(int64_t N, int64_t K, int bits, int group_size) {
  return mfx::qmm::prepared_bytes(N, K, bits, group_size);
}

int mfx_qlinear_prepare(const uint32_t* wq, const void* scales, const void* biases, int sb_dtype, int64_t N,
                        int64_t K, int bits, int group_size, void* prepared, size_t prepared_bytes, void* stream) {
  return mfx::qmm::prepare(wq, scales, biases, sb_dtype, N, K, bits, group_size, prepared, prepared_bytes,
                           static_cast<cudaStream_t>(stream));
}

int mfx_qlinear(const void* x, int64_t M, int64_t K, int64_t ldx, const uint32_t* wq, const void* scales,
                const void* biases, int sb_dtype, int64_t N, int bits, int group_size, const void* bias,
                int bias_dtype, void* y, int y_dtype, int64_t ldy, void* workspace, size_t workspace_bytes,
                void* stream) {
  mfx_qlinear_args a;
  memset(&a, 0, sizeof(a));
  a.x = x;
  a.x_row_stride = ldx;
  a.rows = M;
  a.batch = 1;
  a.K = K;
  a.N = N;
  a.wq = wq;
  a.scales = scales;
  a.biases = biases;
  a.sb_dtype = sb_dtype;
  a.bits = bits;
  a.group_size = group_size;
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  a.bias = bias;
  a.bias_dtype = bias_dtype;
  a.epilogue = MFX_EPI_NONE;
  a.y = y;
  a.y_dtype = y_dtype;
  a.y_row_stride = ldy;
  return mfx_qlinear_ex(&a, stream);
}

int mfx_qlinear_static_scratch(const void* x, int64_t M, int64_t K, int64_t ldx, const uint32_t* wq,
                               const void* scales, const void* biases, int sb_dtype, int64_t N, int bits,
                               int group_size, const void* bias, int bias_dtype, void* y, int y_dtype, int64_t ldy,
                               void* stream) {
  const size_t need = mfx::qmm::prepared_bytes(N, K, bits, group_size);
  if (need == 0) {
    if (!mfx::valid_bits(bits) || group_size != 64) return MFX_ERR_UNSUPPORTED_BITS;
    return MFX_ERR_SHAPE;
  }
  if (need > static_cast<size_t>(MFX_STATIC_SCRATCH_BYTES)) {
    mfx::set_cuda_error_text("mfx_qlinear_static_scratch: the prepared weight does not fit the built-in scratch");
    return MFX_ERR_TOO_LARGE;
  }
  void* scratch = nullptr;
  if (int rc = mfx::qmm::static_scratch_address(&scratch)) return rc;
  return mfx_qlinear(x, M, K, ldx, wq, scales, biases, sb_dtype, N, bits, group_size, bias, bias_dtype, y, y_dtype,
                     ldy, scratch, static_cast<size_t>(MFX_STATIC_SCRATCH_BYTES), stream);
}

}  // extern "C"
