// Quantized linear layer for large M with the dequantized weights as the TENSOR-MEMORY operand.
//
// Same contract as qmm.cu (Y[M,N] = X[M,K] . dequant(Wq[N,K])^T + bias with fused epilogues, replacing
// mlx.nn.QuantizedLinear.__call__ -> mx.quantized_matmul of the reference's transformer blocks, e.g.
// src/mflux/models/flux/model/flux_transformer/joint_attention.py:14-21, feed_forward.py:8-9), computed as the
// transposed product  Y^T[n, m] = sum_k W[n, k] X[m, k]:
//   A operand = dequantized weights, 128 rows per CTA, written by the dequantizer warps straight into tensor
//               memory (tcgen05.st) and read from there by the tensor cores;
//   B operand = activations, 96 tokens per CTA (192 per CTA pair), streamed by TMA into shared memory.
// The kernel in qmm.cu keeps both operands in shared memory (per 128-deep stage and CTA: 512 wavefronts of
// tensor-core operand reads, 320 of dequantized-weight stores, 330 of TMA writes, 150 of code loads, against 1024
// cycles of MMA); here a stage moves 190 wavefronts of operand reads, 265 of TMA writes and 70 of code loads
// against 768 cycles of MMA. Measured, this kernel is nevertheless the slower one (about 1050 against 1300 TFLOP/s
// on M 4096, N 12288, K 3072): tensor memory leaves room for two A slots only beside two accumulators, and with
// the MMAs and the dequantizer arithmetic switched off the kernel still takes 0.85 us per stage, i.e. it is bound
// by the latency of the slot hand-off between the dequantizers of both CTAs and the issuing thread (four slots of
// one group each, with twice the commits, were slower still). It is kept for the epilogue that only its layout
// serves well: thread = output column, so a warp writes 32 consecutive values of one output row, which makes the
// tensor-parallel scatter to peer memory (MFX_EPI_PEER_SCATTER) one 64-byte run per store instruction.
// Per CTA, 512 threads, persistent over tiles of 256 weight rows x 192 tokens per pair:
//   warp 0      TMA producer: per stage (two quantization groups = 128 k) its 96 tokens of X (counted on the
//               leader's barrier), the packed codes of its 128 weight rows and their (scale, bias) pairs
//   warp 1      allocates all 512 tensor-memory columns (two 192-column accumulators + two 64-column A slots);
//               in the leader CTA issues tcgen05.mma.cta_group::2 (M = 256 weight rows, N = 192 tokens, K = 16)
//   warps 4-7   epilogue: thread = output column n (tensor-memory lane), tensor-memory columns = tokens; bias,
//               activation, gated residual, then one scalar store per token (a warp writes 32 consecutive n)
//   warps 8-15  dequantizers: thread = weight row, one quantization group per warp and stage, 64 values ->
//               32 packed bf16 pairs -> one tcgen05.st into the A slot
// All mbarrier waits are bounded.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "host_util.cuh"
#include "ptx.cuh"
#include "qmm_common.cuh"
#include "qmm_t.cuh"

namespace mfx {
namespace qmmt {

using qmm::dequant_w4;
using qmm::dequant_w8_f32;
using qmm::gelu_erf;
using qmm::gelu_tanh;
using qmm::load_scalar;
using qmm::silu;

constexpr int WR = 128;        // weight rows per CTA (tensor-memory lanes); 256 per pair
constexpr int NT = 192;        // tokens per pair tile (the MMA's N)
constexpr int NT_HALF = 96;    // tokens each CTA loads
constexpr int BK = 64;         // one quantization group
constexpr int GPS = 2;         // groups per pipeline stage
constexpr int SA = 2;          // A-operand slots in tensor memory (one stage each)
constexpr int NUM_DQ_WARPS = 8;
constexpr int FIRST_DQ_WARP = 8;
constexpr int FIRST_EPI_WARP = 4;
constexpr int NUM_THREADS = (FIRST_DQ_WARP + NUM_DQ_WARPS) * 32;
constexpr int X_TILE_BYTES = NT_HALF * BK * 2;   // 12 KiB per group (a multiple of the 1 KiB swizzle atom)
constexpr int SB_TILE_BYTES = WR * 4;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t COL_D = 0;                    // two accumulators of NT fp32 columns
constexpr uint32_t COL_A = 2 * NT;               // SA slots of GPS * 32 columns (2 bf16 along k per column)
constexpr uint32_t A_SLOT_COLS = GPS * BK / 2;

struct Params {
  int rows, batch, N, K;
  int tiles_m_per_sample, tiles_m, tiles_n, total_tiles;
  int band_n;
  const void* bias;
  int bias_dtype;
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

template <int BITS, int ST>
struct Smem {
  static constexpr int WQ_TILE_BYTES = WR * BK * BITS / 8;
  static constexpr int X_STAGE = GPS * X_TILE_BYTES;
  static constexpr int WQ_STAGE = GPS * WQ_TILE_BYTES;
  static constexpr int SB_STAGE = GPS * SB_TILE_BYTES;
  static constexpr int OFF_X = 0;
  static constexpr int OFF_WQ = OFF_X + ST * X_STAGE;
  static constexpr int OFF_SB = OFF_WQ + ST * WQ_STAGE;
  static constexpr int OFF_BAR = OFF_SB + ST * SB_STAGE;
  static constexpr int NUM_BARS = 3 * ST + 2 * SA + 4;
  static constexpr int OFF_TMEM = OFF_BAR + NUM_BARS * 8;
  static constexpr int TOTAL = OFF_TMEM + 16;
  static constexpr int DYN_BYTES = TOTAL + 1024;
};

// Same order as the shared-memory kernel: bands of weight tiles that fit in L2, token tile by token tile inside
// a band with the weight-tile index running fastest.
__device__ __forceinline__ void tile_coords(const Params& p, int tile, int& tm, int& tn) {
  const int per_band = p.tiles_m * p.band_n;
  const int band = tile / per_band;
  const int r = tile - band * per_band;
  const int n_first = band * p.band_n;
  const int width = min(p.band_n, p.tiles_n - n_first);
  tm = r / width;
  tn = n_first + r - tm * width;
}

template <int BITS, int ST, typename OUT, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
qmm_t_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
             const __grid_constant__ CUtensorMap tmap_sb, const Params p) {
  using L = Smem<BITS, ST>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const uint32_t x_s = smem_base + L::OFF_X;
  const uint32_t wq_s = smem_base + L::OFF_WQ;
  const uint32_t sb_s = smem_base + L::OFF_SB;
  const uint32_t bar0 = smem_base + L::OFF_BAR;
  auto w_full = [&](int s) { return bar0 + 8u * s; };              // local: codes + pairs landed
  auto x_full = [&](int s) { return bar0 + 8u * (ST + s); };       // leader: X halves of both CTAs landed
  auto t_empty = [&](int s) { return bar0 + 8u * (2 * ST + s); };  // local: TMA stage may be refilled
  constexpr int B0 = 3 * ST;
  auto a_full = [&](int s) { return bar0 + 8u * (B0 + s); };            // leader: A slot written in both CTAs
  auto a_empty = [&](int s) { return bar0 + 8u * (B0 + SA + s); };      // local: A slot consumed
  auto acc_full = [&](int s) { return bar0 + 8u * (B0 + 2 * SA + s); };       // local
  auto acc_empty = [&](int s) { return bar0 + 8u * (B0 + 2 * SA + 2 + s); };  // leader
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + L::OFF_TMEM);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = p.K / BK;
  const int num_st = (num_kb + GPS - 1) / GPS;  // a ragged last stage reads TMA zero fill for its missing group
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < ST; ++s) {
      mbar_init(w_full(s), 1);
      mbar_init(x_full(s), 1);
      mbar_init(t_empty(s), 1 + NUM_DQ_WARPS);  // MMA commit (X tile) + every local dequantizer warp (codes)
    }
    for (int s = 0; s < SA; ++s) {
      mbar_init(a_full(s), 2 * NUM_DQ_WARPS);
      mbar_init(a_empty(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(acc_full(s), 1);
      mbar_init(acc_empty(s), 8);
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
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    int st = 0;
    uint32_t ph = 0;
    bool ok = true;
    for (int tile = pair; tile < p.total_tiles && ok; tile += num_pairs) {
      int tm, tn;
      tile_coords(p, tile, tm, tn);
      const int b = tm / p.tiles_m_per_sample;
      const int r0 = (tm % p.tiles_m_per_sample) * NT + static_cast<int>(rank) * NT_HALF;
      const int n0 = tn * (2 * WR) + static_cast<int>(rank) * WR;
      for (int s = 0; s < num_st; ++s) {
        if (!mbar_wait_sleep(t_empty(st), ph ^ 1u, DEV_TIMEOUT_TMA_EMPTY)) {
          ok = false;
          break;
        }
        if (lane == 0) {
          if (rank == 0) mbar_arrive_expect_tx(x_full(st), 2 * L::X_STAGE);
          mbar_arrive_expect_tx(w_full(st), L::WQ_STAGE + L::SB_STAGE);
#pragma unroll
          for (int g = 0; g < GPS; ++g) {
            const int kb = s * GPS + g;
            tma_load_2d(wq_s + st * L::WQ_STAGE + g * L::WQ_TILE_BYTES, &tmap_w, w_full(st), kb * (BK * BITS / 32),
                        n0);
            tma_load_2d(sb_s + st * L::SB_STAGE + g * SB_TILE_BYTES, &tmap_sb, w_full(st), n0, kb);
            tma_load_3d_pair(x_s + st * L::X_STAGE + g * X_TILE_BYTES, &tmap_x, x_full(st), kb * BK, r0, b);
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
      constexpr uint32_t IDESC = make_idesc(FMT_BF16, FMT_BF16, 2 * WR, NT);  // M = 256 weight rows, N = 192 tokens
      int st = 0, sa = 0;
      uint32_t ph_t = 0, ph_a = 0;
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
        const uint32_t d_tmem = tmem_base + COL_D + a * NT;
        for (int s = 0; s < num_st; ++s) {
          if (!mbar_wait(x_full(st), ph_t, DEV_TIMEOUT_TMA_FULL) || !mbar_wait(a_full(sa), ph_a, DEV_TIMEOUT_DQ_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          if (lane == 0) {
#pragma unroll
            for (int g = 0; g < GPS; ++g) {
              const uint64_t bdesc = smem_desc_sw128(x_s + st * L::X_STAGE + g * X_TILE_BYTES);
              const uint32_t a_tmem = tmem_base + COL_A + sa * A_SLOT_COLS + g * (BK / 2);
#pragma unroll
              for (int k4 = 0; k4 < BK / 16; ++k4) {
                // 8 tensor-memory columns and 32 bytes of the 128-byte swizzle atom per 16-deep k step
                umma_f16_ts_pair(d_tmem, a_tmem + 8 * k4, bdesc + 2 * k4, IDESC, (s | g | k4) != 0 ? 1u : 0u);
              }
            }
            umma_commit_pair(t_empty(st));
            umma_commit_pair(a_empty(sa));
            if (s == num_st - 1) umma_commit_pair(acc_full(a));
          }
          __syncwarp();
          if (++st == ST) {
            st = 0;
            ph_t ^= 1u;
          }
          if (++sa == SA) {
            sa = 0;
            ph_a ^= 1u;
          }
        }
      }
    }
  } else if (warp >= FIRST_DQ_WARP) {
    // ------------------------------------------------------------ dequantizers
    // Warp dq serves group dq / 4 of the stage and the 32 weight rows of tensor-memory lane quarter dq % 4 (a warp
    // may only touch the lanes 32 * (warp % 4) .. + 31, and FIRST_DQ_WARP is a multiple of 4).
    const int dq = warp - FIRST_DQ_WARP;
    const int grp = dq >> 2;
    const int quarter = dq & 3;
    const int row = quarter * 32 + lane;
    constexpr int ROW_BYTES = BK * BITS / 8;   // packed bytes per row per group: 32 or 64
    constexpr int RD_CHUNKS = ROW_BYTES / 16;  // 2 or 4
    // the packed tile is loaded with the TMA swizzle whose span equals one row (see qmm.cu)
    const uint32_t rd_sw = (static_cast<uint32_t>(row * ROW_BYTES) >> 7) & (RD_CHUNKS - 1);
    const uint8_t* rd_base = smem_gen + L::OFF_WQ + grp * L::WQ_TILE_BYTES + row * ROW_BYTES;
    uint32_t rd_off[RD_CHUNKS];
#pragma unroll
    for (int h = 0; h < RD_CHUNKS; ++h) rd_off[h] = (static_cast<uint32_t>(h) ^ rd_sw) << 4;
    const uint32_t* sb_base = reinterpret_cast<const uint32_t*>(smem_gen + L::OFF_SB + grp * SB_TILE_BYTES) + row;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + COL_A + grp * (BK / 2);
    int st = 0, sa = 0;
    uint32_t ph_t = 0, ph_a = 0;
    bool ok = true;
    for (int tile = pair; tile < p.total_tiles && ok; tile += num_pairs) {
      for (int s = 0; s < num_st; ++s) {
        if (!mbar_wait_sleep(a_empty(sa), ph_a ^ 1u, DEV_TIMEOUT_DQ_EMPTY) ||
            !mbar_wait(w_full(st), ph_t, DEV_TIMEOUT_TMA_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sbv = sb_base[st * (L::SB_STAGE / 4)];
        const uint8_t* src = rd_base + st * L::WQ_STAGE;
        uint32_t vals[32];
        if (BITS == 4) {
          const uint32_t s2 = __byte_perm(sbv, sbv, 0x1010);  // (scale, scale)
          const uint32_t b2 = __byte_perm(sbv, sbv, 0x3232);  // (bias, bias)
#pragma unroll
          for (int h = 0; h < RD_CHUNKS; ++h) {
            const uint4 pk = *reinterpret_cast<const uint4*>(src + rd_off[h]);
            const uint32_t wds[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint4 d = dequant_w4(wds[j], s2, b2);   // 8 values of k = 32 h + 8 j ..
              vals[16 * h + 4 * j + 0] = d.x;
              vals[16 * h + 4 * j + 1] = d.y;
              vals[16 * h + 4 * j + 2] = d.z;
              vals[16 * h + 4 * j + 3] = d.w;
            }
          }
        } else {
          const uint32_t sf = sbv << 16, bf = sbv & 0xFFFF0000u;
          uint64_t sc2, bi2;
          asm("mov.b64 %0, {%1, %1};" : "=l"(sc2) : "r"(sf));
          asm("mov.b64 %0, {%1, %1};" : "=l"(bi2) : "r"(bf));
#pragma unroll
          for (int h = 0; h < RD_CHUNKS; ++h) {
            const uint4 pk = *reinterpret_cast<const uint4*>(src + rd_off[h]);
            const uint32_t wds[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint2 d = dequant_w8_f32(wds[j], sc2, bi2);   // 4 values of k = 16 h + 4 j ..
              vals[8 * h + 2 * j + 0] = d.x;
              vals[8 * h + 2 * j + 1] = d.y;
            }
          }
        }
        tmem_st_32x32(t_lane + sa * A_SLOT_COLS, vals);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive_leader(a_full(sa));
          mbar_arrive(t_empty(st));
        }
        if (++st == ST) {
          st = 0;
          ph_t ^= 1u;
        }
        if (++sa == SA) {
          sa = 0;
          ph_a ^= 1u;
        }
      }
    }
  } else if (warp >= FIRST_EPI_WARP) {
    // ------------------------------------------------------------ epilogue (thread = output column n)
    const int q = warp & 3;
    bool ok = true;
    int it = 0;
    for (int tile = pair; tile < p.total_tiles && ok; tile += num_pairs, ++it) {
      const int a = it & 1;
      const uint32_t aph = (it >> 1) & 1;
      int tm, tn;
      tile_coords(p, tile, tm, tn);
      const int b = tm / p.tiles_m_per_sample;
      const int t0 = (tm % p.tiles_m_per_sample) * NT;   // first token of the tile inside its sample
      const int n = tn * (2 * WR) + static_cast<int>(rank) * WR + q * 32 + lane;
      const bool n_ok = n < p.N;
      const float bias_v = (p.bias != nullptr && n_ok) ? load_scalar(p.bias, p.bias_dtype, n) : 0.f;
      float gate_v = 0.f;
      if (EPI == MFX_EPI_GATE_RESIDUAL && n_ok) gate_v = load_scalar(p.gate, p.gate_dtype, b * p.gate_batch_stride + n);
      // SwiGLU: lane pairs (2j, 2j+1) hold (gate, up) of output column n / 2
      const int n_out = EPI == MFX_EPI_SWIGLU ? (n >> 1) : n;
      const bool writer = n_ok && (EPI != MFX_EPI_SWIGLU || (lane & 1) == 0);
      OUT* ycol = static_cast<OUT*>(p.y) + b * p.y_batch_stride + n_out;
      const OUT* rcol = nullptr;
      if (EPI == MFX_EPI_GATE_RESIDUAL) rcol = static_cast<const OUT*>(p.residual) + b * p.res_batch_stride + n;
      if (!mbar_wait_sleep(acc_full(a), aph, DEV_TIMEOUT_ACC_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + COL_D + a * NT;
      const int valid = min(NT, p.rows - t0);   // tokens of this tile that exist
#pragma unroll 1
      for (int c = 0; c < NT / 32; ++c) {
        if (c * 32 >= valid) break;   // uniform over the CTA pair: nothing of this chunk is stored
        uint32_t acc[32];
        tmem_ld_32x32(t_addr + c * 32, acc);
        tmem_ld_wait();
        float res[32];
        if (EPI == MFX_EPI_GATE_RESIDUAL) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int t = c * 32 + j;
            res[j] = 0.f;
            if (n_ok && t < valid) {
              if constexpr (sizeof(OUT) == 4) res[j] = rcol[static_cast<int64_t>(t0 + t) * p.res_row_stride];
              else res[j] = __bfloat162float(rcol[static_cast<int64_t>(t0 + t) * p.res_row_stride]);
            }
          }
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int t = c * 32 + j;
          float v = __uint_as_float(acc[j]) + bias_v;
          if (EPI == MFX_EPI_GELU_ERF) v = gelu_erf(v);
          else if (EPI == MFX_EPI_GELU_TANH) v = gelu_tanh(v);
          else if (EPI == MFX_EPI_SILU) v = silu(v);
          else if (EPI == MFX_EPI_GATE_RESIDUAL) v = res[j] + gate_v * v;
          if (EPI == MFX_EPI_SWIGLU) {
            const float up = __shfl_xor_sync(0xffffffffu, v, 1);
            v = silu(v) * up;
          }
          if (EPI == MFX_EPI_PEER_SCATTER) {
            if (n_ok && t < valid) {
              const int64_t tj = p.sc_row_offset + t0 + t;       // row of the joint sequence
              const int64_t owner = tj / p.sc_rows_per_rank;
              const int64_t local = tj - owner * p.sc_rows_per_rank;
              p.sc_dst[owner][((static_cast<int64_t>(p.sc_rank) * p.batch + b) * p.sc_rows_per_rank + local) * p.N +
                              n] = __float2bfloat16_rn(v);
            }
          } else if (writer && t < valid) {
            OUT* dst = ycol + static_cast<int64_t>(t0 + t) * p.y_row_stride;
            if constexpr (sizeof(OUT) == 4) *dst = v;
            else *dst = __float2bfloat16_rn(v);
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
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

MFX_DEFINE_STATUS_READER(read_status)

template <int BITS, int ST, typename OUT, int EPI>
int launch_epi(const CUtensorMap& tx, const CUtensorMap& tw, const CUtensorMap& tsb, const Params& p, int grid,
               cudaStream_t st) {
  using L = Smem<BITS, ST>;
  auto kern = qmm_t_kernel<BITS, ST, OUT, EPI>;
  static SmemConfigured configured;
  if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kern), L::DYN_BYTES, configured)) return rc;
  kern<<<grid, NUM_THREADS, L::DYN_BYTES, st>>>(tx, tw, tsb, p);
  MFX_CUDA_TRY(cudaGetLastError());
  return MFX_OK;
}

template <int BITS, int ST, typename OUT>
int launch(int epilogue, const CUtensorMap& tx, const CUtensorMap& tw, const CUtensorMap& tsb, const Params& p,
           int grid, cudaStream_t st) {
  switch (epilogue) {
    case MFX_EPI_GELU_ERF: return launch_epi<BITS, ST, OUT, MFX_EPI_GELU_ERF>(tx, tw, tsb, p, grid, st);
    case MFX_EPI_GELU_TANH: return launch_epi<BITS, ST, OUT, MFX_EPI_GELU_TANH>(tx, tw, tsb, p, grid, st);
    case MFX_EPI_GATE_RESIDUAL: return launch_epi<BITS, ST, OUT, MFX_EPI_GATE_RESIDUAL>(tx, tw, tsb, p, grid, st);
    case MFX_EPI_SILU: return launch_epi<BITS, ST, OUT, MFX_EPI_SILU>(tx, tw, tsb, p, grid, st);
    case MFX_EPI_SWIGLU: return launch_epi<BITS, ST, OUT, MFX_EPI_SWIGLU>(tx, tw, tsb, p, grid, st);
    case MFX_EPI_PEER_SCATTER:
      if constexpr (sizeof(OUT) == 2) return launch_epi<BITS, ST, OUT, MFX_EPI_PEER_SCATTER>(tx, tw, tsb, p, grid, st);
      else return MFX_ERR_DTYPE;
    default: return launch_epi<BITS, ST, OUT, MFX_EPI_NONE>(tx, tw, tsb, p, grid, st);
  }
}

// Arguments were validated by the caller (qmm::run); `prepared` is the weight's prepared blob.
int run(const mfx_qlinear_args& a, const void* prepared, size_t codes_bytes, cudaStream_t st) {
  const int kb = kernel_bits(a.bits);
  const void* codes = prepared;
  const void* sb_packed = static_cast<const uint8_t*>(prepared) + codes_bytes;
  CUtensorMap tx, tw, tsb;
  {
    const uint64_t dims[3] = {static_cast<uint64_t>(a.K), static_cast<uint64_t>(a.rows),
                              static_cast<uint64_t>(a.batch)};
    const uint64_t bstride = a.batch > 1 ? static_cast<uint64_t>(a.x_batch_stride) * 2
                                         : static_cast<uint64_t>(a.x_row_stride) * 2 * a.rows;
    const uint64_t strides[2] = {static_cast<uint64_t>(a.x_row_stride) * 2, bstride};
    const uint32_t box[3] = {BK, NT_HALF, 1};
    if (int rc = encode_tmap(&tx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, a.x, dims, strides, box,
                             CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  {
    const uint64_t words_per_row = static_cast<uint64_t>(a.K) * kb / 32;
    const uint64_t dims[2] = {words_per_row, static_cast<uint64_t>(a.N)};
    const uint64_t strides[1] = {words_per_row * 4};
    const uint32_t box[2] = {static_cast<uint32_t>(BK * kb / 32), WR};
    if (int rc = encode_tmap(&tw, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, codes, dims, strides, box,
                             kb == 4 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_64B))
      return rc;
  }
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(a.N), static_cast<uint64_t>(a.K / 64)};
    const uint64_t strides[1] = {static_cast<uint64_t>(a.N) * 4};
    const uint32_t box[2] = {WR, 1};
    if (int rc = encode_tmap(&tsb, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, sb_packed, dims, strides, box,
                             CU_TENSOR_MAP_SWIZZLE_NONE))
      return rc;
  }
  Params p;
  p.rows = static_cast<int>(a.rows);
  p.batch = static_cast<int>(a.batch);
  p.N = static_cast<int>(a.N);
  p.K = static_cast<int>(a.K);
  p.tiles_m_per_sample = static_cast<int>((a.rows + NT - 1) / NT);
  p.tiles_m = p.tiles_m_per_sample * p.batch;
  p.tiles_n = static_cast<int>((a.N + 2 * WR - 1) / (2 * WR));
  const int64_t total = static_cast<int64_t>(p.tiles_m) * p.tiles_n;
  if (total > (1ll << 30)) return MFX_ERR_TOO_LARGE;
  p.total_tiles = static_cast<int>(total);
  {
    const int64_t n_tile_bytes = static_cast<int64_t>(2 * WR) * (a.K * kb / 8 + a.K / 64 * 4);
    const int64_t bands = (n_tile_bytes * p.tiles_n + (32ll << 20) - 1) / (32ll << 20);
    p.band_n = static_cast<int>((p.tiles_n + bands - 1) / bands);
    if (p.band_n < 1) p.band_n = 1;
  }
  p.bias = a.bias;
  p.bias_dtype = a.bias_dtype;
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
  if (a.epilogue == MFX_EPI_PEER_SCATTER) {
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
  const int grid = 2 * (p.total_tiles < pairs ? p.total_tiles : pairs);
  const bool f32 = a.y_dtype == MFX_F32 && a.epilogue != MFX_EPI_PEER_SCATTER;
  if (kb == 4) {
    return f32 ? launch<4, 5, float>(a.epilogue, tx, tw, tsb, p, grid, st)
               : launch<4, 5, __nv_bfloat16>(a.epilogue, tx, tw, tsb, p, grid, st);
  }
  return f32 ? launch<8, 5, float>(a.epilogue, tx, tw, tsb, p, grid, st)
             : launch<8, 5, __nv_bfloat16>(a.epilogue, tx, tw, tsb, p, grid, st);
}

}  // namespace qmmt
}  // namespace mfx
