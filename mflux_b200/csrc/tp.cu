// Tensor-parallel exchange kernels: the elementwise half of a transformer block fused with its collectives over
// peer-mapped memory (NVLink), for the row-split / column-split quantized linears of the Qwen-Image blocks
// (reference arithmetic: src/mflux/models/qwen/model/qwen_transformer/qwen_transformer_block.py:27-76; the split
// over devices has no counterpart in the single-device reference).
//
// Every rank owns `rows_per_rank` consecutive rows of each sample's joint sequence [text rows, image rows]. A
// row-split linear leaves on each rank a partial sum of the whole sequence; the matmul's epilogue stores each
// partial row into a slot of the owning rank's memory (see MFX_EPI_PEER_SCATTER in qmm_t.cu). tp_fuse_kernel then
// runs on the owned rows only:
//     wait until every rank's partials for this exchange have arrived (counters written by the matmuls),
//     x += gate * (sum over ranks of the partials + bias)          (gated residual, float32 stream)
//     n = LayerNorm(x) * (1 + scale) + shift                       (the next sub-layer's modulated pre-norm)
//     store n as bf16 into the full-sequence activation buffer of EVERY rank (plain peer stores) and bump a
//     counter on every rank once all rows are out.
// That is reduce-scatter + gated residual + norm + all-gather in one pass over 1/world of the rows; the next
// column-split matmul waits for the counters (tp_wait_kernel). Counters only grow: a consumer waits for ">=
// target", so nothing is ever reset while a peer may still write. Every wait is bounded and reports through the
// device status word. No multicast, no TMA on peer memory: peers are reached with ordinary st.global.
#include <cuda_bf16.h>

#include "host_util.cuh"
#include "ptx.cuh"

namespace mfx {
namespace tp {

constexpr int THREADS = 128;
constexpr int MAX_D = 4096;
constexpr int E = 8;   // elements per thread and vector: 16-byte bf16 stores to the peers
constexpr int MAXV = MAX_D / E / THREADS;

enum : int { DEV_TIMEOUT_TP = 110 };

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(int* p, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded wait until *flag >= target. Returns false (after recording the failure) when it gives up.
__device__ __forceinline__ bool wait_counter(const int* flag, int target) {
  for (uint32_t i = 0; i < (1u << 22); ++i) {
    if (ld_acquire_sys(flag) - target >= 0) return true;   // difference: the counters may wrap
    __nanosleep(i < 32 ? 64 : 512);
  }
  record_failure(DEV_TIMEOUT_TP);
  return false;
}

__device__ __forceinline__ float ld_scalar(const void* p, int dtype, int64_t i) {
  if (dtype == MFX_F32) return __ldg(static_cast<const float*>(p) + i);
  if (dtype == MFX_BF16) return __bfloat162float(__ldg(static_cast<const __nv_bfloat16*>(p) + i));
  return __half2float(__ldg(static_cast<const __half*>(p) + i));
}
__device__ __forceinline__ void ldv(const void* p, int dtype, int64_t off, float (&o)[E]) {
  if (dtype == MFX_BF16) {
    const uint4 raw = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p) + off);
    const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
    for (int i = 0; i < E; ++i) o[i] = __bfloat162float(h[i]);
  } else if (dtype == MFX_F32) {
    const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(p) + off);
    const float4 b = *(reinterpret_cast<const float4*>(static_cast<const float*>(p) + off) + 1);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w;
    o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
  } else {
#pragma unroll
    for (int i = 0; i < E; ++i) o[i] = ld_scalar(p, dtype, off + i);
  }
}
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  return (red[0] + red[1]) + (red[2] + red[3]);
}

// One 128-thread block per owned row (sample b, local row i); joint row t = rank * rows_per_rank + i. Rows at or
// beyond `seq` are padding: they only take part in the completion count.
__global__ void __launch_bounds__(THREADS) tp_fuse_kernel(const mfx_tp_fuse_args p) {
  __shared__ float red[3][4];
  __shared__ int wait_ok;
  const int tid = threadIdx.x;
  const int64_t R = p.rows_per_rank;
  const int b = static_cast<int>(blockIdx.x / R);
  const int i = static_cast<int>(blockIdx.x % R);
  const int64_t t = static_cast<int64_t>(p.rank) * R + i;
  const bool live = t < p.seq;
  const int seg = t < p.split ? 0 : 1;
  const int nvec = static_cast<int>(p.D / E);

  if (p.partials != nullptr) {
    if (tid == 0) wait_ok = 1;
    __syncthreads();
    const int target = p.rs_target + (p.epoch_base ? __ldg(p.epoch_base) : 0);
    if (tid < p.world && !wait_counter(p.rs_flags + tid, target)) wait_ok = 0;
    __syncthreads();
    if (!wait_ok) return;   // the failure is recorded; nothing is signalled, the peers' waits will run out too
  }

  if (live) {
    float* x = p.x + (static_cast<int64_t>(b) * R + i) * p.D;
    float v[MAXV][E];
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < MAXV; ++k) {
      const int c = tid + THREADS * k;
      if (c < nvec) {
        ldv(x, MFX_F32, static_cast<int64_t>(c) * E, v[k]);
        if (p.partials != nullptr) {
          float acc[E] = {};
          for (int src = 0; src < p.world; ++src) {   // fixed order: the sum does not depend on arrival order
            const __nv_bfloat16* part = static_cast<const __nv_bfloat16*>(p.partials) +
                                        ((static_cast<int64_t>(src) * p.batch + b) * R + i) * p.D;
            // written by a peer over NVLink: read around L1
            const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(part + static_cast<int64_t>(c) * E));
            const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&raw);
#pragma unroll
            for (int j = 0; j < E; ++j) acc[j] += __bfloat162float(h[j]);
          }
          float bias[E] = {}, gate[E];
          if (p.bias[seg]) ldv(p.bias[seg], p.bias_dtype, static_cast<int64_t>(c) * E, bias);
          ldv(p.gate[seg], p.mod_dtype, b * p.mod_batch_stride + static_cast<int64_t>(c) * E, gate);
#pragma unroll
          for (int j = 0; j < E; ++j) v[k][j] += gate[j] * (acc[j] + bias[j]);
          float4* xo = reinterpret_cast<float4*>(x + static_cast<int64_t>(c) * E);
          xo[0] = make_float4(v[k][0], v[k][1], v[k][2], v[k][3]);
          xo[1] = make_float4(v[k][4], v[k][5], v[k][6], v[k][7]);
        }
#pragma unroll
        for (int j = 0; j < E; ++j) sum += v[k][j];
      }
    }
    if (p.scale[seg] != nullptr) {
      const float mean = block_sum(sum, red[0]) / static_cast<float>(p.D);
      float sq = 0.f;
#pragma unroll
      for (int k = 0; k < MAXV; ++k) {
        const int c = tid + THREADS * k;
        if (c < nvec) {
#pragma unroll
          for (int j = 0; j < E; ++j) {
            const float d = v[k][j] - mean;
            sq += d * d;
          }
        }
      }
      const float rstd = rsqrtf(block_sum(sq, red[1]) / static_cast<float>(p.D) + p.eps);
      const int64_t row_off = (static_cast<int64_t>(b) * p.seq_pad + t) * p.D;
#pragma unroll
      for (int k = 0; k < MAXV; ++k) {
        const int c = tid + THREADS * k;
        if (c < nvec) {
          float sc[E], sh[E];
          const int64_t moff = b * p.mod_batch_stride + static_cast<int64_t>(c) * E;
          ldv(p.scale[seg], p.mod_dtype, moff, sc);
          ldv(p.shift[seg], p.mod_dtype, moff, sh);
          __nv_bfloat162 h[E / 2];
#pragma unroll
          for (int j = 0; j < E / 2; ++j)
            h[j] = __floats2bfloat162_rn((v[k][2 * j] - mean) * rstd * (1.0f + sc[2 * j]) + sh[2 * j],
                                         (v[k][2 * j + 1] - mean) * rstd * (1.0f + sc[2 * j + 1]) + sh[2 * j + 1]);
          const uint4 out = *reinterpret_cast<uint4*>(h);
          if (p.push_local_only) {
            *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.push_dst[p.rank]) + row_off +
                                      static_cast<int64_t>(c) * E) = out;
          } else {
            for (int dst = 0; dst < p.world; ++dst)
              *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.push_dst[dst]) + row_off +
                                        static_cast<int64_t>(c) * E) = out;
          }
        }
      }
    }
  }

  if (p.push_local_only || (p.scale[0] == nullptr && p.scale[1] == nullptr)) return;   // nobody waits for this call
  // completion: every thread's peer stores are ordered before the block's arrival; the last block tells the peers
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    const int done = atomicAdd(p.done_counter, 1);
    if (done == static_cast<int>(gridDim.x) - 1) {
      *p.done_counter = 0;
      __threadfence_system();
      for (int dst = 0; dst < p.world; ++dst) red_release_sys_add(p.ag_flags[dst], 1);
    }
  }
}

__global__ void tp_wait_kernel(const int* flags, int world, int target, const int* epoch_base) {
  if (epoch_base) target += __ldg(epoch_base);
  if (static_cast<int>(threadIdx.x) < world) wait_counter(flags + threadIdx.x, target);
}

struct SignalArgs {
  int* flags[MFX_TP_MAX_WORLD];
};
__global__ void tp_signal_kernel(const SignalArgs a, int world) {
  if (static_cast<int>(threadIdx.x) < world) {
    __threadfence_system();
    red_release_sys_add(a.flags[threadIdx.x], 1);
  }
}

MFX_DEFINE_STATUS_READER(read_status)

}  // namespace tp
}  // namespace mfx

extern "C" {

int mfx_tp_fuse(const mfx_tp_fuse_args* a, void* stream) {
  using namespace mfx;
  if (!a) return MFX_ERR_NULL;
  if (a->world < 1 || a->world > MFX_TP_MAX_WORLD || a->rank < 0 || a->rank >= a->world) return MFX_ERR_SHAPE;
  if (a->batch <= 0 || a->rows_per_rank <= 0 || a->D <= 0 || a->D % 8 != 0 || a->D > tp::MAX_D) return MFX_ERR_SHAPE;
  if (a->seq <= 0 || a->seq > a->seq_pad || a->rows_per_rank * a->world != a->seq_pad) return MFX_ERR_SHAPE;
  if (a->split < 0 || a->split > a->seq) return MFX_ERR_SHAPE;
  if (a->batch * a->rows_per_rank > (1ll << 30)) return MFX_ERR_TOO_LARGE;
  if (!a->x || !a->done_counter) return MFX_ERR_NULL;
  if (!aligned16(a->x) || (a->partials && !aligned16(a->partials))) return MFX_ERR_ALIGN;
  if (!valid_dtype(a->mod_dtype) || (a->mod_batch_stride * static_cast<int64_t>(dtype_size(a->mod_dtype))) % 16 != 0)
    return MFX_ERR_DTYPE;
  const bool norm = a->scale[0] != nullptr || a->scale[1] != nullptr;
  for (int s = 0; s < 2; ++s) {
    if (a->partials && !a->gate[s]) return MFX_ERR_NULL;
    if (norm && (!a->scale[s] || !a->shift[s])) return MFX_ERR_NULL;
    if (a->bias[s] && !valid_dtype(a->bias_dtype)) return MFX_ERR_DTYPE;
  }
  if (a->partials && !a->rs_flags) return MFX_ERR_NULL;
  if (norm)
    for (int r = 0; r < a->world; ++r)
      if (!a->push_dst[r] || !a->ag_flags[r] || !aligned16(a->push_dst[r])) return MFX_ERR_NULL;
  if (int rc = check_arch()) return rc;
  const unsigned blocks = static_cast<unsigned>(a->batch * a->rows_per_rank);
  tp::tp_fuse_kernel<<<blocks, tp::THREADS, 0, static_cast<cudaStream_t>(stream)>>>(*a);
  MFX_CUDA_TRY(cudaGetLastError());
  return MFX_OK;
}

int mfx_tp_signal(int* const* flags, int world, void* stream) {
  using namespace mfx;
  if (!flags) return MFX_ERR_NULL;
  if (world < 1 || world > MFX_TP_MAX_WORLD) return MFX_ERR_SHAPE;
  tp::SignalArgs a;
  for (int r = 0; r < world; ++r) {
    if (!flags[r]) return MFX_ERR_NULL;
    a.flags[r] = flags[r];
  }
  if (int rc = check_arch()) return rc;
  tp::tp_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(a, world);
  MFX_CUDA_TRY(cudaGetLastError());
  return MFX_OK;
}

int mfx_tp_wait(const int* flags, int world, int target, const int* epoch_base, void* stream) {
  using namespace mfx;
  if (!flags) return MFX_ERR_NULL;
  if (world < 1 || world > MFX_TP_MAX_WORLD) return MFX_ERR_SHAPE;
  if (int rc = check_arch()) return rc;
  tp::tp_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flags, world, target, epoch_base);
  MFX_CUDA_TRY(cudaGetLastError());
  return MFX_OK;
}

}  // extern "C"
