// Host-side helpers shared by the C-ABI entry points: error bookkeeping, architecture check,
// TMA tensor-map encoding through the driver entry point (no link-time dependency on libcuda).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "../../include/mfx.h"

namespace mfx {

void set_cuda_error(const char* what, cudaError_t e);
void set_cuda_error_text(const char* text);
int check_arch();  // MFX_OK when the current device is compute capability 10.x

#define MFX_CUDA_TRY(expr)                      \
  do {                                          \
    cudaError_t _e = (expr);                    \
    if (_e != cudaSuccess) {                    \
      ::mfx::set_cuda_error(#expr, _e);         \
      return MFX_ERR_CUDA;                      \
    }                                           \
  } while (0)

inline size_t dtype_size(int dt) { return dt == MFX_F32 ? 4 : 2; }
inline bool valid_dtype(int dt) { return dt == MFX_F32 || dt == MFX_BF16 || dt == MFX_F16; }
// Code widths of the affine quantizer (the ones the reference's CLI offers).
inline bool valid_bits(int bits) { return bits == 3 || bits == 4 || bits == 5 || bits == 6 || bits == 8; }
// Width the matmul kernels unpack: 3-bit codes are widened to 4 bits, 5- and 6-bit codes to 8 bits when a weight
// is prepared, so that one dequantizer per kernel width serves all of them.
inline int kernel_bits(int bits) { return bits <= 4 ? 4 : 8; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Number of SMs of the current device (looked up once per device; 148 if the query fails).
int device_sm_count();

// Per-kernel record of the devices on which its dynamic shared-memory limit has been raised. The attribute belongs
// to (function, device), so every device needs the call once; a mutex makes concurrent host threads safe.
struct SmemConfigured {
  bool done[64] = {};
};
// cudaFuncSetAttribute(func, MaxDynamicSharedMemorySize, bytes) on the current device unless `rec` says it was done.
int ensure_dynamic_smem(const void* func, int bytes, SmemConfigured& rec);

// Encodes a tiled tensor map of `rank` dims (innermost first). strides_bytes[i] is the byte stride
// of dim i+1 (rank-1 entries, multiples of 16). Returns MFX_OK or an error status.
int encode_tmap(CUtensorMap* out, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims,
                const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle);

}  // namespace mfx
