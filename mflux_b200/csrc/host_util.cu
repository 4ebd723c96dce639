// Error bookkeeping, architecture check and TMA tensor-map encoding for libmfx.
#include "host_util.cuh"

#include <mutex>
#include <stdio.h>

namespace mfx {

static thread_local char t_err[512] = "";

void set_cuda_error(const char* what, cudaError_t e) {
  snprintf(t_err, sizeof(t_err), "%s: %s", what, cudaGetErrorString(e));
}
void set_cuda_error_text(const char* text) { snprintf(t_err, sizeof(t_err), "%s", text); }

int check_arch() {
  int dev = 0;
  MFX_CUDA_TRY(cudaGetDevice(&dev));
  static std::mutex mu;
  static int cached_major[64];
  static bool have[64];
  int major = 0;
  {
    std::lock_guard<std::mutex> lk(mu);
    if (dev >= 0 && dev < 64 && have[dev]) {
      major = cached_major[dev];
    } else {
      MFX_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
      if (dev >= 0 && dev < 64) {
        cached_major[dev] = major;
        have[dev] = true;
      }
    }
  }
  return major == 10 ? MFX_OK : MFX_ERR_ARCH;
}

int device_sm_count() {
  static std::mutex mu;
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  std::lock_guard<std::mutex> lk(mu);
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

int ensure_dynamic_smem(const void* func, int bytes, SmemConfigured& rec) {
  static std::mutex mu;
  int dev = 0;
  MFX_CUDA_TRY(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lk(mu);
  if (dev >= 0 && dev < 64 && rec.done[dev]) return MFX_OK;
  MFX_CUDA_TRY(cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  if (dev >= 0 && dev < 64) rec.done[dev] = true;
  return MFX_OK;
}

typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static encode_tiled_fn get_encode() {
  static encode_tiled_fn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = reinterpret_cast<encode_tiled_fn>(p);
  });
  return fn;
}

int encode_tmap(CUtensorMap* out, CUtensorMapDataType dt, int rank, const void* base, const uint64_t* dims,
                const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle) {
  encode_tiled_fn fn = get_encode();
  if (!fn) {
    set_cuda_error_text("cuTensorMapEncodeTiled entry point unavailable");
    return MFX_ERR_CUDA;
  }
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bx[5];
  cuuint32_t es[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) {
    if (strides_bytes[i] % 16 != 0) return MFX_ERR_ALIGN;
    gstr[i] = strides_bytes[i];
  }
  if (!aligned16(base)) return MFX_ERR_ALIGN;
  CUresult r = fn(out, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim, gstr, bx, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[128];
    snprintf(buf, sizeof(buf), "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
    set_cuda_error_text(buf);
    return MFX_ERR_CUDA;
  }
  return MFX_OK;
}

}  // namespace mfx

extern "C" {

int mfx_version(void) { return MFX_VERSION; }

const char* mfx_status_str(int status) {
  switch (status) {
    case MFX_OK: return "ok";
    case MFX_ERR_SHAPE: return "bad shape (zero/negative size or divisibility rule violated)";
    case MFX_ERR_ALIGN: return "pointer or stride not 16-byte aligned";
    case MFX_ERR_UNSUPPORTED_BITS: return "unsupported bits/group size (bits must be 3, 4, 5, 6 or 8, group 64)";
    case MFX_ERR_DTYPE: return "unsupported dtype for this entry point";
    case MFX_ERR_ARCH: return "device is not sm_100 (compute capability 10.x)";
    case MFX_ERR_CUDA: return "CUDA call failed";
    case MFX_ERR_NULL: return "required pointer is NULL";
    case MFX_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
    case MFX_ERR_TOO_LARGE: return "size exceeds a fixed limit of this entry point";
    default: return "unknown status";
  }
}

const char* mfx_last_cuda_error(void) { return mfx::t_err; }

}  // extern "C"
