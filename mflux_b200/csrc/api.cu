// Entry points that span several translation units.
#include "host_util.cuh"

namespace mfx {
namespace qmm {
int read_status(int* out, cudaStream_t stream);
}
namespace qmmt {
int read_status(int* out, cudaStream_t stream);
}
namespace attn {
int read_status(int* out, cudaStream_t stream);
}
namespace tp {
int read_status(int* out, cudaStream_t stream);
}
}  // namespace mfx

extern "C" {

int mfx_poll_device_status(int* status_out, void* stream) {
  if (!status_out) return MFX_ERR_NULL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int v = 0, v2 = 0, v3 = 0, v4 = 0;
  if (mfx::qmm::read_status(&v, st) != 0 || mfx::attn::read_status(&v2, st) != 0 ||
      mfx::qmmt::read_status(&v3, st) != 0 || mfx::tp::read_status(&v4, st) != 0) {
    mfx::set_cuda_error_text("reading the device status word failed");
    return MFX_ERR_CUDA;
  }
  if (v == 0) v = v2;
  if (v == 0) v = v3;
  if (v == 0) v = v4;
  *status_out = v;
  return v == 0 ? MFX_OK : MFX_ERR_DEVICE_TIMEOUT;
}

}  // extern "C"
