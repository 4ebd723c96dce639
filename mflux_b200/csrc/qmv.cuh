// Small-M (at most 16 rows) quantized linear over the prepared weight blob; see qmv.cu.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#include "../../include/mfx.h"

namespace mfx {
namespace qmv {

// True when the call can take the weight-streaming path: one sample, at most 16 rows, no epilogue beyond SiLU.
bool eligible(const mfx_qlinear_args& a);
// prepared = blob of mfx_qlinear_prepare; codes_bytes = size of its (padded) code section.
int run(const mfx_qlinear_args& a, const void* prepared, size_t codes_bytes, cudaStream_t st);

}  // namespace qmv
}  // namespace mfx
