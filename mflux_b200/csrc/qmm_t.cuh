// Large-M quantized linear with the dequantized weights as the tensor-memory operand; see qmm_t.cu.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#include "../../include/mfx.h"

namespace mfx {
namespace qmmt {

// `a` was validated by qmm::run; prepared = blob of mfx_qlinear_prepare, codes_bytes = size of its code section.
// Handles every epilogue; calls with a low-rank term stay with the shared-memory kernel.
int run(const mfx_qlinear_args& a, const void* prepared, size_t codes_bytes, cudaStream_t st);
int read_status(int* out, cudaStream_t stream);

}  // namespace qmmt
}  // namespace mfx
