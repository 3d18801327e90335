// Tensor-core prefill kernel for block-sparse attention (16-bit element types).
#include "bsa_common.cuh"

namespace hipattn {

int bsa_mma(const hipattn_bsa_params_t& p, cudaStream_t stream, bool* handled) {
  *handled = false;
  return HIPATTN_OK;
}

}  // namespace hipattn
