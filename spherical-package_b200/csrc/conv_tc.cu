// bf16 tensor-core (tcgen05) path of the mapped convolution family -- stub stage.
#include "common.cuh"
#include "conv_internal.h"

namespace sph {
size_t tc_workspace_bytes(int, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int) { return 0; }
int tc_conv_forward(const void *, const void *, const void *, const void *, const void *, void *, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int, void *, size_t, cudaStream_t) { return SPH_ERR_UNSUPPORTED; }
int tc_conv_backward_input(const void *, const void *, const void *, void *, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, void *, size_t, cudaStream_t) { return SPH_ERR_UNSUPPORTED; }
int tc_conv_backward_weight(const void *, const void *, const void *, const void *, void *, void *, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int, void *, size_t, cudaStream_t) { return SPH_ERR_UNSUPPORTED; }
int tc_tconv_forward(const void *, const void *, const void *, const void *, void *, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, void *, size_t, cudaStream_t) { return SPH_ERR_UNSUPPORTED; }
int tc_tconv_backward_input(const void *, const void *, const void *, const void *, void *, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int, void *, size_t, cudaStream_t) { return SPH_ERR_UNSUPPORTED; }
int tc_tconv_backward_weight(const void *, const void *, const void *, const void *, void *, void *, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int, void *, size_t, cudaStream_t) { return SPH_ERR_UNSUPPORTED; }
}  // namespace sph
