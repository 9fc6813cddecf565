// Tensor-core (tcgen05 + TMEM) route of the sparse-conv contraction. Placeholder
// dispatch until the kernel lands: reports every shape as unsupported so that the
// CUDA-core route serves it.
#include "common.cuh"

namespace lat {

bool tc_conv_supported(int, int, int, int, int, int) { return false; }

size_t tc_conv_workspace_bytes(int, int, int) { return 0; }

int run_tc_conv(
    const void*, int, int, long long, const void*, int, const uint32_t*, const void*,
    const void*, int, int, int, int, const int32_t*, const int32_t*, int, const int32_t*,
    const int32_t*, int, int, const void*, const int32_t*, void*, void*, size_t, int32_t*,
    cudaStream_t
) {
    return fail(LAT_UNSUPPORTED, "tensor-core convolution route is not built.");
}

} // namespace lat
