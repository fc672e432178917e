// Streaming filter-gradient kernels: host-side entry (see bwd_stream.cuh).
#include "bwd_stream.cuh"

namespace ddf {

bool bwd_stream_supported(const Problem&) { return false; }

size_t bwd_stream_workspace(const Problem&, int) { return 0; }

int bwd_stream_filters(const Problem&, const void*, const void*, const void*, const void*, void*,
                       void*, void*, int, int*, cudaStream_t, int* launches) {
    if (launches) *launches = 0;
    return kNotHandled;
}

}  // namespace ddf
