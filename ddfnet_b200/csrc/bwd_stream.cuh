// Streaming kernels for the two filter gradients (grad wrt the channel filter
// and wrt the spatial filter).  Declarations; the kernels live in
// bwd_stream_impl.cuh and are instantiated per element type in
// bwd_inst_<type>.cu.
#pragma once

#include "common.cuh"

namespace ddf {

// True when the streaming filter-gradient kernels cover this problem.
bool bwd_stream_supported(const Problem& p);

// Bytes of scratch bwd_stream_filters needs (float partial sums of the
// spatial-filter gradient, one slot per (CTA, sample) intersection).
size_t bwd_stream_workspace(const Problem& p, int sm_count);

// Enqueues the filter-gradient kernels.  gcf or gsf may be NULL.  Returns 0,
// kNotHandled, or a CUDA error; *launches receives the number of launches.
int bwd_stream_filters(const Problem& p, const void* go, const void* x, const void* cf,
                       const void* sf, void* gcf, void* gsf, void* workspace, int sm_count,
                       int* fault, int device, cudaStream_t st, int* launches);

// Defined in abi.cu: SM count, fault word and index of the current device.
int device_facts(int* sm_count, int** fault, int* index);

}  // namespace ddf
