// Streaming filter-gradient kernels: host-side entry (see bwd_stream.cuh).
#include <atomic>

#include "bwd_stream.cuh"

#include "bwd_stream_impl.cuh"

namespace ddf {

// Pixels per thread: the largest instantiated P that divides the output width and
// lets one plane's threads (padded to whole warps) fit the CTA.  0 = not covered.
static int bwd_pixels(const Problem& p, int sm_count, BwdGeometry& g) {
    if (p.dtype == DDF_B200_F64) return 0;
    const int k = p.k, d = p.d, s = p.s;
    // 8 comes last: it is the two-launch form, used only where no smaller P fits a plane
    // into one CTA's threads
    static const int cand[4] = {4, 2, 1, 8};
    for (int ci = 0; ci < 4; ++ci) {
        const int P = cand[ci];
        bool built = false;
        if (P == 8) built = (k == 3 && d == 1 && s == 1);
        else if (k == 3 && d == 1) built = (s == 1 || s == 2);
        else if (k == 3 && d == 2 && s == 1) built = P >= 2;
        else if (k == 5 && (d == 1 || d == 2) && s == 1) built = P == 2 || P == 4;
        if (!built) continue;
        // the element-wise (sub-word) path of 2-byte types covers a halo of one only
        if (P * s * (p.dtype == DDF_B200_F32 ? 4 : 2) < 4 && (k - 1) / 2 * d > 1) continue;
        if (!bwd_geometry(p, P, sm_count, g)) continue;
        return P;
    }
    return 0;
}

bool bwd_stream_supported(const Problem& p) {
    BwdGeometry g;
    return bwd_pixels(p, 148, g) > 0;
}

size_t bwd_stream_workspace(const Problem& p, int sm_count) {
    BwdGeometry g;
    if (bwd_pixels(p, sm_count, g) == 0) return 0;
    return (bwd_workspace_bytes(p, g) + 255) / 256 * 256;
}

int bwd_stream_filters(const Problem& p, const void* go, const void* x, const void* cf,
                       const void* sf, void* gcf, void* gsf, void* workspace, int sm_count,
                       int* fault, int device, cudaStream_t st, int* launches) {
    *launches = 0;
    BwdGeometry g;
    const int P = bwd_pixels(p, sm_count, g);
    if (P == 0) return kNotHandled;
    BwdArgs a{go, x, cf, sf, gcf, gsf, workspace, p, sm_count, fault, P, device, p.k == 3};
    switch (p.dtype) {
        case DDF_B200_F32: return bwd_dispatch<float>(a, st, launches);
        case DDF_B200_F16: return bwd_dispatch<__half>(a, st, launches);
        case DDF_B200_BF16: return bwd_dispatch<__nv_bfloat16>(a, st, launches);
        default: return kNotHandled;
    }
}

}  // namespace ddf

// ---------------------------------------------------------------------------
// Backward for callers that cannot allocate device memory.
//
// The filter-gradient kernel needs scratch for its float partial sums.  The
// regular entry point takes that scratch from the caller; some callers have no
// way to provide it: code running under a fixed memory plan or inside another
// framework's allocator-free region (a serving runtime that sized its arena at
// start-up, a plugin called where cudaMalloc is forbidden because it would
// synchronise the device or fragment a tightly packed pool).  For them the
// scratch lives in this library's own image: a file-scope device array of
// kStaticScratchBytes that every GPU loading the library holds until exit.
//
// In host code the array's NAME is only a host-side handle, not a device
// address (a kernel handed it would fault, or scribble over host memory where
// the GPU can reach it).  The device address is obtained once per device, with
// that device current, by cudaGetSymbolAddress, and that pointer is what the
// kernels receive.
// ---------------------------------------------------------------------------
namespace ddf {

constexpr size_t kStaticScratchBytes = 16u << 20;  // 16 MiB per GPU
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

static std::atomic<void*> g_static_scratch_ptr[64];

// Device address of the static scratch on the current device (set up on first use).
static int static_scratch_address(int device, void** out) {
    if (device < 0 || device >= 64) return DDF_B200_E_DEVICE;
    void* ptr = g_static_scratch_ptr[device].load(std::memory_order_acquire);
    if (ptr == nullptr) {
        const cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_static_scratch);
        if (e != cudaSuccess) return (int)e;
        g_static_scratch_ptr[device].store(ptr, std::memory_order_release);
    }
    *out = ptr;
    return 0;
}

}  // namespace ddf

extern "C" {

size_t ddf_b200_backward_noalloc_limit(void) { return ddf::kStaticScratchBytes; }

int ddf_b200_backward_noalloc(const void* go, const void* x, const void* cf, const void* sf,
                              void* gx, void* gcf, void* gsf, int B, int C, int H, int W, int k,
                              int d, int s, int combine, int dtype, void* stream) {
    using namespace ddf;
    // Argument checks only: the regular entry point with no gradient requested
    // validates everything and launches nothing.
    int rc = ddf_b200_backward(go, x, cf, sf, nullptr, nullptr, nullptr, nullptr, 0, B, C, H, W, k, d,
                               s, combine, dtype, DDF_B200_VARIANT_AUTO, stream);
    if (rc) return rc;

    Problem p;
    p.B = B; p.C = C; p.H = H; p.W = W; p.OH = H / s; p.OW = W / s;
    p.k = k; p.d = d; p.s = s; p.combine = combine; p.dtype = dtype;
    int sm_count = 0, index = 0;
    int* fault = nullptr;
    rc = device_facts(&sm_count, &fault, &index);
    if (rc) return rc;

    // The same kernel choice as ddf_b200_backward makes under AUTO, so that both entry
    // points give bit-identical results.  Only the spatial-filter gradient uses scratch:
    // refuse, before anything is launched, if it would need more than the array holds.
    const bool streaming = (gcf || gsf) &&
                           ddf_b200_plan(B, C, H, W, k, d, s, combine, dtype, 1) == DDF_B200_VARIANT_STREAM;
    if (streaming && gsf && bwd_stream_workspace(p, sm_count) > kStaticScratchBytes)
        return DDF_B200_E_SCRATCH_LIMIT;

    // grad-x needs no scratch: regular entry point, filter gradients not requested.
    if (gx) {
        rc = ddf_b200_backward(go, x, cf, sf, gx, nullptr, nullptr, nullptr, 0, B, C, H, W, k, d, s,
                               combine, dtype, DDF_B200_VARIANT_AUTO, stream);
        if (rc) return rc;
    }
    if (!gcf && !gsf) return 0;

    if (streaming) {
        void* scratch = nullptr;
        if (gsf) {
            rc = static_scratch_address(index, &scratch);
            if (rc) return rc;
        }
        int launches = 0;
        rc = bwd_stream_filters(p, go, x, cf, sf, gcf, gsf, scratch, sm_count, fault, index,
                                reinterpret_cast<cudaStream_t>(stream), &launches);
        if (rc != kNotHandled) return rc;
    }
    // Outside the streaming kernel's range: the generic kernels use no scratch at all.
    return ddf_b200_backward(go, x, cf, sf, nullptr, gcf, gsf, nullptr, 0, B, C, H, W, k, d, s,
                             combine, dtype, DDF_B200_VARIANT_GENERIC, stream);
}

}  // extern "C"
