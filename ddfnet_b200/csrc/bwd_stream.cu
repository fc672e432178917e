// Streaming filter-gradient kernels: host-side entry (see bwd_stream.cuh).
#include "bwd_stream.cuh"

#include "bwd_stream_impl.cuh"

namespace ddf {

// Pixels per thread: the largest instantiated P that divides the output width and
// lets one plane's threads (padded to whole warps) fit the CTA.  0 = not covered.
static int bwd_pixels(const Problem& p, int sm_count, BwdGeometry& g) {
    if (p.dtype == DDF_B200_F64) return 0;
    const int k = p.k, d = p.d, s = p.s;
    static const int cand[3] = {4, 2, 1};
    for (int ci = 0; ci < 3; ++ci) {
        const int P = cand[ci];
        bool built = false;
        if (k == 3 && d == 1) built = (s == 1 || s == 2);
        else if (k == 3 && d == 2 && s == 1) built = P >= 2;
        else if (k == 5 && (d == 1 || d == 2) && s == 1) built = P == 2;
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
    BwdArgs a{go, x, cf, sf, gcf, gsf, workspace, p, sm_count, fault, P, device};
    switch (p.dtype) {
        case DDF_B200_F32: return bwd_dispatch<float>(a, st, launches);
        case DDF_B200_F16: return bwd_dispatch<__half>(a, st, launches);
        case DDF_B200_BF16: return bwd_dispatch<__nv_bfloat16>(a, st, launches);
        default: return kNotHandled;
    }
}

}  // namespace ddf
