// C ABI of libddf_b200.so (declared in include/ddf_b200.h): argument checks,
// kernel choice and launches.  No allocation, no host synchronisation, no
// exceptions cross this boundary; every entry point returns a status.
#include <atomic>

#include "bwd_stream.cuh"
#include "common.cuh"
#include "generic.cuh"
#include "ring_fwd.cuh"
#include "row_fwd.cuh"
#include "stream_fwd.cuh"

#include <cstdlib>

namespace ddf {

__device__ int g_fault_word = 0;

std::atomic<unsigned long long> g_launches{0};  // also counted from layout.cu
struct DeviceInfo {
    int sm_count = 0;
    int cc_major = 0;
    int* fault = nullptr;
    int index = 0;
    std::atomic<bool> ready{false};
};
static DeviceInfo g_dev[64];

// Per-device facts, fetched once per device.  Two threads may both fill the entry (with
// the same values); `ready` is published with release / read with acquire so that a thread
// that sees it set also sees the fields.
static int device_info(DeviceInfo*& out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return DDF_B200_E_DEVICE;
    DeviceInfo& di = g_dev[dev];
    if (!di.ready.load(std::memory_order_acquire)) {
        int sm = 0, major = 0;
        e = cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev);
        if (e != cudaSuccess) return (int)e;
        e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        if (e != cudaSuccess) return (int)e;
        void* fp = nullptr;
        e = cudaGetSymbolAddress(&fp, g_fault_word);
        if (e != cudaSuccess) return (int)e;
        di.sm_count = sm;
        di.cc_major = major;
        di.fault = reinterpret_cast<int*>(fp);
        di.index = dev;
        di.ready.store(true, std::memory_order_release);
    }
    if (di.cc_major != 10) return DDF_B200_E_DEVICE;
    out = &di;
    return 0;
}

// Per-device facts for other translation units of this library.
int device_facts(int* sm_count, int** fault, int* index) {
    DeviceInfo* di = nullptr;
    const int rc = device_info(di);
    if (rc) return rc;
    *sm_count = di->sm_count;
    *fault = di->fault;
    *index = di->index;
    return 0;
}

static int check_problem(int B, int C, int H, int W, int k, int d, int s, int combine, int dtype,
                         int variant, Problem& p) {
    if (B < 1 || C < 1 || H < 1 || W < 1) return DDF_B200_E_SHAPE;
    if (k < 1 || (k - 1) % 2 != 0 || d < 1 || s < 1) return DDF_B200_E_KERNEL;
    if (H / s < 1 || W / s < 1) return DDF_B200_E_SHAPE;
    if (combine != DDF_B200_MUL && combine != DDF_B200_ADD) return DDF_B200_E_COMBINE;
    if (dtype < DDF_B200_F32 || dtype > DDF_B200_F64) return DDF_B200_E_DTYPE;
    if (variant < DDF_B200_VARIANT_AUTO || variant > DDF_B200_VARIANT_STREAM) return DDF_B200_E_VARIANT;
    // The kernels index planes with 64-bit offsets but pixel positions inside a
    // plane, and B*C, with 32-bit integers.
    if ((long long)H * W > (1ll << 30) || (long long)B * C > (1ll << 30) ||
        (long long)k * k > 1024 || (long long)k * d > (1 << 20))
        return DDF_B200_E_TOO_LARGE;
    p.B = B; p.C = C; p.H = H; p.W = W;
    p.OH = H / s; p.OW = W / s;
    p.k = k; p.d = d; p.s = s;
    p.combine = combine; p.dtype = dtype;
    return 0;
}

static int grid_for(long long total, int threads, int sm_count) {
    long long blocks = (total + threads - 1) / threads;
    const long long cap = (long long)sm_count * 32;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

// ------------------------------------------------------------------ generic launches
template <typename T>
static int generic_forward_launch(const Problem& p, const void* x, const void* cf, const void* sf,
                                  void* out, int sm_count, cudaStream_t st) {
    const long long total = (long long)p.B * p.C * p.OH * p.OW;
    const int grid = grid_for(total, 256, sm_count);
    if (p.combine == DDF_B200_MUL)
        generic_forward<T, DDF_B200_MUL><<<grid, 256, 0, st>>>((const T*)x, (const T*)cf, (const T*)sf, (T*)out, p, total);
    else
        generic_forward<T, DDF_B200_ADD><<<grid, 256, 0, st>>>((const T*)x, (const T*)cf, (const T*)sf, (T*)out, p, total);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}

template <typename T>
static int generic_grad_x_launch(const Problem& p, const void* go, const void* cf, const void* sf,
                                 void* gx, int sm_count, cudaStream_t st) {
    // the down-sampling layers' case has a kernel of its own (no per-tap divisions)
    if (p.k == 3 && p.d == 1 && p.s == 2 && p.H == 2 * p.OH && p.W == 2 * p.OW && p.B <= 65535) {
        constexpr int CH = 16;
        dim3 grid((unsigned)((p.OH * p.OW + 255) / 256), (unsigned)((p.C + CH - 1) / CH), (unsigned)p.B);
        if (grid.y <= 65535u) {
            if (p.combine == DDF_B200_MUL)
                grad_x_k3s2<T, DDF_B200_MUL, CH><<<grid, 256, 0, st>>>((const T*)go, (const T*)cf, (const T*)sf, (T*)gx, p);
            else
                grad_x_k3s2<T, DDF_B200_ADD, CH><<<grid, 256, 0, st>>>((const T*)go, (const T*)cf, (const T*)sf, (T*)gx, p);
            g_launches.fetch_add(1, std::memory_order_relaxed);
            return (int)cudaGetLastError();
        }
    }
    const long long total = (long long)p.B * p.C * p.H * p.W;
    const int grid = grid_for(total, 256, sm_count);
    if (p.combine == DDF_B200_MUL)
        generic_grad_x<T, DDF_B200_MUL><<<grid, 256, 0, st>>>((const T*)go, (const T*)cf, (const T*)sf, (T*)gx, p, total);
    else
        generic_grad_x<T, DDF_B200_ADD><<<grid, 256, 0, st>>>((const T*)go, (const T*)cf, (const T*)sf, (T*)gx, p, total);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}

template <typename T>
static int generic_grad_filters_launch(const Problem& p, const void* go, const void* x,
                                       const void* cf, const void* sf, void* gcf, void* gsf,
                                       int sm_count, cudaStream_t st) {
    if (gsf) {
        const long long total = (long long)p.B * p.k * p.k * p.OH * p.OW;
        const int grid = grid_for(total, 256, sm_count);
        if (p.combine == DDF_B200_MUL)
            generic_grad_sf<T, DDF_B200_MUL><<<grid, 256, 0, st>>>((const T*)go, (const T*)x, (const T*)cf, (T*)gsf, p, total);
        else
            generic_grad_sf<T, DDF_B200_ADD><<<grid, 256, 0, st>>>((const T*)go, (const T*)x, (const T*)cf, (T*)gsf, p, total);
        g_launches.fetch_add(1, std::memory_order_relaxed);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    if (gcf) {
        const long long planes = (long long)p.B * p.C;
        long long blocks = planes < (long long)sm_count * 16 ? planes : (long long)sm_count * 16;
        if (p.combine == DDF_B200_MUL)
            generic_grad_cf<T, DDF_B200_MUL><<<(int)blocks, 128, 0, st>>>((const T*)go, (const T*)x, (const T*)sf, (T*)gcf, p, planes);
        else
            generic_grad_cf<T, DDF_B200_ADD><<<(int)blocks, 128, 0, st>>>((const T*)go, (const T*)x, (const T*)sf, (T*)gcf, p, planes);
        g_launches.fetch_add(1, std::memory_order_relaxed);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return (int)e;
    }
    return 0;
}

#define DDF_BY_DTYPE(dtype, CALL)                                     \
    switch (dtype) {                                                  \
        case DDF_B200_F32: { using T = float; return CALL; }          \
        case DDF_B200_F16: { using T = __half; return CALL; }         \
        case DDF_B200_BF16: { using T = __nv_bfloat16; return CALL; } \
        case DDF_B200_F64: { using T = double; return CALL; }         \
        default: return DDF_B200_E_DTYPE;                             \
    }

static int run_generic_forward(const Problem& p, const void* x, const void* cf, const void* sf,
                               void* out, int sm, cudaStream_t st) {
    DDF_BY_DTYPE(p.dtype, (generic_forward_launch<T>(p, x, cf, sf, out, sm, st)))
}
static int run_generic_grad_x(const Problem& p, const void* go, const void* cf, const void* sf,
                              void* gx, int sm, cudaStream_t st) {
    DDF_BY_DTYPE(p.dtype, (generic_grad_x_launch<T>(p, go, cf, sf, gx, sm, st)))
}
static int run_generic_grad_filters(const Problem& p, const void* go, const void* x, const void* cf,
                                    const void* sf, void* gcf, void* gsf, int sm, cudaStream_t st) {
    DDF_BY_DTYPE(p.dtype, (generic_grad_filters_launch<T>(p, go, x, cf, sf, gcf, gsf, sm, st)))
}

// ------------------------------------------------------------------ streaming choice
static int elem_size(int dtype) { return dtype == DDF_B200_F32 ? 4 : dtype == DDF_B200_F64 ? 8 : 2; }

// Pixels per thread for the streaming kernels: the largest instantiated P that
// divides the output width and keeps a whole plane within one CTA's threads.
// Returns 0 when the problem is outside the instantiated set.
static int stream_pixels(const Problem& p, bool bwdx) {
    if (p.dtype == DDF_B200_F64) return 0;
    const int k = p.k, d = p.d, s = p.s;
    if (bwdx && s != 1) return 0;
    if (p.W != p.OW * s) return 0;
    const int halo = (k - 1) / 2 * d;
    // 7 = a whole or half row of a 7- or 14-pixel-wide output (element-wise loads).
    static const int cand[5] = {8, 4, 7, 2, 1};
    for (int ci = 0; ci < 5; ++ci) {
        const int P = cand[ci];
        bool built = false;
        if (P == 7) built = k == 3 && d == 1 && (s == 1 || s == 2) && p.OW <= 14;
        else if (k == 3 && d == 1 && s == 1) built = true;
        else if (k == 3 && d == 1 && s == 2) built = P <= 4;
        else if (k == 3 && d == 2 && s == 1) built = P >= 2;
        else if (k == 5 && d == 1 && s == 1) built = P == 4 || P == 2;
        else if (k == 5 && d == 2 && s == 1) built = P == 4;
        if (!built || halo > P * s) continue;
        if (p.OW % P != 0) continue;
        const long long tp = (long long)p.OH * p.OW / P;
        if (tp > kMaxComputeThreads) continue;
        return P;
    }
    return 0;
}

static int run_stream(const StreamArgs& a, cudaStream_t st) {
    int rc;
    switch (a.p.dtype) {
        case DDF_B200_F32: rc = stream_dispatch<float>(a, st); break;
        case DDF_B200_F16: rc = stream_dispatch<__half>(a, st); break;
        case DDF_B200_BF16: rc = stream_dispatch<__nv_bfloat16>(a, st); break;
        default: rc = kNotHandled;
    }
    if (rc == 0) g_launches.fetch_add(1, std::memory_order_relaxed);
    return rc;
}

// Plane-ring kernels (2-byte element types).  Returns kNotHandled when no instantiation
// covers the problem.
static int run_ring(const RingArgs& a, cudaStream_t st) {
    int rc;
    switch (a.p.dtype) {
        case DDF_B200_F16: rc = ring_dispatch<__half>(a, st); break;
        case DDF_B200_BF16: rc = ring_dispatch<__nv_bfloat16>(a, st); break;
        default: rc = kNotHandled;
    }
    if (rc == 0) g_launches.fetch_add(1, std::memory_order_relaxed);
    return rc;
}

// Row kernel (7 x 7 outputs, 2-byte element types).
static int run_row(const RowArgs& a, cudaStream_t st) {
    int rc;
    switch (a.p.dtype) {
        case DDF_B200_F16: rc = row_dispatch<__half>(a, st); break;
        case DDF_B200_BF16: rc = row_dispatch<__nv_bfloat16>(a, st); break;
        case DDF_B200_F32: rc = row_dispatch<float>(a, st); break;
        default: rc = kNotHandled;
    }
    if (rc == 0) g_launches.fetch_add(1, std::memory_order_relaxed);
    return rc;
}

// AUTO prefers the streaming kernels once there is at least one plane group per SM
// and a quarter megabyte of input; below that the generic kernels launch faster.
static bool stream_worthwhile(const Problem& p, int sm_count) {
    const long long planes = (long long)p.B * p.C;
    const long long bytes = planes * p.H * p.W * elem_size(p.dtype);
    return planes >= sm_count && bytes >= (256ll << 10);
}

// Forward for a checked problem: the streaming kernel where it applies, else the generic one.
static int forward_impl(const Problem& p, const void* x, const void* cf, const void* sf, void* out,
                        int variant, void* stream) {
    DeviceInfo* di = nullptr;
    int rc = device_info(di);
    if (rc) return rc;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

    if (variant != DDF_B200_VARIANT_GENERIC) {
        const int P = stream_pixels(p, false);
        const bool want = variant == DDF_B200_VARIANT_STREAM || stream_worthwhile(p, di->sm_count);
        if (want) {
            RingArgs ra{x, cf, sf, out, p, false, di->sm_count, di->fault, di->index,
                        true, 0, 0u};
            RowArgs wa{x, cf, sf, out, p, false, di->sm_count, di->fault, di->index};
            rc = run_row(wa, st);
            if (rc != kNotHandled) return rc;
            rc = run_ring(ra, st);
            if (rc != kNotHandled) return rc;
        }
        if (P > 0 && want) {
            StreamArgs a{x, cf, sf, out, p, false, di->sm_count, di->fault, P, di->index, 2, 0, p.k == 3};
            rc = run_stream(a, st);
            if (rc != kNotHandled) return rc;
        }
        if (variant == DDF_B200_VARIANT_STREAM) return DDF_B200_E_UNSUPPORTED;
    }
    return run_generic_forward(p, x, cf, sf, out, di->sm_count, st);
}

}  // namespace ddf

using namespace ddf;

extern "C" {

int ddf_b200_version(void) { return 100; }

const char* ddf_b200_strerror(int status) {
    switch (status) {
        case 0: return "success";
        case DDF_B200_E_NULL: return "ddf_b200: a required pointer is NULL";
        case DDF_B200_E_SHAPE: return "ddf_b200: B, C, H, W, H/s and W/s must all be >= 1";
        case DDF_B200_E_KERNEL: return "ddf_b200: kernel_size must be odd and >= 1, dilation >= 1, stride >= 1";
        case DDF_B200_E_COMBINE: return "ddf_b200: combine must be mul (0) or add (1)";
        case DDF_B200_E_DTYPE: return "ddf_b200: unknown element type";
        case DDF_B200_E_VARIANT: return "ddf_b200: unknown kernel variant";
        case DDF_B200_E_UNSUPPORTED: return "ddf_b200: the streaming kernels do not cover this problem";
        case DDF_B200_E_WORKSPACE: return "ddf_b200: workspace is NULL or too small";
        case DDF_B200_E_TOO_LARGE: return "ddf_b200: problem exceeds the kernels' index ranges";
        case DDF_B200_E_DEVICE: return "ddf_b200: current device is not an sm_100 GPU";
        case DDF_B200_E_SCRATCH_LIMIT:
            return "ddf_b200: this problem needs more scratch than ddf_b200_backward_noalloc's "
                   "built-in 16 MiB array; use ddf_b200_backward with a caller-provided workspace";
        default: break;
    }
    if (status > 0) return cudaGetErrorString((cudaError_t)status);
    return "ddf_b200: unknown status";
}

unsigned long long ddf_b200_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int ddf_b200_take_fault(void) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return -(int)e - 1000;
    int v = 0;
    e = cudaMemcpyFromSymbol(&v, g_fault_word, sizeof(int));
    if (e != cudaSuccess) return -(int)e - 1000;
    if (v != 0) {
        int zero = 0;
        e = cudaMemcpyToSymbol(g_fault_word, &zero, sizeof(int));
        if (e != cudaSuccess) return -(int)e - 1000;
    }
    return v;
}

int ddf_b200_plan(int B, int C, int H, int W, int k, int d, int s, int combine, int dtype,
                  int backward) {
    Problem p;
    int rc = check_problem(B, C, H, W, k, d, s, combine, dtype, DDF_B200_VARIANT_AUTO, p);
    if (rc) return rc;
    DeviceInfo* di = nullptr;
    int sm = 148;
    if (device_info(di) == 0) sm = di->sm_count;
    if (backward) {
        return (bwd_stream_supported(p) && stream_worthwhile(p, sm)) ? DDF_B200_VARIANT_STREAM
                                                                     : DDF_B200_VARIANT_GENERIC;
    }
    return (stream_pixels(p, false) > 0 && stream_worthwhile(p, sm)) ? DDF_B200_VARIANT_STREAM
                                                                    : DDF_B200_VARIANT_GENERIC;
}

int ddf_b200_forward(const void* x, const void* cf, const void* sf, void* out, int B, int C, int H,
                     int W, int k, int d, int s, int combine, int dtype, int variant, void* stream) {
    Problem p;
    int rc = check_problem(B, C, H, W, k, d, s, combine, dtype, variant, p);
    if (rc) return rc;
    if (!x || !cf || !sf || !out) return DDF_B200_E_NULL;
    return forward_impl(p, x, cf, sf, out, variant, stream);
}

int ddf_b200_forward_waitlimit(const void* x, const void* cf, const void* sf, void* out, int B, int C,
                               int H, int W, int k, int d, int s, int combine, int dtype,
                               long long wait_cycles, int starve, void* stream) {
    Problem p;
    int rc = check_problem(B, C, H, W, k, d, s, combine, dtype, DDF_B200_VARIANT_STREAM, p);
    if (rc) return rc;
    if (!x || !cf || !sf || !out) return DDF_B200_E_NULL;
    if (wait_cycles < 1) return DDF_B200_E_SHAPE;
    DeviceInfo* di = nullptr;
    rc = device_info(di);
    if (rc) return rc;
    RingArgs ra{x, cf, sf, out, p, false, di->sm_count, di->fault, di->index, false, wait_cycles,
                starve ? 16u : 0u};
    rc = run_ring(ra, reinterpret_cast<cudaStream_t>(stream));
    return rc == kNotHandled ? DDF_B200_E_UNSUPPORTED : rc;
}

int ddf_b200_forward_sfnorm(const void* x, const void* cf, const void* sf_raw, void* out, int B,
                            int C, int H, int W, int k, int d, int s, int combine, int dtype,
                            int variant, double sf_scale, void* stream) {
    Problem p;
    int rc = check_problem(B, C, H, W, k, d, s, combine, dtype, variant, p);
    if (rc) return rc;
    if (k < 3) return DDF_B200_E_KERNEL;  // the unbiased std over k*k taps needs k*k > 1
    if (!x || !cf || !sf_raw || !out) return DDF_B200_E_NULL;
    p.sf_norm = 1;
    p.sf_scale = sf_scale;
    return forward_impl(p, x, cf, sf_raw, out, variant, stream);
}

size_t ddf_b200_backward_workspace(int B, int C, int H, int W, int k, int d, int s, int combine,
                                   int dtype, int variant) {
    Problem p;
    if (check_problem(B, C, H, W, k, d, s, combine, dtype, variant, p)) return 0;
    if (variant == DDF_B200_VARIANT_GENERIC) return 0;
    DeviceInfo* di = nullptr;
    int sm = 148;
    if (device_info(di) == 0) sm = di->sm_count;
    if (!bwd_stream_supported(p)) return 0;
    return bwd_stream_workspace(p, sm);
}

int ddf_b200_backward(const void* go, const void* x, const void* cf, const void* sf, void* gx,
                      void* gcf, void* gsf, void* workspace, size_t workspace_bytes, int B, int C,
                      int H, int W, int k, int d, int s, int combine, int dtype, int variant,
                      void* stream) {
    Problem p;
    int rc = check_problem(B, C, H, W, k, d, s, combine, dtype, variant, p);
    if (rc) return rc;
    if (!go || !x || !cf || !sf) return DDF_B200_E_NULL;
    DeviceInfo* di = nullptr;
    rc = device_info(di);
    if (rc) return rc;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const bool allow_stream = variant != DDF_B200_VARIANT_GENERIC;
    const bool want = variant == DDF_B200_VARIANT_STREAM || stream_worthwhile(p, di->sm_count);

    // Decide the filter-gradient path first, so that a missing workspace is reported before
    // anything has been launched.  Only the spatial-filter gradient uses the workspace.
    const bool filters_stream = (gcf || gsf) && allow_stream && want && bwd_stream_supported(p);
    if (filters_stream && gsf) {
        const size_t need = bwd_stream_workspace(p, di->sm_count);
        if (need > 0 && (!workspace || workspace_bytes < need)) return DDF_B200_E_WORKSPACE;
    }

    // grad wrt x: the streaming forward kernel run over go with mirrored taps.
    if (gx) {
        bool done = false;
        if (allow_stream && want) {
            RingArgs ra{go, cf, sf, gx, p, true, di->sm_count, di->fault, di->index,
                        true, 0, 0u};
            RowArgs wa{go, cf, sf, gx, p, true, di->sm_count, di->fault, di->index};
            rc = run_row(wa, st);
            if (rc == 0) done = true;
            else if (rc != kNotHandled) return rc;
            if (!done) {
                rc = run_ring(ra, st);
                if (rc == 0) done = true;
                else if (rc != kNotHandled) return rc;
            }
            const int P = done ? 0 : stream_pixels(p, true);
            if (P > 0) {
                StreamArgs a{go, cf, sf, gx, p, true, di->sm_count, di->fault, P, di->index, 2, 0, p.k == 3};
                rc = run_stream(a, st);
                if (rc == 0) done = true;
                else if (rc != kNotHandled) return rc;
            }
            if (!done && variant == DDF_B200_VARIANT_STREAM) return DDF_B200_E_UNSUPPORTED;
        }
        if (!done) {
            rc = run_generic_grad_x(p, go, cf, sf, gx, di->sm_count, st);
            if (rc) return rc;
        }
    }

    // grads wrt the two filters.
    if (gcf || gsf) {
        bool done = false;
        if (filters_stream) {
            int launches = 0;
            rc = bwd_stream_filters(p, go, x, cf, sf, gcf, gsf, gsf ? workspace : nullptr, di->sm_count, di->fault,
                                    di->index, st, &launches);
            if (rc == 0) {
                done = true;
                g_launches.fetch_add((unsigned long long)launches, std::memory_order_relaxed);
            } else if (rc != kNotHandled) {
                return rc;
            }
        }
        if (!done && variant == DDF_B200_VARIANT_STREAM) return DDF_B200_E_UNSUPPORTED;
        if (!done) {
            rc = run_generic_grad_filters(p, go, x, cf, sf, gcf, gsf, di->sm_count, st);
            if (rc) return rc;
        }
    }
    return 0;
}

}  // extern "C"
