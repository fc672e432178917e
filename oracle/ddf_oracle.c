/*
 * CPU oracle for the Decoupled Dynamic Filter (DDF) operator.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the CUDA path is
 * compared against; nothing in the shipped package may call it.
 *
 * It restates, as plain loops, the arithmetic of the reference project
 * (theFoxofSky/ddfnet).  The reference has no CPU implementation of the op
 * (ddf/src/ddf_mul_ext.cpp:33 raises "not implemented on CPU"), so this is a
 * restatement and not a build of reference sources:
 *
 *   forward   tap order t = i*k + j, centre k/2, dilation, zero padding and the
 *             mul / add combination follow grad_check.py:11-30 (py_forward);
 *             the stride (window start = p*s - ((k-1)/2)*d) and the floor
 *             output size H/s x W/s follow
 *             ddf/src/cuda/ddf_mul_cuda_kernel.cu:102-113,135-147 and
 *             ddf/ddf.py:56,74.  The 'add' expression follows
 *             ddf/src/cuda/ddf_add_cuda_kernel.cu:150-152.
 *   grad_x    ddf/src/cuda/ddf_mul_cuda_kernel.cu:255-289 (written here in the
 *             scatter form: every output pixel adds into the input pixels it
 *             read, which is the same sum the reference gathers with flipped
 *             tap indices);  add: ddf_add_cuda_kernel.cu:278-279.
 *   grad_sf   ddf/src/cuda/ddf_mul_cuda_kernel.cu:317-345; add variant drops
 *             the channel-filter factor (ddf_add_cuda_kernel.cu:338).
 *   grad_cf   ddf/src/cuda/ddf_mul_cuda_kernel.cu:379-411; add variant drops
 *             the spatial-filter factor (ddf_add_cuda_kernel.cu:403).
 *
 * Parity status: the reference ships no stored vectors.  The oracle is pinned
 * (tests/test_oracle.py) against a restatement of the reference's own
 * py_forward test oracle, against an independent unfold+autograd derivation in
 * float64, and against fixtures under tests/golden/ .
 *
 * Layout: contiguous NCHW everywhere.
 *   x  (B,C,H,W)   cf (B,C,k,k)   sf (B,k*k,OH,OW)   out/go (B,C,OH,OW)
 *   OH = H / s, OW = W / s (floor).
 * combine: 0 = mul, 1 = add.
 *
 * Two instances are generated from one body: *_f64 (golden, accumulates in
 * double) and *_f32 (the timed CPU baseline, accumulates in float).  Both are
 * parallelised with OpenMP over (b, c) planes or (b, pixel) as the reduction
 * allows.
 */
#include <stddef.h>
#include <stdint.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

int ddf_oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void ddf_oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

#define DDF_COMBINE(cfv, sfv, combine) ((combine) == 0 ? (cfv) * (sfv) : (cfv) + (sfv))

#define DDF_DEFINE(T, SUFFIX)                                                              \
                                                                                           \
void ddf_oracle_forward_##SUFFIX(const T* x, const T* cf, const T* sf, T* out,             \
                                 int B, int C, int H, int W, int k, int d, int s,          \
                                 int combine) {                                            \
    const int OH = H / s, OW = W / s, r = (k - 1) / 2, kk = k * k;                         \
    const long planes = (long)B * C;                                                       \
    _Pragma("omp parallel for schedule(static)")                                           \
    for (long pl = 0; pl < planes; ++pl) {                                                 \
        const int b = (int)(pl / C);                                                       \
        const T* xp = x + (size_t)pl * H * W;                                              \
        const T* cfp = cf + (size_t)pl * kk;                                               \
        const T* sfb = sf + (size_t)b * kk * OH * OW;                                      \
        T* op = out + (size_t)pl * OH * OW;                                                \
        for (int q = 0; q < OH * OW; ++q) op[q] = 0;                                       \
        /* tap-outer order: per pixel the taps are still added in ascending t */           \
        for (int i = 0; i < k; ++i) {                                                      \
            for (int j = 0; j < k; ++j) {                                                  \
                const int t = i * k + j;                                                   \
                const int oi = (i - r) * d, oj = (j - r) * d;                              \
                const T cfv = cfp[t];                                                      \
                for (int y = 0; y < OH; ++y) {                                             \
                    const int iy = y * s + oi;                                             \
                    if (iy < 0 || iy >= H) continue;                                       \
                    /* valid xo: 0 <= xo*s + oj < W */                                     \
                    int lo = oj < 0 ? (-oj + s - 1) / s : 0;                               \
                    int hi = (W - 1 - oj) >= 0 ? (W - 1 - oj) / s + 1 : 0;                 \
                    if (hi > OW) hi = OW;                                                  \
                    const T* xrow = xp + (size_t)iy * W + oj;                              \
                    const T* sfrow = sfb + ((size_t)t * OH + y) * OW;                      \
                    T* orow = op + (size_t)y * OW;                                         \
                    if (combine == 0) {                                                    \
                        for (int xo = lo; xo < hi; ++xo)                                   \
                            orow[xo] += xrow[(size_t)xo * s] * (cfv * sfrow[xo]);          \
                    } else {                                                               \
                        for (int xo = lo; xo < hi; ++xo)                                   \
                            orow[xo] += xrow[(size_t)xo * s] * (cfv + sfrow[xo]);          \
                    }                                                                      \
                }                                                                          \
            }                                                                              \
        }                                                                                  \
    }                                                                                      \
}                                                                                          \
                                                                                           \
/* grad wrt x and wrt cf: independent per (b,c) plane. Either output may be NULL. */       \
static void ddf_oracle_bwd_planes_##SUFFIX(const T* go, const T* x, const T* cf,           \
                                           const T* sf, T* gx, T* gcf,                     \
                                           int B, int C, int H, int W, int k, int d,       \
                                           int s, int combine) {                           \
    const int OH = H / s, OW = W / s, r = (k - 1) / 2, kk = k * k;                         \
    const long planes = (long)B * C;                                                       \
    _Pragma("omp parallel for schedule(static)")                                           \
    for (long pl = 0; pl < planes; ++pl) {                                                 \
        const int b = (int)(pl / C);                                                       \
        const T* xp = x + (size_t)pl * H * W;                                              \
        const T* cfp = cf + (size_t)pl * kk;                                               \
        const T* sfb = sf + (size_t)b * kk * OH * OW;                                      \
        const T* gop = go + (size_t)pl * OH * OW;                                          \
        T* gxp = gx ? gx + (size_t)pl * H * W : NULL;                                      \
        if (gxp) memset(gxp, 0, sizeof(T) * (size_t)H * W);                                \
        for (int i = 0; i < k; ++i) {                                                      \
            for (int j = 0; j < k; ++j) {                                                  \
                const int t = i * k + j;                                                   \
                T tap_sum = 0;                                                             \
                for (int y = 0; y < OH; ++y) {                                             \
                    const int iy = y * s + (i - r) * d;                                    \
                    if (iy < 0 || iy >= H) continue;                                       \
                    for (int xo = 0; xo < OW; ++xo) {                                      \
                        const int ix = xo * s + (j - r) * d;                               \
                        if (ix < 0 || ix >= W) continue;                                   \
                        const T g = gop[(size_t)y * OW + xo];                              \
                        const T sfv = sfb[((size_t)t * OH + y) * OW + xo];                 \
                        if (gxp)                                                           \
                            gxp[(size_t)iy * W + ix] += g * DDF_COMBINE(cfp[t], sfv, combine); \
                        tap_sum += g * xp[(size_t)iy * W + ix] * (combine == 0 ? sfv : (T)1); \
                    }                                                                      \
                }                                                                          \
                if (gcf) gcf[(size_t)pl * kk + t] = tap_sum;                               \
            }                                                                              \
        }                                                                                  \
    }                                                                                      \
}                                                                                          \
                                                                                           \
/* grad wrt sf: a sum over channels, independent per (b, tap, pixel). */                   \
static void ddf_oracle_bwd_spatial_##SUFFIX(const T* go, const T* x, const T* cf,          \
                                            T* gsf, int B, int C, int H, int W, int k,     \
                                            int d, int s, int combine) {                   \
    const int OH = H / s, OW = W / s, r = (k - 1) / 2, kk = k * k;                         \
    const long rows = (long)B * kk * OH;                                                   \
    _Pragma("omp parallel for schedule(static)")                                           \
    for (long row = 0; row < rows; ++row) {                                                \
        const int y = (int)(row % OH);                                                     \
        const int t = (int)((row / OH) % kk);                                              \
        const int b = (int)(row / ((long)OH * kk));                                        \
        const int i = t / k, j = t % k;                                                    \
        const int iy = y * s + (i - r) * d;                                                \
        T* dst = gsf + (size_t)row * OW;                                                   \
        for (int xo = 0; xo < OW; ++xo) dst[xo] = 0;                                       \
        if (iy < 0 || iy >= H) continue;                                                   \
        for (int c = 0; c < C; ++c) {                                                      \
            const size_t pl = (size_t)b * C + c;                                           \
            const T* xrow = x + (pl * H + iy) * W;                                         \
            const T* gorow = go + (pl * OH + y) * OW;                                      \
            const T cfv = combine == 0 ? cf[pl * kk + t] : (T)1;                           \
            for (int xo = 0; xo < OW; ++xo) {                                              \
                const int ix = xo * s + (j - r) * d;                                       \
                if (ix < 0 || ix >= W) continue;                                           \
                dst[xo] += gorow[xo] * xrow[ix] * cfv;                                     \
            }                                                                              \
        }                                                                                  \
    }                                                                                      \
}                                                                                          \
                                                                                           \
void ddf_oracle_backward_##SUFFIX(const T* go, const T* x, const T* cf, const T* sf,       \
                                  T* gx, T* gcf, T* gsf,                                   \
                                  int B, int C, int H, int W, int k, int d, int s,         \
                                  int combine) {                                           \
    if (gx || gcf)                                                                         \
        ddf_oracle_bwd_planes_##SUFFIX(go, x, cf, sf, gx, gcf, B, C, H, W, k, d, s, combine); \
    if (gsf)                                                                               \
        ddf_oracle_bwd_spatial_##SUFFIX(go, x, cf, gsf, B, C, H, W, k, d, s, combine);     \
}

DDF_DEFINE(double, f64)
DDF_DEFINE(float, f32)
