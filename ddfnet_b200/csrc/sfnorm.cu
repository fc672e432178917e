// The spatial FilterNorm (ddf/ddf.py:146-157, built by build_spatial_branch with neither a
// running std nor a running mean) as two small kernels, for the backward of the op with the
// fused norm: the forward kernel keeps the normalised filter in registers, so the backward
// (a) recomputes it from the raw filter, once, for the gradient kernels that consume it and
// (b) carries the gradient with respect to the normalised filter back through the
// normalisation.  One thread per (sample, pixel): its k*k values lie OH*OW elements apart,
// so neighbouring threads read neighbouring addresses.
//
//   c_t = v_t - mean(v),  s = sqrt(sum c_t^2 / (n-1)),  a = 1 / (s + 1e-10),  y_t = scale * a * c_t
//   dL/dc_t = scale * (a * g_t - a^2 * c_t * G / ((n-1) s)),  G = sum_u g_u c_u   (second term 0 when s = 0)
//   dL/dv_t = dL/dc_t - mean_u(dL/dc_u)
#include <atomic>

#include "common.cuh"

namespace ddf {

extern std::atomic<unsigned long long> g_launches;

template <typename T, typename A, int KK, bool BWD>
__global__ void __launch_bounds__(256) sfnorm_kernel(const T* __restrict__ raw, const T* __restrict__ gy,
                                                     T* __restrict__ out, long long pixels, long long ohw,
                                                     A scale) {
    const long long p = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= pixels) return;
    const long long b = p / ohw, q = p - b * ohw;
    const long long base = b * KK * ohw + q;
    A c[KK];
    A sum = 0;
#pragma unroll
    for (int t = 0; t < KK; ++t) {
        c[t] = (A)Elem<T>::load(raw + base + t * ohw);
        sum += c[t];
    }
    const A mean = sum / (A)KK;
    A var = 0;
#pragma unroll
    for (int t = 0; t < KK; ++t) {
        c[t] -= mean;
        var += c[t] * c[t];
    }
    const A s = sqrt(var / (A)(KK - 1));
    const A a = (A)1 / (s + (A)1e-10);
    if constexpr (!BWD) {
#pragma unroll
        for (int t = 0; t < KK; ++t) Elem<T>::store(out + base + t * ohw, (typename Elem<T>::acc_t)(scale * a * c[t]));
    } else {
        A g[KK];
        A G = 0;
#pragma unroll
        for (int t = 0; t < KK; ++t) {
            g[t] = (A)Elem<T>::load(gy + base + t * ohw);
            G += g[t] * c[t];
        }
        const A k2 = s > (A)0 ? a * a * G / ((A)(KK - 1) * s) : (A)0;
        A dsum = 0;
#pragma unroll
        for (int t = 0; t < KK; ++t) {
            g[t] = scale * (a * g[t] - k2 * c[t]);
            dsum += g[t];
        }
        const A dmean = dsum / (A)KK;
#pragma unroll
        for (int t = 0; t < KK; ++t) Elem<T>::store(out + base + t * ohw, (typename Elem<T>::acc_t)(g[t] - dmean));
    }
}

template <typename T, typename A, bool BWD>
static int sfnorm_launch(const void* raw, const void* gy, void* out, long long pixels, long long ohw, int k,
                         double scale, cudaStream_t st) {
    const unsigned grid = (unsigned)((pixels + 255) / 256);
    if (k == 3) sfnorm_kernel<T, A, 9, BWD><<<grid, 256, 0, st>>>((const T*)raw, (const T*)gy, (T*)out, pixels, ohw, (A)scale);
    else if (k == 5) sfnorm_kernel<T, A, 25, BWD><<<grid, 256, 0, st>>>((const T*)raw, (const T*)gy, (T*)out, pixels, ohw, (A)scale);
    else if (k == 7) sfnorm_kernel<T, A, 49, BWD><<<grid, 256, 0, st>>>((const T*)raw, (const T*)gy, (T*)out, pixels, ohw, (A)scale);
    else return DDF_B200_E_UNSUPPORTED;
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}

template <bool BWD>
static int sfnorm_entry(const void* raw, const void* gy, void* out, int B, int k, int OH, int OW, int dtype,
                        double scale, void* stream) {
    if (!raw || !out || (BWD && !gy)) return DDF_B200_E_NULL;
    if (B < 1 || OH < 1 || OW < 1) return DDF_B200_E_SHAPE;
    if (k < 3 || (k - 1) % 2 != 0) return DDF_B200_E_KERNEL;
    const long long ohw = (long long)OH * OW, pixels = (long long)B * ohw;
    if (pixels > (1ll << 31) * 255) return DDF_B200_E_TOO_LARGE;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    switch (dtype) {
        case DDF_B200_F32: return sfnorm_launch<float, float, BWD>(raw, gy, out, pixels, ohw, k, scale, st);
        case DDF_B200_F16: return sfnorm_launch<__half, float, BWD>(raw, gy, out, pixels, ohw, k, scale, st);
        case DDF_B200_BF16: return sfnorm_launch<__nv_bfloat16, float, BWD>(raw, gy, out, pixels, ohw, k, scale, st);
        case DDF_B200_F64: return sfnorm_launch<double, double, BWD>(raw, gy, out, pixels, ohw, k, scale, st);
        default: return DDF_B200_E_DTYPE;
    }
}

}  // namespace ddf

extern "C" {

int ddf_b200_sfnorm(const void* raw, void* normed, int B, int k, int OH, int OW, int dtype, double sf_scale,
                    void* stream) {
    return ddf::sfnorm_entry<false>(raw, nullptr, normed, B, k, OH, OW, dtype, sf_scale, stream);
}

int ddf_b200_sfnorm_backward(const void* raw, const void* grad_normed, void* grad_raw, int B, int k, int OH,
                             int OW, int dtype, double sf_scale, void* stream) {
    return ddf::sfnorm_entry<true>(raw, grad_normed, grad_raw, B, k, OH, OW, dtype, sf_scale, stream);
}

}  // extern "C"
