// Generic DDF kernels: any odd k, any dilation and stride, any element type
// (float, double, half, bfloat16), any plane size.  One thread per element (or a
// block per reduction); no shared-memory staging.  These are the reference
// point for the streaming kernels and the path AUTO falls back to.
//
// Arithmetic: products and sums in float (double for double tensors); the
// result is rounded once to the element type.
#pragma once

#include "common.cuh"

namespace ddf {

// Compensated (Neumaier) running sum, as the reference's kernels use for their
// long sums (ddf/src/cuda/ddf_mul_cuda_kernel.cu:340-349, 406-414): the channel
// sum of grad-sf and the pixel sum of grad-cf reach thousands of terms.
template <typename A>
struct CompSum {
    A sum = 0, lost = 0;
    __device__ __forceinline__ void add(A v) {
        const A t = sum + v;
        lost += (fabs(sum) >= fabs(v)) ? (sum - t) + v : (v - t) + sum;
        sum = t;
    }
    __device__ __forceinline__ A value() const { return sum + lost; }
};

// out[b,c,y,x] = sum_t x[b,c,y*s+oi,x*s+oj] * w(cf[b,c,t], sf[b,t,y,x])
// Replaces DDFForward (ddf/src/cuda/ddf_mul_cuda_kernel.cu:85-165).
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
generic_forward(const T* __restrict__ x, const T* __restrict__ cf, const T* __restrict__ sf,
                T* __restrict__ out, Problem p, long long total) {
    using A = typename Elem<T>::acc_t;
    const int r = (p.k - 1) / 2;
    const int kk = p.k * p.k;
    const long long opl = (long long)p.OH * p.OW;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const int xo = (int)(idx % p.OW);
        const int y = (int)((idx / p.OW) % p.OH);
        const long long plane = idx / opl;  // b*C + c
        const long long b = plane / p.C;
        const T* xp = x + plane * p.H * p.W;
        const T* cfp = cf + plane * kk;
        const T* sfp = sf + b * kk * opl + (long long)y * p.OW + xo;
        // Fused spatial FilterNorm: statistics of this pixel's k*k raw filter values.
        A sf_mean = 0, sf_inv = 1;
        if (p.sf_norm) {
            A sum = 0;
            for (int t = 0; t < kk; ++t) sum += Elem<T>::load(sfp + t * opl);
            sf_mean = sum / kk;
            A var = 0;
            for (int t = 0; t < kk; ++t) {
                const A dv = Elem<T>::load(sfp + t * opl) - sf_mean;
                var += dv * dv;
            }
            sf_inv = (A)p.sf_scale / (sqrt(var / (kk - 1)) + (A)1e-10);
        }
        A acc = 0;
        for (int i = 0; i < p.k; ++i) {
            const int iy = y * p.s + (i - r) * p.d;
            if (iy < 0 || iy >= p.H) continue;
            for (int j = 0; j < p.k; ++j) {
                const int ix = xo * p.s + (j - r) * p.d;
                if (ix < 0 || ix >= p.W) continue;
                const int t = i * p.k + j;
                const A sfv = ((A)Elem<T>::load(sfp + t * opl) - sf_mean) * sf_inv;
                const A w = combine_w<MODE, A>(Elem<T>::load(cfp + t), sfv);
                acc += Elem<T>::load(xp + (long long)iy * p.W + ix) * w;
            }
        }
        Elem<T>::store(out + idx, acc);
    }
}

// gx[b,c,py,px] = sum_t go[b,c,q] * w(cf[b,c,t], sf[b,t,q]),  q*s + off_t = p.
// Replaces DDFBackward_Feature (ddf/src/cuda/ddf_mul_cuda_kernel.cu:198-290)
// and the two transposes around it (:433-443, :463-473).
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
generic_grad_x(const T* __restrict__ go, const T* __restrict__ cf, const T* __restrict__ sf,
               T* __restrict__ gx, Problem p, long long total) {
    using A = typename Elem<T>::acc_t;
    const int r = (p.k - 1) / 2;
    const int kk = p.k * p.k;
    const long long ipl = (long long)p.H * p.W;
    const long long opl = (long long)p.OH * p.OW;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const int px = (int)(idx % p.W);
        const int py = (int)((idx / p.W) % p.H);
        const long long plane = idx / ipl;
        const long long b = plane / p.C;
        const T* gop = go + plane * opl;
        const T* cfp = cf + plane * kk;
        const T* sfb = sf + b * kk * opl;
        A acc = 0;
        for (int i = 0; i < p.k; ++i) {
            const int ny = py - (i - r) * p.d;
            if (ny < 0 || ny % p.s != 0) continue;
            const int qy = ny / p.s;
            if (qy >= p.OH) continue;
            for (int j = 0; j < p.k; ++j) {
                const int nx = px - (j - r) * p.d;
                if (nx < 0 || nx % p.s != 0) continue;
                const int qx = nx / p.s;
                if (qx >= p.OW) continue;
                const int t = i * p.k + j;
                const long long q = (long long)qy * p.OW + qx;
                const A w = combine_w<MODE, A>(Elem<T>::load(cfp + t), Elem<T>::load(sfb + t * opl + q));
                acc += Elem<T>::load(gop + q) * w;
            }
        }
        Elem<T>::store(gx + idx, acc);
    }
}

// gsf[b,t,y,x] = sum_c go[b,c,y,x] * x[b,c,y*s+oi,x*s+oj] * (cf[b,c,t] | 1)
// Replaces DDFBackward_Spatial_Filter (ddf/src/cuda/ddf_mul_cuda_kernel.cu:293-355)
// and the transpose after it (:492-502).
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
generic_grad_sf(const T* __restrict__ go, const T* __restrict__ x, const T* __restrict__ cf,
                T* __restrict__ gsf, Problem p, long long total) {
    using A = typename Elem<T>::acc_t;
    const int r = (p.k - 1) / 2;
    const int kk = p.k * p.k;
    const long long ipl = (long long)p.H * p.W;
    const long long opl = (long long)p.OH * p.OW;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const int xo = (int)(idx % p.OW);
        const int y = (int)((idx / p.OW) % p.OH);
        const int t = (int)((idx / opl) % kk);
        const long long b = idx / (opl * kk);
        const int iy = y * p.s + (t / p.k - r) * p.d;
        const int ix = xo * p.s + (t % p.k - r) * p.d;
        CompSum<A> acc;
        if (iy >= 0 && iy < p.H && ix >= 0 && ix < p.W) {
            const T* gop = go + b * p.C * opl + (long long)y * p.OW + xo;
            const T* xp = x + b * p.C * ipl + (long long)iy * p.W + ix;
            const T* cfp = cf + b * p.C * kk + t;
            for (int c = 0; c < p.C; ++c) {
                const A cfv = MODE == DDF_B200_MUL ? (A)Elem<T>::load(cfp + (long long)c * kk) : (A)1;
                acc.add(Elem<T>::load(gop + c * opl) * Elem<T>::load(xp + c * ipl) * cfv);
            }
        }
        Elem<T>::store(gsf + idx, acc.value());
    }
}

// gcf[b,c,t] = sum_{y,x} go[b,c,y,x] * x[b,c,y*s+oi,x*s+oj] * (sf[b,t,y,x] | 1)
// One block per (b,c) plane; every thread keeps a partial per tap in turn and the
// block reduces it.  Replaces DDFBackward_Channel_Filter
// (ddf/src/cuda/ddf_mul_cuda_kernel.cu:358-420).
template <typename T, int MODE>
__global__ void __launch_bounds__(128)
generic_grad_cf(const T* __restrict__ go, const T* __restrict__ x, const T* __restrict__ sf,
                T* __restrict__ gcf, Problem p, long long planes) {
    using A = typename Elem<T>::acc_t;
    __shared__ A warp_part[4];
    const int r = (p.k - 1) / 2;
    const int kk = p.k * p.k;
    const long long ipl = (long long)p.H * p.W;
    const int opl = p.OH * p.OW;
    for (long long plane = blockIdx.x; plane < planes; plane += gridDim.x) {
        const long long b = plane / p.C;
        const T* gop = go + plane * opl;
        const T* xp = x + plane * ipl;
        const T* sfb = sf + b * kk * (long long)opl;
        for (int t = 0; t < kk; ++t) {
            const int oi = (t / p.k - r) * p.d, oj = (t % p.k - r) * p.d;
            CompSum<A> part;
            for (int q = threadIdx.x; q < opl; q += blockDim.x) {
                const int y = q / p.OW, xo = q - y * p.OW;
                const int iy = y * p.s + oi, ix = xo * p.s + oj;
                if (iy < 0 || iy >= p.H || ix < 0 || ix >= p.W) continue;
                const A sfv = MODE == DDF_B200_MUL ? (A)Elem<T>::load(sfb + (long long)t * opl + q) : (A)1;
                part.add(Elem<T>::load(gop + q) * Elem<T>::load(xp + (long long)iy * p.W + ix) * sfv);
            }
            A acc = part.value();
            for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = acc;
            __syncthreads();
            if (threadIdx.x == 0) {
                A tot = 0;
                for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += warp_part[w];
                Elem<T>::store(gcf + plane * kk + t, tot);
            }
            __syncthreads();
        }
    }
}

}  // namespace ddf
