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

// grad-x for k = 3, dilation 1, stride 2, even H and W (H = 2*OH, W = 2*OW): the case of the
// down-sampling layers.  A thread owns one OUTPUT pixel q = (qy, qx) of a sample and walks a
// chunk of channels; per channel it writes the 2 x 2 input pixels (2qy.., 2qx..).  With stride
// 2 each input pixel receives only the taps whose offset has its parity -- 1, 2, 2 and 4 of
// the nine -- so the four results need exactly nine products, and the nine spatial-filter
// values they use (at q and its right / lower / lower-right neighbours) stay in registers for
// all channels:
//   gx[2qy  ][2qx  ] = go[q]*w4[q]
//   gx[2qy  ][2qx+1] = go[q]*w5[q]  + go[q+x]*w3[q+x]
//   gx[2qy+1][2qx  ] = go[q]*w7[q]  + go[q+y]*w1[q+y]
//   gx[2qy+1][2qx+1] = go[q]*w8[q]  + go[q+x]*w6[q+x] + go[q+y]*w2[q+y] + go[q+x+y]*w0[q+x+y]
// (w_t[q] = cf[c,t] (.) sf[t,q]; neighbours outside the plane contribute nothing).
// Same arithmetic as generic_grad_x, without its per-tap divisions and parity tests.
template <typename T, int MODE, int CH>
__global__ void __launch_bounds__(256)
grad_x_k3s2(const T* __restrict__ go, const T* __restrict__ cf, const T* __restrict__ sf,
            T* __restrict__ gx, Problem p) {
    using A = typename Elem<T>::acc_t;
    const int q = blockIdx.x * blockDim.x + threadIdx.x;
    const int opl = p.OH * p.OW;
    if (q >= opl) return;
    const int qy = q / p.OW, qx = q - qy * p.OW;
    const long long b = blockIdx.z;
    const bool has_x = qx + 1 < p.OW, has_y = qy + 1 < p.OH;
    const T* sfb = sf + b * 9 * (long long)opl + q;
    auto sfv = [&](int t, int off, bool ok) -> A { return ok ? (A)Elem<T>::load(sfb + (long long)t * opl + off) : (A)0; };
    const A s4 = sfv(4, 0, true), s5 = sfv(5, 0, true), s7 = sfv(7, 0, true), s8 = sfv(8, 0, true);
    const A s3 = sfv(3, 1, has_x), s6 = sfv(6, 1, has_x);
    const A s1 = sfv(1, p.OW, has_y), s2 = sfv(2, p.OW, has_y);
    const A s0 = sfv(0, p.OW + 1, has_x && has_y);
    const int c_lo = blockIdx.y * CH;
    const int c_hi = c_lo + CH < p.C ? c_lo + CH : p.C;
    const long long ipl = (long long)p.H * p.W;
    for (int c = c_lo; c < c_hi; ++c) {
        const long long plane = b * p.C + c;
        const T* gop = go + plane * opl + q;
        const T* cfp = cf + plane * 9;
        A w[9];
#pragma unroll
        for (int t = 0; t < 9; ++t) w[t] = Elem<T>::load(cfp + t);
        const A g00 = Elem<T>::load(gop);
        const A g01 = has_x ? (A)Elem<T>::load(gop + 1) : (A)0;
        const A g10 = has_y ? (A)Elem<T>::load(gop + p.OW) : (A)0;
        const A g11 = (has_x && has_y) ? (A)Elem<T>::load(gop + p.OW + 1) : (A)0;
        const A r00 = g00 * combine_w<MODE, A>(w[4], s4);
        const A r01 = g00 * combine_w<MODE, A>(w[5], s5) + g01 * combine_w<MODE, A>(w[3], s3);
        const A r10 = g00 * combine_w<MODE, A>(w[7], s7) + g10 * combine_w<MODE, A>(w[1], s1);
        const A r11 = g00 * combine_w<MODE, A>(w[8], s8) + g01 * combine_w<MODE, A>(w[6], s6) +
                      g10 * combine_w<MODE, A>(w[2], s2) + g11 * combine_w<MODE, A>(w[0], s0);
        T* o = gx + plane * ipl + (long long)(2 * qy) * p.W + 2 * qx;
        Elem<T>::store(o, r00);
        Elem<T>::store(o + 1, r01);
        Elem<T>::store(o + p.W, r10);
        Elem<T>::store(o + p.W + 1, r11);
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
