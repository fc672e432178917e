// Layout adapters between a channels-last (NHWC) network and the NCHW tensors the DDF
// kernels work on: tiled transposes through shared memory, optionally with a per-channel
// affine map and ReLU applied on the way out (an eval-mode BatchNorm + ReLU after the op).
//
// The reference has no counterpart: its op rejects non-contiguous input
// (ddf/src/cuda/ddf_mul_cuda.cpp:28-32), so a channels_last model copies with generic
// strided-copy kernels around every DDF layer.
//
// One CTA moves a 64-channel x 64-pixel tile of one sample: 256 threads read four
// consecutive elements each along the source's contiguous dimension (one 8- or 16-byte
// load where the row pitch allows), park the tile in shared memory with a padded pitch,
// and write four consecutive elements each along the destination's contiguous dimension.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>

#include "../../include/ddf_b200.h"
#include "common.cuh"

namespace ddf {

extern std::atomic<unsigned long long> g_launches;

constexpr int kTile = 64;

template <typename T>
struct Vec4 {  // four consecutive elements
    T v[4];
};

template <typename T>
__device__ __forceinline__ void load4(const T* p, bool vec, int n_valid, T (&out)[4]) {
    if (vec && n_valid == 4) {
        *reinterpret_cast<Vec4<T>*>(out) = *reinterpret_cast<const Vec4<T>*>(p);
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) out[i] = i < n_valid ? p[i] : T(0.f);
    }
}

template <typename T>
__device__ __forceinline__ void store4(T* p, bool vec, int n_valid, const T (&in)[4]) {
    if (vec && n_valid == 4) {
        *reinterpret_cast<Vec4<T>*>(p) = *reinterpret_cast<const Vec4<T>*>(in);
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (i < n_valid) p[i] = in[i];
    }
}

// TO_NHWC = true : src (B,C,HW) -> dst (B,HW,C), optional dst = relu(src * scale[c] + shift[c])
// TO_NHWC = false: src (B,HW,C) -> dst (B,C,HW)
// SC: channels per pixel in the NHWC SOURCE of the TO_NHWC = false direction (>= C; only the
// first C are taken, e.g. a convolution padded to a friendlier channel count); = C otherwise.
template <typename T, bool TO_NHWC>
__global__ void __launch_bounds__(256)
layout_kernel(const T* __restrict__ src, T* __restrict__ dst, int C, int HW, int SC,
              const float* __restrict__ scale, const float* __restrict__ shift, int relu) {
    constexpr int PITCH = kTile + (sizeof(T) == 2 ? 2 : 1);
    __shared__ T tile[kTile][PITCH];  // [channel][pixel]
    const int t = threadIdx.x;
    const int p0 = blockIdx.x * kTile, c0 = blockIdx.y * kTile;
    const long long b = blockIdx.z;
    const T* s = src + b * (long long)(TO_NHWC ? C : SC) * HW;
    T* d = dst + b * (long long)C * HW;
    const int sub = t >> 4;        // 0..15: row within a pass
    const int q = (t & 15) * 4;    // first of the thread's four elements along the row
    // 8-byte (2-byte types) or 16-byte (float) accesses need rows that keep that alignment.
    const bool vec_hw = (HW % 4) == 0, vec_c = (C % 4) == 0, vec_sc = (SC % 4) == 0;

    if (TO_NHWC) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int c = c0 + r * 16 + sub, p = p0 + q;
            if (c < C && p < HW) {
                T v[4];
                load4(s + (long long)c * HW + p, vec_hw, HW - p < 4 ? HW - p : 4, v);
                if (scale != nullptr) {
                    const float a = scale[c], sh = shift[c];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float f = fmaf((float)v[i], a, sh);
                        if (relu) f = fmaxf(f, 0.f);
                        v[i] = (T)f;
                    }
                } else if (relu) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) v[i] = (T)fmaxf((float)v[i], 0.f);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) tile[r * 16 + sub][q + i] = v[i];
            }
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int p = p0 + r * 16 + sub, c = c0 + q;
            if (p < HW && c < C) {
                T v[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) v[i] = tile[q + i][r * 16 + sub];
                store4(d + (long long)p * C + c, vec_c, C - c < 4 ? C - c : 4, v);
            }
        }
    } else {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int p = p0 + r * 16 + sub, c = c0 + q;
            if (p < HW && c < C) {
                T v[4];
                load4(s + (long long)p * SC + c, vec_sc, C - c < 4 ? C - c : 4, v);
                if (scale != nullptr) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (c + i < C) {
                            float f = fmaf((float)v[i], scale[c + i], shift[c + i]);
                            if (relu) f = fmaxf(f, 0.f);
                            v[i] = (T)f;
                        }
                    }
                } else if (relu) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) v[i] = (T)fmaxf((float)v[i], 0.f);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) tile[q + i][r * 16 + sub] = v[i];
            }
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int c = c0 + r * 16 + sub, p = p0 + q;
            if (c < C && p < HW) {
                T v[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) v[i] = tile[r * 16 + sub][q + i];
                store4(d + (long long)c * HW + p, vec_hw, HW - p < 4 ? HW - p : 4, v);
            }
        }
    }
}

template <typename T, bool TO_NHWC>
static int layout_launch(const void* src, void* dst, int B, int C, int HW, int SC, const float* scale,
                         const float* shift, int relu, cudaStream_t st) {
    // The vector accesses also need 8- / 16-byte aligned bases.
    const uintptr_t mask = sizeof(T) * 4 - 1;
    if ((reinterpret_cast<uintptr_t>(src) & mask) || (reinterpret_cast<uintptr_t>(dst) & mask))
        return DDF_B200_E_UNSUPPORTED;
    dim3 grid((unsigned)((HW + kTile - 1) / kTile), (unsigned)((C + kTile - 1) / kTile), (unsigned)B);
    if (grid.y > 65535u || grid.z > 65535u) return DDF_B200_E_TOO_LARGE;
    layout_kernel<T, TO_NHWC><<<grid, 256, 0, st>>>((const T*)src, (T*)dst, C, HW, SC, scale, shift, relu);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}

template <bool TO_NHWC>
static int layout_any(const void* src, void* dst, int B, int C, int H, int W, int SC, int dtype,
                      const float* scale, const float* shift, int relu, void* stream) {
    if (!src || !dst) return DDF_B200_E_NULL;
    if (B < 1 || C < 1 || H < 1 || W < 1 || SC < C) return DDF_B200_E_SHAPE;
    if ((long long)H * W > (1ll << 30)) return DDF_B200_E_TOO_LARGE;
    if ((scale == nullptr) != (shift == nullptr)) return DDF_B200_E_NULL;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int HW = H * W;
    switch (dtype) {
        case DDF_B200_F32: return layout_launch<float, TO_NHWC>(src, dst, B, C, HW, SC, scale, shift, relu, st);
        case DDF_B200_F16: return layout_launch<__half, TO_NHWC>(src, dst, B, C, HW, SC, scale, shift, relu, st);
        case DDF_B200_BF16:
            return layout_launch<__nv_bfloat16, TO_NHWC>(src, dst, B, C, HW, SC, scale, shift, relu, st);
        default: return DDF_B200_E_DTYPE;
    }
}

}  // namespace ddf

extern "C" {

int ddf_b200_nhwc_to_nchw(const void* src, void* dst, int B, int C, int H, int W, int dtype,
                          void* stream) {
    return ddf::layout_any<false>(src, dst, B, C, H, W, C, dtype, nullptr, nullptr, 0, stream);
}

int ddf_b200_nhwc_to_nchw_affine(const void* src, void* dst, int B, int C, int H, int W,
                                 int src_channels, int dtype, const float* ch_scale,
                                 const float* ch_shift, int relu, void* stream) {
    return ddf::layout_any<false>(src, dst, B, C, H, W, src_channels, dtype, ch_scale, ch_shift, relu,
                                  stream);
}

int ddf_b200_nchw_to_nhwc(const void* src, void* dst, int B, int C, int H, int W, int dtype,
                          const float* ch_scale, const float* ch_shift, int relu, void* stream) {
    return ddf::layout_any<true>(src, dst, B, C, H, W, C, dtype, ch_scale, ch_shift, relu, stream);
}

}  // extern "C"

// ---------------------------------------------------------------------------------------
// Front end of a DDF layer in a channels-last network, one pass over x (B,H,W,C):
//   x_nchw (B,C,H,W)          the op's input (the transpose above),
//   pooled (B,NT,C) float     per-channel sums over each 64-pixel tile: the global average
//                             pool of the channel branch (ddf/ddf.py:187) as partial sums
//                             that ddf_b200_channel_filter adds in a fixed order.
// The reference reads x once for each of these; here the tile that is being transposed
// through shared memory also feeds the sums.  (The spatial branch's 1x1 convolution is left
// to the tensor-core library: computed here on CUDA cores it cost more than it saved.)
namespace ddf {

constexpr int kFeMaxC = 2048;

template <typename T>
__global__ void __launch_bounds__(256)
frontend_kernel(const T* __restrict__ x, T* __restrict__ x_nchw, float* __restrict__ pooled,
                int C, int H, int W) {
    constexpr int PITCH = kTile + (sizeof(T) == 2 ? 2 : 1);
    __shared__ T tile[kTile][PITCH];  // [channel][pixel]
    const int t = threadIdx.x;
    const int HW = H * W;
    const int p0 = blockIdx.x * kTile;
    const long long b = blockIdx.y;
    const T* s = x + b * (long long)C * HW;
    T* d = x_nchw + b * (long long)C * HW;
    const int sub = t >> 4, q = (t & 15) * 4;
    const bool vec_hw = (HW % 4) == 0, vec_c = (C % 4) == 0;
    // pooled sums: thread = (channel of the tile, quarter of its pixels)
    const int pc = t >> 2, pq = t & 3;
    const int c0 = (int)blockIdx.z * kTile;

#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int p = p0 + r * 16 + sub, c = c0 + q;
        T v[4];
        if (p < HW && c < C) {
            load4(s + (long long)p * C + c, vec_c, C - c < 4 ? C - c : 4, v);
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = T(0.f);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) tile[q + i][r * 16 + sub] = v[i];
    }
    __syncthreads();
    // (1) transpose out
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int c = c0 + r * 16 + sub, p = p0 + q;
        if (c < C && p < HW) {
            T v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = tile[r * 16 + sub][q + i];
            store4(d + (long long)c * HW + p, vec_hw, HW - p < 4 ? HW - p : 4, v);
        }
    }
    // (2) per-channel sums over the tile's pixels (out-of-range entries are zero)
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) sum += (float)tile[pc][pq * 16 + i];
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    if (pq == 0 && c0 + pc < C)
        pooled[(b * gridDim.x + blockIdx.x) * (long long)C + c0 + pc] = sum;
}

template <typename T>
static int frontend_launch(const void* x, void* x_nchw, float* pooled, int B, int C, int H, int W,
                           cudaStream_t st) {
    const uintptr_t mask = sizeof(T) * 4 - 1;
    if ((reinterpret_cast<uintptr_t>(x) & mask) || (reinterpret_cast<uintptr_t>(x_nchw) & mask))
        return DDF_B200_E_UNSUPPORTED;
    const int HW = H * W;
    dim3 grid((unsigned)((HW + kTile - 1) / kTile), (unsigned)B, (unsigned)((C + kTile - 1) / kTile));
    if (grid.y > 65535u) return DDF_B200_E_TOO_LARGE;
    frontend_kernel<T><<<grid, 256, 0, st>>>((const T*)x, (T*)x_nchw, pooled, C, H, W);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}

}  // namespace ddf

extern "C" int ddf_b200_frontend_tiles(int H, int W) { return (H * W + ddf::kTile - 1) / ddf::kTile; }

extern "C" int ddf_b200_pack_frontend(const void* x_nhwc, void* x_nchw, float* pooled, int B, int C,
                                      int H, int W, int dtype, void* stream) {
    using namespace ddf;
    if (!x_nhwc || !x_nchw || !pooled) return DDF_B200_E_NULL;
    if (B < 1 || C < 1 || H < 1 || W < 1) return DDF_B200_E_SHAPE;
    if (C > kFeMaxC || (long long)H * W > (1ll << 30)) return DDF_B200_E_UNSUPPORTED;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    switch (dtype) {
        case DDF_B200_F32: return frontend_launch<float>(x_nhwc, x_nchw, pooled, B, C, H, W, st);
        case DDF_B200_F16: return frontend_launch<__half>(x_nhwc, x_nchw, pooled, B, C, H, W, st);
        case DDF_B200_BF16: return frontend_launch<__nv_bfloat16>(x_nhwc, x_nchw, pooled, B, C, H, W, st);
        default: return DDF_B200_E_DTYPE;
    }
}
