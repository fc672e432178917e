// Channels-innermost (NHWC, torch "channels_last") DDF forward for 2-byte element types, and
// the pooled sums the channel branch needs, so that a channels_last network runs its DDF
// layers without any layout copy.
//
// Mapping.  A thread owns 8 adjacent channels (one 16-byte vector) of one output pixel column.  Its channel-filter values -- K*K taps x 8 channels, fixed for a sample -- sit in
// registers as packed 2-byte pairs laid out like the input words (channels 2q, 2q+1 in word
// q), so the mixed-precision FMA forms x * cf for both halves of a word without any
// unpacking:  y = x * cf (exact in float),  acc = fma(y, sf, acc)  with the pixel's
// spatial-filter value in float.  The spatial filter is the same for all channels of a
// pixel: every thread takes its pixels' K*K values (adding the convolution bias and applying
// the spatial FilterNorm in float when asked to) once per pixel and reuses them for its 8
// channels.  The threads of a pixel read C contiguous channels -- full 128-byte lines --
// and the 3 x 3 window of a thread overlaps its neighbours', which the L1 cache
// absorbs: there is no shared-memory staging and no barrier in this kernel.  Pixels outside
// the image are not loaded (zeros take their place).  An optional per-channel affine map
// and ReLU (an eval-mode BatchNorm + activation) ride on the store.
#include <atomic>

#include "common.cuh"
#include "ring_fwd.cuh"

namespace ddf {

extern std::atomic<unsigned long long> g_launches;
int device_facts(int* sm_count, int** fault, int* index);

struct NhwcPlan {
    const void* x;          // (B, H, W, C)
    const void* cf;         // (B, C, K, K)
    const void* sf;         // K*K values per output pixel, addressed by the two strides below
    const float* sf_bias;   // K*K values added to the raw filter, or null
    void* out;              // (B, OH, OW, C)
    const float* oscale;    // per-channel output scale / shift, or null
    const float* oshift;
    int B, C, H, W, OH, OW;
    long long sf_batch_stride, sf_pixel_stride, sf_tap_stride;   // in elements
    int relu;
    float sf_scale;
    int vecs;               // C / 8
    int slots;              // strips a CTA works on = blockDim / vecs
    int strip_rows;         // output rows per strip
    int sf_vector;          // the K*K values of a pixel are contiguous and 16-byte aligned
};

__device__ __forceinline__ uint4 ldg128(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

template <typename T> __device__ __forceinline__ float elem_to_float(uint32_t h);
template <> __device__ __forceinline__ float elem_to_float<__nv_bfloat16>(uint32_t h) { return __uint_as_float(h << 16); }
template <> __device__ __forceinline__ float elem_to_float<__half>(uint32_t h) {
    return __uint_as_float(Mix<__half>::f32_bits(h));
}
template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b) { return Word<T>::put(a, b); }

constexpr int kNhwcThreads = 256;

// A thread walks a strip of output rows: PX adjacent columns wide, up to `strip_rows` high.
// Going down one output row it loads only the input rows it has not seen (one at stride 1,
// two at stride 2) and keeps the others in registers; the loop is unrolled by three so that
// the row rotation is register renaming, not moves.
// NORM: `sf` holds the raw output of the spatial branch's convolution; bias and FilterNorm here.
template <typename T, int S, int PX, int MODE, bool NORM>
__global__ void __launch_bounds__(kNhwcThreads, 2) nhwc_forward_kernel(const NhwcPlan pl) {
    constexpr int K = 3, KK = 9;
    constexpr int NCOL = (PX - 1) * S + 3;
    const int tid = threadIdx.x;
    const int vec = tid % pl.vecs, slot = tid / pl.vecs;
    const int b = blockIdx.y;
    const int C = pl.C, W = pl.W, H = pl.H, OW = pl.OW, OH = pl.OH;
    const int ppr = OW / PX;                                  // column groups per row
    const int strip = blockIdx.x * pl.slots + slot;
    const int seg = strip / ppr, cg = strip - seg * ppr;
    const int oy0 = seg * pl.strip_rows;
    if (oy0 >= OH) return;
    const int oy1 = (oy0 + pl.strip_rows) < OH ? (oy0 + pl.strip_rows) : OH;
    const int ox0 = cg * PX;
    const T* xb = reinterpret_cast<const T*>(pl.x) + (size_t)b * H * W * C + vec * 8;
    T* op = reinterpret_cast<T*>(pl.out) + ((size_t)b * OH * OW + (size_t)oy0 * OW + ox0) * C + vec * 8;
    const T* sp = reinterpret_cast<const T*>(pl.sf) + (long long)b * pl.sf_batch_stride +
                  ((long long)oy0 * OW + ox0) * pl.sf_pixel_stride;

    // channel filter of this thread's 8 channels: 72 contiguous values -> cfw[t][q] = channels (2q, 2q+1) of tap t
    uint32_t cfw[KK][4];
    {
        const uint4* cp = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(pl.cf) + ((size_t)b * C + vec * 8) * KK);
        uint32_t raw[36];
#pragma unroll
        for (int v = 0; v < 9; ++v) {
            const uint4 u = ldg128(cp + v);
            raw[4 * v] = u.x; raw[4 * v + 1] = u.y; raw[4 * v + 2] = u.z; raw[4 * v + 3] = u.w;
        }
#pragma unroll
        for (int t = 0; t < KK; ++t) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int ha = (2 * q) * KK + t, hb = (2 * q + 1) * KK + t;   // element indices
                const uint32_t lo = (ha & 1) ? (raw[ha / 2] >> 16) : (raw[ha / 2] & 0xffffu);
                const uint32_t hi = (hb & 1) ? (raw[hb / 2] & 0xffff0000u) : (raw[hb / 2] << 16);
                cfw[t][q] = lo | hi;
            }
        }
    }
    // which window columns lie inside the image (the same for every row of the strip)
    bool colok[NCOL];
#pragma unroll
    for (int cidx = 0; cidx < NCOL; ++cidx) {
        const int ix = ox0 * S + cidx - 1;
        colok[cidx] = ix >= 0 && ix < W;
    }
    const T* xcol = xb + (ptrdiff_t)(ox0 * S - 1) * C;   // window column 0 of input row 0
    auto load_row = [&](int iy, uint32_t (&v)[NCOL][4]) {
        const bool rowok = iy >= 0 && iy < H;
        const T* rp = xcol + (size_t)(rowok ? iy : 0) * W * C;
#pragma unroll
        for (int cidx = 0; cidx < NCOL; ++cidx) {
            uint4 u = make_uint4(0u, 0u, 0u, 0u);
            if (rowok && colok[cidx]) u = ldg128(rp + (size_t)cidx * C);
            v[cidx][0] = u.x; v[cidx][1] = u.y; v[cidx][2] = u.z; v[cidx][3] = u.w;
        }
    };

    // raw spatial-filter values of PX pixels as packed pairs (taps 2u, 2u+1)
    auto load_sf = [&](const T* spp0, uint32_t (&raw)[PX][5]) {
#pragma unroll
        for (int px = 0; px < PX; ++px) {
            const T* spp = spp0 + (long long)px * pl.sf_pixel_stride;
            if (pl.sf_vector) {   // K*K contiguous values, 16-byte aligned
                const uint4 u = ldg128(spp);
                raw[px][0] = u.x; raw[px][1] = u.y; raw[px][2] = u.z; raw[px][3] = u.w;
                raw[px][4] = __ldg(reinterpret_cast<const uint16_t*>(spp + 8));
            } else {
#pragma unroll
                for (int u = 0; u < 5; ++u) {
                    const uint32_t lo = __ldg(reinterpret_cast<const uint16_t*>(spp + (2 * u) * pl.sf_tap_stride));
                    const uint32_t hi = 2 * u + 1 < KK ? __ldg(reinterpret_cast<const uint16_t*>(spp + (2 * u + 1) * pl.sf_tap_stride)) : 0u;
                    raw[px][u] = lo | (hi << 16);
                }
            }
        }
    };
    uint32_t sraw[PX][5];
    load_sf(sp, sraw);
    // the spatial branch's bias (added before the FilterNorm), in registers for the whole strip
    float bias[NORM ? KK : 1];
    if constexpr (NORM) {
#pragma unroll
        for (int t = 0; t < KK; ++t) bias[t] = pl.sf_bias != nullptr ? __ldg(pl.sf_bias + t) : 0.f;
    }

    uint32_t w0[NCOL][4], w1[NCOL][4], w2[NCOL][4];   // input rows oy*S - 1, oy*S, oy*S + 1
    load_row(oy0 * S - 1, w0);
    if constexpr (S == 1) load_row(oy0, w1);

#pragma unroll 3
    for (int oy = oy0; oy < oy1; ++oy) {
        if constexpr (S == 2) load_row(oy * 2, w1);
        load_row(oy * S + 1, w2);
        // ---- the pixels' spatial-filter values in float (bias, FilterNorm); the raw values were
        // requested one row ahead, and the next row's are requested now
        float sfv[PX][KK];
#pragma unroll
        for (int px = 0; px < PX; ++px) {
#pragma unroll
            for (int t = 0; t < KK; ++t)
                sfv[px][t] = elem_to_float<T>((t & 1) ? (sraw[px][t / 2] >> 16) : (sraw[px][t / 2] & 0xffffu));
        }
        sp += (long long)OW * pl.sf_pixel_stride;
        if (oy + 1 < oy1) load_sf(sp, sraw);
#pragma unroll
        for (int px = 0; px < PX; ++px) {
            if constexpr (NORM) {
                float sum = 0.f;
#pragma unroll
                for (int t = 0; t < KK; ++t) {
                    sfv[px][t] += bias[t];
                    sum += sfv[px][t];
                }
                const float mean = sum * (1.f / KK);
                float var = 0.f;
#pragma unroll
                for (int t = 0; t < KK; ++t) {
                    sfv[px][t] -= mean;
                    var = fmaf(sfv[px][t], sfv[px][t], var);
                }
                const float inv = norm_gain(var * (1.f / (KK - 1)), pl.sf_scale);
#pragma unroll
                for (int t = 0; t < KK; ++t) sfv[px][t] *= inv;
            }
        }
        uint32_t sfh[PX][(KK + 1) / 2];   // add mode: the same values as packed 2-byte pairs (taps 2u, 2u+1)
        if constexpr (MODE == DDF_B200_ADD) {
#pragma unroll
            for (int px = 0; px < PX; ++px)
#pragma unroll
                for (int u = 0; u < (KK + 1) / 2; ++u)
                    sfh[px][u] = pack2<T>(sfv[px][2 * u], 2 * u + 1 < KK ? sfv[px][2 * u + 1] : 0.f);
        }

        float acc[PX][8];
#pragma unroll
        for (int px = 0; px < PX; ++px)
#pragma unroll
            for (int c = 0; c < 8; ++c) acc[px][c] = 0.f;
#pragma unroll
        for (int i = 0; i < K; ++i) {
#pragma unroll
            for (int j = 0; j < K; ++j) {
                const int t = i * K + j;
#pragma unroll
                for (int px = 0; px < PX; ++px) {
                    const int cidx = px * S + j;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint32_t xw = i == 0 ? w0[cidx][q] : (i == 1 ? w1[cidx][q] : w2[cidx][q]);
                        if constexpr (MODE == DDF_B200_MUL) {
                            // the two channels of a word: exact products, then one packed f32x2 FMA
                            // against the tap's spatial-filter value (half the issue slots of two FFMAs)
                            const float y0 = Mix<T>::fmaw(0, 0, xw, cfw[t][q], 0.f);
                            const float y1 = Mix<T>::fmaw(1, 1, xw, cfw[t][q], 0.f);
                            const unsigned long long r = f2_fma(f2_pack(y0, y1), f2_pack(sfv[px][t], sfv[px][t]),
                                                                f2_pack(acc[px][2 * q], acc[px][2 * q + 1]));
                            f2_unpack(r, acc[px][2 * q], acc[px][2 * q + 1]);
                        } else {
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                float a = acc[px][2 * q + h];
                                a = Mix<T>::fmaw(h, h, xw, cfw[t][q], a);
                                a = Mix<T>::fmaw(h, t & 1, xw, sfh[px][t / 2], a);
                                acc[px][2 * q + h] = a;
                            }
                        }
                    }
                }
            }
        }
#pragma unroll
        for (int px = 0; px < PX; ++px) {
            float r[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) r[c] = acc[px][c];
            if (pl.oscale != nullptr) {
                const float4* sc = reinterpret_cast<const float4*>(pl.oscale + vec * 8);
                const float4* sh = reinterpret_cast<const float4*>(pl.oshift + vec * 8);
                const float4 a0 = __ldg(sc), a1 = __ldg(sc + 1), b0 = __ldg(sh), b1 = __ldg(sh + 1);
                r[0] = fmaf(r[0], a0.x, b0.x); r[1] = fmaf(r[1], a0.y, b0.y); r[2] = fmaf(r[2], a0.z, b0.z); r[3] = fmaf(r[3], a0.w, b0.w);
                r[4] = fmaf(r[4], a1.x, b1.x); r[5] = fmaf(r[5], a1.y, b1.y); r[6] = fmaf(r[6], a1.z, b1.z); r[7] = fmaf(r[7], a1.w, b1.w);
            }
            if (pl.relu) {
#pragma unroll
                for (int c = 0; c < 8; ++c) r[c] = fmaxf(r[c], 0.f);
            }
            const uint4 o = make_uint4(pack2<T>(r[0], r[1]), pack2<T>(r[2], r[3]), pack2<T>(r[4], r[5]), pack2<T>(r[6], r[7]));
            *reinterpret_cast<uint4*>(op + (size_t)px * C) = o;
        }
        op += (size_t)OW * C;
        // rotate the rows: what was below becomes what is above
        if constexpr (S == 1) {
#pragma unroll
            for (int cidx = 0; cidx < NCOL; ++cidx)
#pragma unroll
                for (int q = 0; q < 4; ++q) { w0[cidx][q] = w1[cidx][q]; w1[cidx][q] = w2[cidx][q]; }
        } else {
#pragma unroll
            for (int cidx = 0; cidx < NCOL; ++cidx)
#pragma unroll
                for (int q = 0; q < 4; ++q) w0[cidx][q] = w2[cidx][q];
        }
    }
}

// Partial sums of x over tiles of 196 pixels: partials[b][tile][c] (float), for the channel branch's
// global average pool.  One CTA per (tile, sample).
constexpr int kPoolTile = 196;
template <typename T>
__global__ void __launch_bounds__(256) nhwc_pool_kernel(const T* __restrict__ x, float* __restrict__ partials, int C,
                                                        int HW, int n_tiles) {
    extern __shared__ float red[];   // [lanes][C]
    const int vecs = C / 8, tid = threadIdx.x;
    const int vec = tid % vecs, lane = tid / vecs, lanes = blockDim.x / vecs;
    const int b = blockIdx.y, tile = blockIdx.x;
    const int p0 = tile * kPoolTile, p1 = (p0 + kPoolTile) < HW ? (p0 + kPoolTile) : HW;
    float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const T* xb = x + (size_t)b * HW * C + vec * 8;
    for (int p = p0 + lane; p < p1; p += lanes) {
        const uint4 u = ldg128(xb + (size_t)p * C);
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            s[2 * q] += elem_to_float<T>(w[q] & 0xffffu);
            s[2 * q + 1] += elem_to_float<T>(w[q] >> 16);
        }
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) red[lane * C + vec * 8 + c] = s[c];
    __syncthreads();
    for (int c = tid; c < C; c += blockDim.x) {
        float t = 0.f;
        for (int l = 0; l < lanes; ++l) t += red[l * C + c];   // fixed order
        partials[((size_t)b * n_tiles + tile) * C + c] = t;
    }
}

template <typename T, int S, int PX>
static int nhwc_launch(const NhwcPlan& pl, int combine, int norm, dim3 grid, cudaStream_t st) {
    if (combine == DDF_B200_MUL) {
        if (norm) nhwc_forward_kernel<T, S, PX, DDF_B200_MUL, true><<<grid, kNhwcThreads, 0, st>>>(pl);
        else nhwc_forward_kernel<T, S, PX, DDF_B200_MUL, false><<<grid, kNhwcThreads, 0, st>>>(pl);
    } else {
        if (norm) nhwc_forward_kernel<T, S, PX, DDF_B200_ADD, true><<<grid, kNhwcThreads, 0, st>>>(pl);
        else nhwc_forward_kernel<T, S, PX, DDF_B200_ADD, false><<<grid, kNhwcThreads, 0, st>>>(pl);
    }
    return (int)cudaGetLastError();
}

// One pixel column per thread: two columns would halve the window loads per output but need
// 48 registers for the window alone, which does not fit beside the resident channel filter.
constexpr int kNhwcPX = 1;

template <typename T>
static int nhwc_dispatch(const NhwcPlan& pl, int s, int combine, int norm, dim3 grid, cudaStream_t st) {
    if (s == 1) return nhwc_launch<T, 1, kNhwcPX>(pl, combine, norm, grid, st);
    return nhwc_launch<T, 2, kNhwcPX>(pl, combine, norm, grid, st);
}

}  // namespace ddf

using namespace ddf;

extern "C" {

int ddf_b200_pool_nhwc_tiles(int H, int W) {
    if (H < 1 || W < 1) return DDF_B200_E_SHAPE;
    return (H * W + kPoolTile - 1) / kPoolTile;
}

int ddf_b200_pool_nhwc(const void* x, float* partials, int B, int C, int H, int W, int dtype, void* stream) {
    if (!x || !partials) return DDF_B200_E_NULL;
    if (B < 1 || C < 1 || H < 1 || W < 1) return DDF_B200_E_SHAPE;
    if (dtype != DDF_B200_F16 && dtype != DDF_B200_BF16) return DDF_B200_E_UNSUPPORTED;
    if (C % 8 != 0 || C > 2048 || 256 % (C / 8) != 0 || B > 65535) return DDF_B200_E_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(x) & 15u) != 0) return DDF_B200_E_UNSUPPORTED;
    const int nt = (H * W + kPoolTile - 1) / kPoolTile;
    const int lanes = 256 / (C / 8);
    const size_t smem = (size_t)lanes * C * sizeof(float);   // = 8 KB
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    dim3 grid((unsigned)nt, (unsigned)B);
    if (dtype == DDF_B200_F16)
        nhwc_pool_kernel<__half><<<grid, 256, smem, st>>>((const __half*)x, partials, C, H * W, nt);
    else
        nhwc_pool_kernel<__nv_bfloat16><<<grid, 256, smem, st>>>((const __nv_bfloat16*)x, partials, C, H * W, nt);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return (int)cudaGetLastError();
}

int ddf_b200_forward_nhwc(const void* x, const void* cf, const void* sf, const float* sf_bias, void* out,
                          const float* out_scale, const float* out_shift, int relu, int B, int C, int H, int W,
                          int k, int d, int s, int combine, int dtype, long long sf_batch_stride,
                          long long sf_pixel_stride, long long sf_tap_stride, int norm, double sf_scale,
                          void* stream) {
    if (!x || !cf || !sf || !out) return DDF_B200_E_NULL;
    if ((out_scale == nullptr) != (out_shift == nullptr)) return DDF_B200_E_NULL;
    if (B < 1 || C < 1 || H < 1 || W < 1 || s < 1 || H / s < 1 || W / s < 1) return DDF_B200_E_SHAPE;
    if (combine != DDF_B200_MUL && combine != DDF_B200_ADD) return DDF_B200_E_COMBINE;
    if (dtype < DDF_B200_F32 || dtype > DDF_B200_F64) return DDF_B200_E_DTYPE;
    if (k < 1 || (k - 1) % 2 != 0 || d < 1) return DDF_B200_E_KERNEL;
    // built for the DDF-ResNet layers: k = 3, d = 1, stride 1 or 2, 2-byte types, C a multiple of 8
    if (k != 3 || d != 1 || s > 2 || (dtype != DDF_B200_F16 && dtype != DDF_B200_BF16)) return DDF_B200_E_UNSUPPORTED;
    if (C % 8 != 0 || C > 2048 || kNhwcThreads % (C / 8) != 0 || B > 65535) return DDF_B200_E_UNSUPPORTED;
    if (W != (W / s) * s) return DDF_B200_E_UNSUPPORTED;
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    if (!al16(x) || !al16(cf) || !al16(out)) return DDF_B200_E_UNSUPPORTED;
    int sm_count = 0, index = 0;
    int* fault = nullptr;
    int rc = device_facts(&sm_count, &fault, &index);
    if (rc) return rc;

    NhwcPlan pl;
    pl.x = x; pl.cf = cf; pl.sf = sf; pl.sf_bias = sf_bias; pl.out = out;
    pl.oscale = out_scale; pl.oshift = out_shift;
    pl.B = B; pl.C = C; pl.H = H; pl.W = W; pl.OH = H / s; pl.OW = W / s;
    pl.sf_batch_stride = sf_batch_stride; pl.sf_pixel_stride = sf_pixel_stride; pl.sf_tap_stride = sf_tap_stride;
    pl.relu = relu; pl.sf_scale = (float)sf_scale;
    pl.vecs = C / 8;
    pl.slots = kNhwcThreads / pl.vecs;
    // Strips of output rows, PX columns wide: long enough that the two extra input rows a
    // strip reads are a small share, short enough that there are a few CTAs per SM.
    const int ppr = pl.OW / kNhwcPX;
    int rows = pl.OH < 8 ? pl.OH : 8;
    auto n_ctas = [&](int r) { return (long long)B * (((long long)ppr * ((pl.OH + r - 1) / r) + pl.slots - 1) / pl.slots); };
    while (rows > 2 && n_ctas(rows) < 4ll * sm_count) rows = (rows + 1) / 2;
    pl.strip_rows = rows;
    const long long strips = (long long)ppr * ((pl.OH + rows - 1) / rows);
    dim3 grid((unsigned)((strips + pl.slots - 1) / pl.slots), (unsigned)B);
    // vector loads of the spatial filter: taps contiguous, pixels 16-byte aligned
    pl.sf_vector = (sf_tap_stride == 1 && sf_pixel_stride % 8 == 0 && sf_batch_stride % 8 == 0 && al16(sf)) ? 1 : 0;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    rc = dtype == DDF_B200_F16 ? nhwc_dispatch<__half>(pl, s, combine, norm, grid, st)
                               : nhwc_dispatch<__nv_bfloat16>(pl, s, combine, norm, grid, st);
    if (rc == 0) g_launches.fetch_add(1, std::memory_order_relaxed);
    return rc;
}

}  // extern "C"
