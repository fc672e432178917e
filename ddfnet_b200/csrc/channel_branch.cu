// The channel branch of a DDF layer after its global average pool, as one kernel:
//   h   = relu(W1 g + b1)                      (1x1 convolution C -> mid, ReLU)
//   r   = W2 h + b2                            (1x1 convolution mid -> C*k*k)
//   cf  = (r - mean_t r) / (std_t r + 1e-10) * gain[c*k*k + t]    per sample and channel,
//                                              over the k*k taps, std unbiased
// i.e. build_channel_branch (ddf/ddf.py:183-192) minus its AdaptiveAvgPool2d, including
// FilterNorm(filter_type='channel', running_std=True) (ddf/ddf.py:158-170).  The reference
// runs this as about ten small launches per layer; all arithmetic here is float.
//
// One CTA (16 warps) serves kSB = 4 samples and a slice of CW <= 256 channels; in the second
// layer a thread owns one channel and two of the samples.  Both weight matrices reach
// the CTA through a ring of shared-memory slots filled by untiled TMA bulk copies (one
// elected thread issues them a few chunks ahead), so the inner loops read shared memory
// only: with a single CTA of eight warps per SM, loops over global loads were bound by
// L2 latency (about 1 us per hidden unit).  To make every chunk one contiguous run, W2 is
// passed re-laid-out as (C / CW, mid, k*k, CW): slice, hidden unit, tap, channel in slice.
// The pooled vector g may arrive as partial sums (added here in a fixed order, scaled by
// pool_scale).  Waits on the ring are bounded like those of the streaming kernels.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>

#include "../../include/ddf_b200.h"
#include "common.cuh"

namespace ddf {

extern std::atomic<unsigned long long> g_launches;
int device_facts(int* sm_count, int** fault, int* index);

constexpr int kSB = 4;               // samples per CTA
constexpr int kCbSlice = 256;        // widest channel slice of a CTA
constexpr int kCbThreads = 512;      // 16 warps: two threads per channel, two samples each
constexpr int kCbSlots = 3;
constexpr uint32_t kCbChunk = 48 * 1024;  // bytes per ring slot
constexpr int kCbMaxC = 2048;
constexpr int kCbMaxMid = 512;
constexpr int kFaultChannelBranch = 5;

// element -> float through the read-only path
template <typename T>
__device__ __forceinline__ float ldf(const T* p) { return (float)Elem<T>::load(p); }

template <typename T>
__device__ __forceinline__ float lds_elem(uint32_t a) {
    if constexpr (sizeof(T) == 4) return __uint_as_float(lds32(a));
    else return Word<T>::get(lds16(a), 0);
}

struct CbPlan {
    const float* pooled;
    int n_part;
    float pool_scale;
    const void *w1, *b1, *w2s, *b2, *gain;
    void* cf;
    int B, C, mid, CW;
    int rows_per_chunk;  // W1 rows (hidden units) per ring chunk
    int m_per_chunk;     // hidden units of the W2 slice per ring chunk
    int n_chunks_a, n_chunks_b;
    uint32_t off_h, off_ring;
    int* fault;
};

template <typename T, int KK>
__global__ void __launch_bounds__(kCbThreads)
channel_branch_kernel(const __grid_constant__ CbPlan pl) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const uint32_t sbase = smem_u32(smem_raw);
    float* g = reinterpret_cast<float*>(smem_raw + 64);          // [kSB][C]
    float* h = reinterpret_cast<float*>(smem_raw + pl.off_h);    // [mid][kSB]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int C = pl.C, mid = pl.mid, CW = pl.CW;
    const int b0 = blockIdx.x * kSB;
    const int nb = (pl.B - b0) < kSB ? (pl.B - b0) : kSB;
    constexpr int ES = (int)sizeof(T);
    constexpr int NW = kCbThreads / 32;

#define CB_FULL(s) (sbase + 8u * (uint32_t)(s))
#define CB_EMPTY(s) (sbase + 8u * (uint32_t)(kCbSlots + (s)))
#define CB_SLOT(s) (sbase + pl.off_ring + (uint32_t)(s) * kCbChunk)
    if (tid == 0) {
        for (int s = 0; s < kCbSlots; ++s) {
            mbar_init(CB_FULL(s), 1);
            mbar_init(CB_EMPTY(s), NW);
        }
        mbar_fence_init();
    }
    __syncthreads();

    // Chunk i of the stream: first the n_chunks_a chunks of W1, then the n_chunks_b chunks
    // of this CTA's W2 slice.
    const int n_chunks = pl.n_chunks_a + pl.n_chunks_b;
    const char* w2_slice = reinterpret_cast<const char*>(pl.w2s) +
                           (size_t)blockIdx.y * (size_t)mid * KK * CW * ES;
    auto issue = [&](int i) {  // thread 0 only
        const int slot = i % kCbSlots;
        const char* src;
        uint32_t bytes;
        if (i < pl.n_chunks_a) {
            const int r0 = i * pl.rows_per_chunk;
            const int nr = (mid - r0) < pl.rows_per_chunk ? (mid - r0) : pl.rows_per_chunk;
            src = reinterpret_cast<const char*>(pl.w1) + (size_t)r0 * C * ES;
            bytes = (uint32_t)nr * (uint32_t)C * ES;
        } else {
            const int m0 = (i - pl.n_chunks_a) * pl.m_per_chunk;
            const int nm = (mid - m0) < pl.m_per_chunk ? (mid - m0) : pl.m_per_chunk;
            src = w2_slice + (size_t)m0 * KK * CW * ES;
            bytes = (uint32_t)nm * KK * (uint32_t)CW * ES;
        }
        mbar_arrive_expect_tx(CB_FULL(slot), bytes);
        bulk_g2s(CB_SLOT(slot), src, bytes, CB_FULL(slot));
    };
    if (tid == 0) {
        for (int i = 0; i < kCbSlots - 1 && i < n_chunks; ++i) issue(i);
    }

    // pooled vector of this CTA's samples: fixed-order sum of the partials
#pragma unroll 4
    for (int i = tid; i < kSB * C; i += kCbThreads) {
        const int s = i / C, c = i - s * C;
        float v = 0.f;
        if (s < nb) {
            const float* p = pl.pooled + ((long long)(b0 + s) * pl.n_part) * C + c;
            for (int q = 0; q < pl.n_part; ++q) v += p[(long long)q * C];
            v *= pl.pool_scale;
        }
        g[i] = v;
    }
    // first-layer biases, parked in the slots of the hidden vector they will be added to
    // (a global load per hidden unit inside the loop would cost an L2 round trip each)
    for (int m = tid; m < mid; m += kCbThreads) h[m * kSB] = ldf(reinterpret_cast<const T*>(pl.b1) + m);
    __syncthreads();

    // second-layer accumulators of this thread's channel (threads beyond the slice idle there)
    constexpr int ST = 2;                      // samples per thread in the second layer
    const int ch = tid & (kCbSlice - 1);       // channel within the slice
    const int s0 = (tid / kCbSlice) * ST;      // first of the thread's samples (warp-uniform)
    const bool has_channel = ch < CW;
    const int c = blockIdx.y * CW + (has_channel ? ch : 0);
    float r[KK][ST];
#pragma unroll
    for (int t = 0; t < KK; ++t) {
        const float bias = ldf(reinterpret_cast<const T*>(pl.b2) + (long long)c * KK + t);
#pragma unroll
        for (int s = 0; s < ST; ++s) r[t][s] = bias;
    }

    for (int i = 0; i < n_chunks; ++i) {
        const int slot = i % kCbSlots;
        // keep the ring full: the chunk kCbSlots-1 ahead goes into the slot chunk i-1 used
        if (tid == 0 && i + kCbSlots - 1 < n_chunks) {
            const int j = i + kCbSlots - 1;
            if (j >= kCbSlots && !mbar_wait(CB_EMPTY(j % kCbSlots), (uint32_t)((j / kCbSlots - 1) & 1))) {
                atomicCAS(pl.fault, 0, kFaultChannelBranch);
                // fall through without issuing: the consumers' bounded waits end the kernel
            } else {
                issue(j);
            }
        }
        if (i == pl.n_chunks_a) __syncthreads();  // every h value written before the second layer
        if (!mbar_wait(CB_FULL(slot), (uint32_t)((i / kCbSlots) & 1))) {
            atomicCAS(pl.fault, 0, kFaultChannelBranch);
            return;
        }
        const uint32_t base = CB_SLOT(slot);
        if (i < pl.n_chunks_a) {
            // first layer: one warp per hidden unit of the chunk, lanes over the channels
            const int r0 = i * pl.rows_per_chunk;
            const int nr = (mid - r0) < pl.rows_per_chunk ? (mid - r0) : pl.rows_per_chunk;
            for (int rr = warp; rr < nr; rr += NW) {
                float acc[kSB];
#pragma unroll
                for (int s = 0; s < kSB; ++s) acc[s] = 0.f;
                const uint32_t row = base + (uint32_t)rr * (uint32_t)C * ES;
                for (int cc = lane; cc < C; cc += 32) {
                    const float w = lds_elem<T>(row + (uint32_t)cc * ES);
#pragma unroll
                    for (int s = 0; s < kSB; ++s) acc[s] = fmaf(w, g[s * C + cc], acc[s]);
                }
#pragma unroll
                for (int s = 0; s < kSB; ++s) {
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) acc[s] += __shfl_xor_sync(0xffffffffu, acc[s], o);
                }
                if (lane == 0) {
                    const int m = r0 + rr;
                    const float bias = h[m * kSB];  // parked there before the loop
#pragma unroll
                    for (int s = 0; s < kSB; ++s) h[m * kSB + s] = fmaxf(acc[s] + bias, 0.f);
                }
            }
        } else if (has_channel) {
            // second layer: this thread's channel, the chunk's hidden units
            const int m0 = (i - pl.n_chunks_a) * pl.m_per_chunk;
            const int nm = (mid - m0) < pl.m_per_chunk ? (mid - m0) : pl.m_per_chunk;
            uint32_t wa = base + (uint32_t)ch * ES;
#pragma unroll 2
            for (int mm = 0; mm < nm; ++mm) {
                const float2 hv = *reinterpret_cast<const float2*>(h + (m0 + mm) * kSB + s0);
#pragma unroll
                for (int t = 0; t < KK; ++t) {
                    const float w = lds_elem<T>(wa + (uint32_t)(t * CW) * ES);
                    r[t][0] = fmaf(w, hv.x, r[t][0]);
                    r[t][1] = fmaf(w, hv.y, r[t][1]);
                }
                wa += (uint32_t)(KK * CW) * ES;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(CB_EMPTY(slot));
    }
#undef CB_FULL
#undef CB_EMPTY
#undef CB_SLOT
    if (!has_channel) return;

    // FilterNorm over the taps, gain, store
    float gn[KK];
#pragma unroll
    for (int t = 0; t < KK; ++t) gn[t] = ldf(reinterpret_cast<const T*>(pl.gain) + (long long)c * KK + t);
#pragma unroll
    for (int s = 0; s < ST; ++s) {
        if (s0 + s >= nb) break;
        float sum = 0.f;
#pragma unroll
        for (int t = 0; t < KK; ++t) sum += r[t][s];
        const float mean = sum * (1.f / KK);
        float var = 0.f;
#pragma unroll
        for (int t = 0; t < KK; ++t) {
            const float dv = r[t][s] - mean;
            var = fmaf(dv, dv, var);
        }
        const float inv = 1.f / (sqrtf(var * (1.f / (KK - 1))) + 1e-10f);
        T* o = reinterpret_cast<T*>(pl.cf) + ((long long)(b0 + s0 + s) * C + c) * KK;
#pragma unroll
        for (int t = 0; t < KK; ++t) o[t] = (T)((r[t][s] - mean) * inv * gn[t]);
    }
}

template <typename T>
static int channel_branch_launch(CbPlan& pl, int k, int device, cudaStream_t st) {
    static_assert(kSB == 4 && kCbThreads == 2 * kCbSlice, "two threads per channel, two samples each");
    constexpr int ES = (int)sizeof(T);
    const int KK = k * k;
    pl.rows_per_chunk = (int)(kCbChunk / ((uint32_t)pl.C * ES));
    pl.m_per_chunk = (int)(kCbChunk / ((uint32_t)KK * pl.CW * ES));
    if (pl.rows_per_chunk < 1 || pl.m_per_chunk < 1) return DDF_B200_E_UNSUPPORTED;
    pl.n_chunks_a = (pl.mid + pl.rows_per_chunk - 1) / pl.rows_per_chunk;
    pl.n_chunks_b = (pl.mid + pl.m_per_chunk - 1) / pl.m_per_chunk;
    pl.off_h = 64u + (uint32_t)(kSB * pl.C) * 4u;              // multiple of 16
    pl.off_ring = (pl.off_h + (uint32_t)(kSB * pl.mid) * 4u + 127u) & ~127u;
    const size_t smem = pl.off_ring + (size_t)kCbSlots * kCbChunk;
    dim3 grid((unsigned)((pl.B + kSB - 1) / kSB), (unsigned)(pl.C / pl.CW));
    auto launch = [&](auto kern, std::atomic<unsigned long long>& opted) -> int {
        const unsigned long long bit = 1ull << (device & 63);
        if (!(opted.load(std::memory_order_acquire) & bit)) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 200 * 1024);
            if (e != cudaSuccess) return (int)e;
            opted.fetch_or(bit, std::memory_order_release);
        }
        kern<<<grid, kCbThreads, smem, st>>>(pl);
        return (int)cudaGetLastError();
    };
    static std::atomic<unsigned long long> opted9{0}, opted25{0};
    int rc;
    if (k == 3) rc = launch(channel_branch_kernel<T, 9>, opted9);
    else rc = launch(channel_branch_kernel<T, 25>, opted25);
    if (rc == 0) g_launches.fetch_add(1, std::memory_order_relaxed);
    return rc;
}

}  // namespace ddf

extern "C" int ddf_b200_channel_filter_slice(int C) {
    // channels per slice of the re-laid-out second weight
    return C >= ddf::kCbSlice ? ddf::kCbSlice : C;
}

extern "C" int ddf_b200_channel_filter(const float* pooled, int n_partials, float pool_scale,
                                       const void* w1, const void* b1, const void* w2s,
                                       const void* b2, const void* gain, void* cf, int B, int C,
                                       int mid, int k, int dtype, void* stream) {
    using namespace ddf;
    if (!pooled || !w1 || !b1 || !w2s || !b2 || !gain || !cf) return DDF_B200_E_NULL;
    if (B < 1 || C < 1 || mid < 1 || n_partials < 1) return DDF_B200_E_SHAPE;
    if (k != 3 && k != 5) return DDF_B200_E_UNSUPPORTED;
    const int CW = ddf_b200_channel_filter_slice(C);
    // bulk copies: 16-byte aligned sources, rows and slices that are multiples of 16 bytes
    if (C > kCbMaxC || mid > kCbMaxMid || C % 8 != 0 || C % CW != 0) return DDF_B200_E_UNSUPPORTED;
    if ((reinterpret_cast<uintptr_t>(w1) & 15u) || (reinterpret_cast<uintptr_t>(w2s) & 15u))
        return DDF_B200_E_UNSUPPORTED;
    int sm = 0, index = 0;
    int* fault = nullptr;
    int rc = device_facts(&sm, &fault, &index);
    if (rc) return rc;
    CbPlan pl{};
    pl.pooled = pooled; pl.n_part = n_partials; pl.pool_scale = pool_scale;
    pl.w1 = w1; pl.b1 = b1; pl.w2s = w2s; pl.b2 = b2; pl.gain = gain; pl.cf = cf;
    pl.B = B; pl.C = C; pl.mid = mid; pl.CW = CW; pl.fault = fault;
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    switch (dtype) {
        case DDF_B200_F32: return channel_branch_launch<float>(pl, k, index, st);
        case DDF_B200_F16: return channel_branch_launch<__half>(pl, k, index, st);
        case DDF_B200_BF16: return channel_branch_launch<__nv_bfloat16>(pl, k, index, st);
        default: return DDF_B200_E_DTYPE;
    }
}
