// Shared definitions for the DDF kernels: element-type traits, the problem
// descriptor passed from the C ABI to the launchers, and thin PTX wrappers
// (mbarrier, bulk async copy, packed f32x2 arithmetic) for sm_100a.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ddf_b200.h"

namespace ddf {

// ------------------------------------------------------------------ problem descriptor
struct Problem {
    int B, C, H, W;    // input (for the backward: the shape of x / gx)
    int OH, OW;        // H / s, W / s
    int k, d, s;
    int combine;       // DDF_B200_MUL / DDF_B200_ADD
    int dtype;         // DDF_B200_F32 ...
    // Forward only: `sf` holds the raw output of the spatial branch's 1x1 convolution and
    // the kernel applies the spatial FilterNorm itself (ddf/ddf.py:146-157): per sample and
    // pixel, over the k*k taps, (v - mean) / (unbiased std + 1e-10) * sf_scale.
    int sf_norm = 0;
    double sf_scale = 1.0;
};

// Status used internally by launchers that may decline a problem.
constexpr int kNotHandled = 1 << 30;

// ------------------------------------------------------------------ element traits
template <typename T> struct Elem;
template <> struct Elem<float> {
    using acc_t = float;
    static __device__ __forceinline__ float load(const float* p) { return __ldg(p); }
    static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
};
template <> struct Elem<double> {
    using acc_t = double;
    static __device__ __forceinline__ double load(const double* p) { return __ldg(p); }
    static __device__ __forceinline__ void store(double* p, double v) { *p = v; }
};
template <> struct Elem<__half> {
    using acc_t = float;
    static __device__ __forceinline__ float load(const __half* p) {
        return __half2float(__ldg(p));
    }
    static __device__ __forceinline__ void store(__half* p, float v) { *p = __float2half_rn(v); }
};
template <> struct Elem<__nv_bfloat16> {
    using acc_t = float;
    static __device__ __forceinline__ float load(const __nv_bfloat16* p) {
        return __bfloat162float(__ldg(p));
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) {
        *p = __float2bfloat16_rn(v);
    }
};

template <int MODE, typename A>
__device__ __forceinline__ A combine_w(A cfv, A sfv) {
    return MODE == DDF_B200_MUL ? cfv * sfv : cfv + sfv;
}

// ------------------------------------------------------------------ shared-memory PTX
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
// One probe: true when the phase with this parity has completed.  Used by the
// service warps' polling loops, which must stay responsive to several barriers.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after about a second (kWaitCycles SM clocks).  Returns
// false when the limit ran out (the caller records a fault and leaves); never
// spins forever.  mbarrier.try_wait without a time hint blocks for a short,
// hardware-chosen time and returns as soon as the phase completes; the hinted form
// compiles to sleep loops that add microseconds to every stage hand-over.
constexpr long long kWaitCycles = 2000000000ll;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_test(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i)
            if (mbar_test(bar, parity)) return true;
        if (clock64() - t0 > kWaitCycles) return false;
    }
}

// Bulk asynchronous copy global -> shared (TMA, untiled).  dst, src 16-byte
// aligned, bytes a multiple of 16.  Completion is counted on `bar`.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes,
                                         uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
            "r"(dst),
        "l"(__cvta_generic_to_global(src)), "r"(bytes), "r"(bar)
        : "memory");
}

__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
// Volatile form: for values read from a buffer that is handed back (mbarrier arrive) right after
// the read and kept in registers for a long time.  The assembler may otherwise move or repeat a
// plain ld.shared closer to its first use, i.e. past the hand-back, where the buffer may already
// hold the next data.
__device__ __forceinline__ uint32_t lds32v(uint32_t a) {
    uint32_t v;
    asm volatile("ld.volatile.shared.b32 %0, [%1];" : "=r"(v) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t lds16v(uint32_t a) {
    uint16_t v;
    asm volatile("ld.volatile.shared.u16 %0, [%1];" : "=h"(v) : "r"(a) : "memory");
    return v;
}
__device__ __forceinline__ void lds64v(uint32_t a, uint32_t& x, uint32_t& y) {
    asm volatile("ld.volatile.shared.v2.b32 {%0, %1}, [%2];" : "=r"(x), "=r"(y) : "r"(a) : "memory");
}
__device__ __forceinline__ void lds128v(uint32_t a, uint32_t& x, uint32_t& y, uint32_t& z, uint32_t& w) {
    asm volatile("ld.volatile.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(x), "=r"(y), "=r"(z), "=r"(w)
                 : "r"(a)
                 : "memory");
}
__device__ __forceinline__ uint32_t lds16(uint32_t a) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void lds64(uint32_t a, uint32_t& x, uint32_t& y) {
    asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(x), "=r"(y) : "r"(a));
}
__device__ __forceinline__ void lds128(uint32_t a, uint32_t& x, uint32_t& y, uint32_t& z,
                                       uint32_t& w) {
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(x), "=r"(y), "=r"(z), "=r"(w)
                 : "r"(a));
}
__device__ __forceinline__ float ldsf(uint32_t a) { return __uint_as_float(lds32(a)); }
__device__ __forceinline__ unsigned long long lds64_pair(uint32_t a) {
    unsigned long long v;
    asm volatile("ld.shared.b64 %0, [%1];" : "=l"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ void sts64(uint32_t a, uint32_t x, uint32_t y) {
    asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(a), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void sts32(uint32_t a, uint32_t v) {
    asm volatile("st.shared.b32 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}

__device__ __forceinline__ void sts16(uint32_t a, uint32_t v) {
    asm volatile("st.shared.u16 [%0], %1;" ::"r"(a), "h"((uint16_t)v) : "memory");
}

// Copy-issuer helper: bytes [g0, g1) of a tensor (16-byte aligned base, `total` bytes) go to
// shared memory such that byte g lands at dst + (g - (g0 & ~15)).  The aligned superset is
// fetched by one bulk copy, clamped to the tensor's last whole 16 bytes; what is left of a
// ragged end is fetched with plain 2-byte loads.  span_prepare does the plain part and
// returns the bulk part; call it before mbarrier.arrive.expect_tx, span_issue after.
struct Span { uint32_t dst; const char* src; uint32_t bytes; };
__device__ __forceinline__ Span span_prepare(uint32_t dst, const void* base, unsigned long long g0,
                                             unsigned long long g1, unsigned long long total) {
    const unsigned long long a0 = g0 & ~15ull;
    unsigned long long a1 = (g1 + 15ull) & ~15ull;
    const unsigned long long lim = total & ~15ull;
    if (a1 > lim) a1 = lim;
    if (a1 < a0) a1 = a0;
    const char* b = reinterpret_cast<const char*>(base);
    for (unsigned long long g = (a1 > g0 ? a1 : g0); g < g1; g += 2) {
        uint16_t v;
        asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(b + g));
        sts16(dst + (uint32_t)(g - a0), v);
    }
    return Span{dst, b + a0, (uint32_t)(a1 - a0)};
}
__device__ __forceinline__ void span_issue(const Span& s, uint32_t bar) {
    if (s.bytes) bulk_g2s(s.dst, s.src, s.bytes, bar);
}

// ------------------------------------------------------------------ packed f32x2
__device__ __forceinline__ unsigned long long f2_pack(float a, float b) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void f2_unpack(unsigned long long v, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ unsigned long long f2_fma(unsigned long long a, unsigned long long b,
                                                     unsigned long long c) {
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ unsigned long long f2_mul(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ unsigned long long f2_add(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

// ------------------------------------------------------------------ raw word <-> float
// A 32-bit word holds EPW = 4 / sizeof(T) elements; element 0 is the low half.
template <typename T> struct Word;
template <> struct Word<float> {
    static constexpr int EPW = 1;
    static __device__ __forceinline__ float get(uint32_t w, int) { return __uint_as_float(w); }
    static __device__ __forceinline__ uint32_t put(float a, float) { return __float_as_uint(a); }
};
template <> struct Word<__nv_bfloat16> {
    static constexpr int EPW = 2;
    static __device__ __forceinline__ float get(uint32_t w, int e) {
        return __uint_as_float(e == 0 ? (w << 16) : (w & 0xffff0000u));
    }
    static __device__ __forceinline__ uint32_t put(float a, float b) {
        __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&v);
    }
};
template <> struct Word<__half> {
    static constexpr int EPW = 2;
    static __device__ __forceinline__ float get(uint32_t w, int e) {
        __half2 h = *reinterpret_cast<__half2*>(&w);
        return e == 0 ? __low2float(h) : __high2float(h);
    }
    static __device__ __forceinline__ uint32_t put(float a, float b) {
        __half2 v = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t*>(&v);
    }
};

// Per-device fault word written by the streaming kernels (see take_fault()).
enum Fault : int {
    kFaultNone = 0,
    kFaultConsumerFull = 1,   // a compute warp gave up waiting for a stage to land
    kFaultConsumerSf = 2,     // a compute warp gave up waiting for the spatial filter
    kFaultService = 3,        // the service warp made no progress for the whole limit
    kFaultDrain = 4,          // copies still in flight when the service warp left
};

}  // namespace ddf
