// Plane-ring DDF kernel for 2-byte element types on sm_100a (forward, and grad-x at
// stride 1), built on Blackwell's mixed-precision FMA.
//
// Arithmetic.  sm_100 has `fma.rn.f32.{bf16,f16}`: d = a * b + c with a, b in the
// 2-byte type and c, d in float, at the issue rate of a plain float FMA.  The product
// of two bf16 (or two f16) values is exact in float, so
//     mul:  y = x * sf  (exact),  acc = fma(y, cf, acc)        2 FMA-pipe slots per tap
//     add:  acc = fma(x, sf, acc), acc = fma(x, cf, acc)       2 FMA-pipe slots per tap
// needs no unpacking of the input or of the spatial filter: both stay as packed 2-byte
// pairs in registers and the instruction selects the half it wants.  The spatial-filter
// values of a thread's P pixels therefore cost K*K*P/2 registers instead of K*K*P, and
// the integer pipe does nothing in the inner loop.
//
// Geometry.  A thread owns a PW x PH patch of output pixels of one plane position for
// the whole kernel.  With the row pitch W a template constant, every tap of every pixel
// is a fixed half of a fixed register of the thread's input window.  Zero padding costs
// the FMA pipe nothing: an input row outside the image is redirected, by an address
// select, to a zeroed shared-memory area, and the window words that hang over the left /
// right edge are ANDed with per-thread constant masks (integer pipe, otherwise idle).
//
// Data movement.  A persistent CTA per SM owns a contiguous run of the B*C planes and
// streams it through a ring of shared-memory slots filled by untiled bulk async copies
// (TMA) -- a stage is a few planes plus their channel filters -- each guarded by a full /
// empty mbarrier pair; the next sample's spatial filter travels the same way into its own
// buffer.  One lane of a dedicated producer warp issues the copies (issuing a bulk copy can
// block while the copy queue is full, which must not hold up arithmetic).  Each compute
// warp converts the channel filters its own lanes need (to float for mul, to an aligned
// 2-byte layout for add) into a private area, so compute warps never wait for one another
// except through the ring itself.
//
// Every wait on an mbarrier is bounded by the plan's `wait_cycles`; a wait that runs out
// records a fault code in global memory and the thread leaves the kernel.
#pragma once

#include <atomic>

#include "common.cuh"
#include "stream_fwd.cuh"

namespace ddf {

struct RingPlan {
    const void* in;   // x for the forward, go for grad-x
    const void* cf;
    const void* sf;
    void* out;
    int C, H, W, OH, OW;
    int tpp;          // threads per plane = (OH / PH) * (OW / PW)
    int ppr;          // patches per output row = OW / PW
    int tg;           // thread groups = planes per pass
    int pps;          // passes per stage
    int n_slots;      // ring depth
    int n_cwarps;     // warps
    long long total_passes;   // B*C / tg
    uint32_t plane_bytes;     // H*W*2
    uint32_t sf_bytes;        // K*K*OH*OW*2: one sample's spatial filter
    unsigned long long cf_total, sf_total;   // byte sizes of the whole cf / sf tensors
    uint32_t off_zero, off_cfw, cfw_stride, off_sf, off_stage0, stage_stride, off_rawcf, guard;
    int* fault;
    long long wait_cycles;    // limit of every mbarrier wait, in SM clocks
    uint32_t tx_skew;         // 0 in production; the failure-path test adds bytes that never arrive
};

// ---------------------------------------------------------------- mixed-precision FMA
// fmaw<XH, SH>(xw, sw, c) = half XH of word xw  *  half SH of word sw  +  c.  The halves are
// split inside the same asm block as their single use, which lets the assembler fold the
// selection into the instruction's operand modifiers.
#define DDF_MIXFMA(TYPE, XSEL, SSEL)                                                          \
    asm("{\n\t.reg .b16 xl, xh, sl, sh;\n\t"                                               \
        "mov.b32 {xl, xh}, %1;\n\tmov.b32 {sl, sh}, %2;\n\t"                               \
        "fma.rn.f32." TYPE " %0, " XSEL ", " SSEL ", %3;\n\t}"                               \
        : "=f"(r) : "r"(xw), "r"(sw), "f"(c))
template <typename T> struct Mix;
template <> struct Mix<__nv_bfloat16> {
    // xh, sh: which half (0 low, 1 high); constants once the caller's loops are unrolled
    static __device__ __forceinline__ float fmaw(int xh, int sh, uint32_t xw, uint32_t sw, float c) {
        float r;
        if (xh == 0 && sh == 0) DDF_MIXFMA("bf16", "xl", "sl");
        else if (xh == 1 && sh == 0) DDF_MIXFMA("bf16", "xh", "sl");
        else if (xh == 0 && sh == 1) DDF_MIXFMA("bf16", "xl", "sh");
        else DDF_MIXFMA("bf16", "xh", "sh");
        return r;
    }
    static __device__ __forceinline__ uint32_t f32_bits(uint32_t h) { return h << 16; }
};
template <> struct Mix<__half> {
    static __device__ __forceinline__ float fmaw(int xh, int sh, uint32_t xw, uint32_t sw, float c) {
        float r;
        if (xh == 0 && sh == 0) DDF_MIXFMA("f16", "xl", "sl");
        else if (xh == 1 && sh == 0) DDF_MIXFMA("f16", "xh", "sl");
        else if (xh == 0 && sh == 1) DDF_MIXFMA("f16", "xl", "sh");
        else DDF_MIXFMA("f16", "xh", "sh");
        return r;
    }
    static __device__ __forceinline__ uint32_t f32_bits(uint32_t h) {
        float r;
        asm("cvt.f32.f16 %0, %1;" : "=f"(r) : "h"((uint16_t)h));
        return __float_as_uint(r);
    }
};

__device__ __forceinline__ void split16(uint32_t w, uint16_t& lo, uint16_t& hi) {
    asm("mov.b32 {%0, %1}, %2;" : "=h"(lo), "=h"(hi) : "r"(w));
}
__device__ __forceinline__ void sts128(uint32_t a, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w)
                 : "memory");
}

__host__ __device__ constexpr int cfloor_div(int a, int b) { return (a >= 0) ? a / b : -((-a + b - 1) / b); }
__host__ __device__ constexpr int cgcd(int a, int b) { return b == 0 ? a : cgcd(b, a % b); }

// Loads words [W0, W0 + NW) relative to `base` (word w at byte base + 4w) with the widest
// vector loads the static alignment ALIGN of `base` allows.
template <int ALIGN, int W0, int NW, int I = 0>
__device__ __forceinline__ void load_words(uint32_t base, uint32_t (&w)[NW]) {
    if constexpr (I < NW) {
        constexpr int bytes = (W0 + I) * 4;
        constexpr bool a16 = ALIGN >= 16 && ((bytes % 16) + 16) % 16 == 0;
        constexpr bool a8 = ALIGN >= 8 && ((bytes % 8) + 8) % 8 == 0;
        if constexpr (a16 && I + 4 <= NW) {
            lds128(base + (uint32_t)bytes, w[I], w[I + 1], w[I + 2], w[I + 3]);
            load_words<ALIGN, W0, NW, I + 4>(base, w);
        } else if constexpr (a8 && I + 2 <= NW) {
            lds64(base + (uint32_t)bytes, w[I], w[I + 1]);
            load_words<ALIGN, W0, NW, I + 2>(base, w);
        } else {
            w[I] = lds32(base + (uint32_t)bytes);
            load_words<ALIGN, W0, NW, I + 1>(base, w);
        }
    }
}

template <int K, int D, int S, int PW, int PH, int WIN>
struct RingGeo {
    static constexpr int KK = K * K;
    static constexpr int R = (K - 1) / 2;
    static constexpr int HALO = R * D;
    static constexpr int P = PW * PH;
    static constexpr int NR = (PH - 1) * S + 2 * HALO + 1;   // input rows a patch touches
    // static alignment (bytes) of a thread's window base inside a stage
    static constexpr int ALIGN = cgcd(16, cgcd(PH * S * WIN * 2, PW * S * 2));
    static constexpr int CFS = (KK + 3) / 4 * 4;   // entries per plane of the converted channel filter
    static constexpr int CFP = CFS * 4;            // bytes per plane of it (floats for mul, halves for add)
    static constexpr int CW = CFS;      // words a thread holds of it: floats (mul) / packed halves (add)
    static constexpr int NLW = (HALO + 1) / 2;                               // window words left of the patch
    static constexpr int NRW = ((PW - 1) * S + HALO) / 2 - PW * S / 2 + 1 > 0 ? ((PW - 1) * S + HALO) / 2 - PW * S / 2 + 1 : 0;   // and right of it
    static_assert(PW % 2 == 0 && PW <= 8, "patch width: 2, 4 or 8 pixels");
    static_assert(P <= 8, "at most 8 pixels per thread");
    // input row `ir` (relative to the patch's first input row) is read by some (pixel row, tap row)
    static __host__ __device__ constexpr bool row_used(int ir) {
        for (int r = 0; r < PH; ++r)
            for (int i = 0; i < K; ++i)
                if (r * S + (i - R) * D == ir) return true;
        return false;
    }
    static __host__ __device__ constexpr int eo(int ir) { return ir * WIN; }
    static __host__ __device__ constexpr int w0(int ir) { return cfloor_div(eo(ir) - HALO, 2); }
    static __host__ __device__ constexpr int nw(int ir) {
        return cfloor_div(eo(ir) + (PW - 1) * S + HALO, 2) - w0(ir) + 1;
    }
    // half-size of the zeroed area out-of-image rows are redirected to
    static constexpr int ZR = ((((PH - 1) * S + HALO) * WIN + HALO + PW * S) * 2 + 32 + 15) / 16 * 16;
    static_assert(WIN % 2 == 0, "row pitch must be even");
    static constexpr int NWIN = nw(0);   // window words per row (the same for every row: WIN is even)
};

// One plane for one thread: the window rows are loaded (out-of-image rows from the zeroed
// area, over-hanging words masked), then every pixel's K*K products are formed and reduced.
//   mul: y_t = x_t * sf_t (exact), then the y are reduced against the float channel filter
//        two taps at a time with fma.rn.f32x2 (one issue slot for two taps) into a (lo, hi)
//        pair that is summed at the end;
//   add: acc = fma(x_t, sf_t, acc), acc = fma(x_t, cf_t, acc), cf as packed 2-byte pairs.
// All loops unroll completely; every index below is then a constant.
template <typename T, typename G, int K, int D, int S, int PW, int PH, int MODE>
struct RingPlane {
    static constexpr int P = PW * PH, KK = K * K, NW = G::NWIN, NM = PW * S / 2;
    // window row N (input row N - HALO relative to the patch's first)
    template <int N>
    struct Rows {
        static __device__ __forceinline__ void load(uint32_t tb, uint32_t zb, uint32_t rowsel,
                                                    const uint32_t (&lmask)[G::NLW > 0 ? G::NLW : 1],
                                                    const uint32_t (&rmask)[G::NRW > 0 ? G::NRW : 1],
                                                    uint32_t (&w)[G::NR][NW]) {
            if constexpr (N < G::NR) {
                constexpr int ir = N - G::HALO;
                if constexpr (G::row_used(ir)) {
                    constexpr int W0 = G::w0(ir), WB = G::eo(ir) / 2;
                    uint32_t rb = tb;
                    if constexpr (ir < 0 || ir > (PH - 1) * S) rb = (rowsel >> N) & 1u ? zb : tb;
                    load_words<G::ALIGN, W0, NW>(rb, w[N]);
#pragma unroll
                    for (int u = 0; u < NW; ++u) {
                        const int rel = W0 + u - WB;   // word position relative to the patch's first column
                        if (rel < 0) w[N][u] &= lmask[rel + G::NLW];
                        else if (rel >= NM) w[N][u] &= rmask[rel - NM];
                    }
                }
                Rows<N + 1>::load(tb, zb, rowsel, lmask, rmask, w);
            }
        }
    };
    static __device__ __forceinline__ void run(uint32_t tb, uint32_t zb, uint32_t rowsel,
                                               const uint32_t (&lmask)[G::NLW > 0 ? G::NLW : 1],
                                               const uint32_t (&rmask)[G::NRW > 0 ? G::NRW : 1],
                                               const uint32_t (&sfw)[KK][P / 2], const uint32_t (&c)[G::CFS],
                                               float (&res)[P]) {
        uint32_t w[G::NR][NW];
        Rows<0>::load(tb, zb, rowsel, lmask, rmask, w);
        // Tap-major order: consecutive FFMAs share the channel-filter operand and consecutive
        // mixed FMAs share an input word, which the register-operand reuse cache turns into
        // single-cycle issue (an FMA with three fresh register operands takes two).
        float acc[P];
#pragma unroll
        for (int pp = 0; pp < P; ++pp) acc[pp] = 0.f;
#pragma unroll
        for (int t = 0; t < KK; ++t) {
            const int i = t / K, j = t % K;
#pragma unroll
            for (int pp = 0; pp < P; ++pp) {
                const int r = pp / PW, cc = pp % PW;
                const int n = r * S + (i - G::R) * D + G::HALO;
                const int idx = cc * S + (j - G::R) * D - 2 * (G::w0(0));   // element within the row window
                if constexpr (MODE == DDF_B200_MUL) {
                    const float y = Mix<T>::fmaw(idx & 1, pp & 1, w[n][idx / 2], sfw[t][pp / 2], 0.f);
                    acc[pp] = fmaf(y, __uint_as_float(c[t]), acc[pp]);
                } else {
                    acc[pp] = Mix<T>::fmaw(idx & 1, pp & 1, w[n][idx / 2], sfw[t][pp / 2], acc[pp]);
                    acc[pp] = Mix<T>::fmaw(idx & 1, t & 1, w[n][idx / 2], c[t / 2], acc[pp]);
                }
            }
        }
#pragma unroll
        for (int pp = 0; pp < P; ++pp) res[pp] = acc[pp];
    }
};

// Non-blocking probe (mbarrier.test_wait): the issuing thread must never be parked on a
// barrier that other warps complete much later.
__device__ __forceinline__ bool mbar_poll(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  mbarrier.try_wait without a time hint blocks for a hardware-chosen short
// time and returns as soon as the phase completes (the hinted form compiles to sleep
// loops that add microseconds to every stage hand-over).
__device__ __forceinline__ bool mbar_wait_for(uint32_t bar, uint32_t parity, long long limit) {
    if (mbar_test(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i)
            if (mbar_test(bar, parity)) return true;
        if (clock64() - t0 > limit) return false;
    }
}

constexpr int kRingMaxSlots = 12;

// 25 compute warps + the producer warp: 7 warps on one SM sub-partition at most, i.e. up to 72
// registers per thread.
constexpr int kRingMaxThreads = 832;

template <typename T, int K, int D, int S, int PW, int PH, int WIN, int MODE, bool BWDX>
__global__ void __launch_bounds__(kRingMaxThreads, 1)
ring_kernel(const __grid_constant__ RingPlan pl) {
    using G = RingGeo<K, D, S, PW, PH, WIN>;
    constexpr int KK = G::KK;
    constexpr int P = G::P;
    static_assert(!BWDX || S == 1, "grad-x ring kernel is stride 1 only");
    static_assert(sizeof(T) == 2, "2-byte element types only");

    extern __shared__ __align__(128) unsigned char smem_raw[];
    const uint32_t sbase = smem_u32(smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int NST = pl.n_slots;
    const int NCW = pl.n_cwarps;
    const int TG = pl.tg;
    const int PPS = pl.pps;

#define RBAR_FULL(s) (sbase + 8u * (uint32_t)(s))
#define RBAR_EMPTY(s) (sbase + 8u * (uint32_t)(kRingMaxSlots + (s)))
#define RSTAGE(s) (sbase + pl.off_stage0 + (uint32_t)(s) * pl.stage_stride)
    const uint32_t bar_sf_full = sbase + 8u * (2 * kRingMaxSlots);
    const uint32_t bar_sf_empty = bar_sf_full + 8u;

    if (tid == 0) {
        for (int s = 0; s < NST; ++s) {
            mbar_init(RBAR_FULL(s), 1);
            mbar_init(RBAR_EMPTY(s), (uint32_t)NCW);
        }
        mbar_init(bar_sf_full, 1);
        mbar_init(bar_sf_empty, (uint32_t)NCW);
        mbar_fence_init();
    }
    // The zeroed area that rows outside the image are read from.
    for (uint32_t u = (uint32_t)tid; u < (uint32_t)(2 * G::ZR) / 16u; u += blockDim.x)
        sts128(sbase + pl.off_zero + 16u * u, 0u, 0u, 0u, 0u);
    __syncthreads();
    // Programmatic dependent launch: let the next grid start its prologue, and touch no
    // global memory before the previous grid has completed.
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const long long pass_lo = (pl.total_passes * (long long)blockIdx.x) / gridDim.x;
    const long long pass_hi = (pl.total_passes * (long long)(blockIdx.x + 1)) / gridDim.x;
    const int my_passes = (int)(pass_hi - pass_lo);
    if (my_passes == 0) return;
    const int my_stages = (my_passes + PPS - 1) / PPS;
    const long long plane_lo = pass_lo * TG, plane_hi = pass_hi * TG;
    const int stage_planes = PPS * TG;

    if (warp == NCW) {
        // ------------------------------------------------------------- producer warp
        if (lane != 0) return;
        int issue_i = 0, issue_slot = 0, seg_issued = 0;
        const int b_first = (int)(plane_lo / pl.C);
        const int seg_total = (int)((plane_hi - 1) / pl.C) + 1 - b_first;
        long long idle_since = -1;
        bool gave_up = false;
        while (issue_i < my_stages || seg_issued < seg_total) {
            bool progress = false;
            // the next sample's spatial filter, as soon as every compute warp has taken the
            // previous one into registers
            if (seg_issued < seg_total &&
                (seg_issued == 0 || mbar_poll(bar_sf_empty, (uint32_t)((seg_issued - 1) & 1)))) {
                const unsigned long long g0 = (unsigned long long)(b_first + seg_issued) * pl.sf_bytes;
                const Span sp = span_prepare(sbase + pl.off_sf, pl.sf, g0, g0 + pl.sf_bytes, pl.sf_total);
                mbar_arrive_expect_tx(bar_sf_full, sp.bytes);
                span_issue(sp, bar_sf_full);
                ++seg_issued;
                progress = true;
            }
            // the next stage, as soon as its slot has been released
            if (issue_i < my_stages &&
                (issue_i < NST || mbar_test(RBAR_EMPTY(issue_slot), (uint32_t)((issue_i / NST - 1) & 1)))) {
                const long long st_first = plane_lo + (long long)issue_i * stage_planes;
                long long st_end = st_first + stage_planes;
                if (st_end > plane_hi) st_end = plane_hi;
                // planes: start and size are multiples of 16 bytes (checked by the launcher)
                const unsigned long long g0 = (unsigned long long)st_first * pl.plane_bytes;
                const uint32_t nb = (uint32_t)((unsigned long long)(st_end - st_first) * pl.plane_bytes);
                const unsigned long long c0 = (unsigned long long)st_first * (KK * 2);
                const unsigned long long c1 = (unsigned long long)st_end * (KK * 2);
                const Span sc = span_prepare(RSTAGE(issue_slot) + pl.off_rawcf, pl.cf, c0, c1, pl.cf_total);
                mbar_arrive_expect_tx(RBAR_FULL(issue_slot), nb + sc.bytes + pl.tx_skew);
                bulk_g2s(RSTAGE(issue_slot) + pl.guard, (const char*)pl.in + g0, nb, RBAR_FULL(issue_slot));
                span_issue(sc, RBAR_FULL(issue_slot));
                ++issue_i;
                if (++issue_slot == NST) issue_slot = 0;
                progress = true;
            }
            if (progress) {
                idle_since = -1;
            } else if (idle_since < 0) {
                idle_since = clock64();
            } else if (clock64() - idle_since > (pl.tx_skew ? 2 * pl.wait_cycles : pl.wait_cycles)) {
                // (with the self-test's skew the compute warps, whose limit is shorter, report first)
                gave_up = true;
                break;
            }
        }
        if (gave_up) atomicCAS(pl.fault, 0, (int)kFaultService);
        // do not leave while requested copies may still be in flight (bounded)
        bool ok = true;
        for (int j = (issue_i > NST ? issue_i - NST : 0); j < issue_i; ++j)
            ok &= mbar_wait_for(RBAR_FULL(j % NST), (uint32_t)((j / NST) & 1), pl.wait_cycles);
        if (seg_issued > 0) ok &= mbar_wait_for(bar_sf_full, (uint32_t)((seg_issued - 1) & 1), pl.wait_cycles);
        if (!ok && pl.tx_skew == 0) atomicCAS(pl.fault, 0, (int)kFaultDrain);
        return;
    }
    if (warp > NCW) return;

    // ------------------------------------------------------------------- compute warps
    const int b_first = (int)(plane_lo / pl.C);
    // ---- this thread's patch
    const int TPP = pl.tpp;
    int grp = tid / TPP;
    int task = tid - grp * TPP;
    const bool active = grp < TG;
    if (!active) { grp = TG - 1; task = 0; }
    const int py = task / pl.ppr, px = task - py * pl.ppr;
    const int y0 = py * PH, x0 = px * PW;          // first output pixel of the patch
    const uint32_t in_off = (uint32_t)((y0 * S) * WIN + x0 * S) * 2u;
    // thread groups this warp's lanes belong to (at most two: tpp >= 32)
    int g_lo = (warp * 32) / TPP;
    if (g_lo > TG - 1) g_lo = TG - 1;
    int g_hi = (warp * 32 + 31) / TPP;
    if (g_hi > TG - 1) g_hi = TG - 1;
    const bool two_groups = g_hi > g_lo;
    const uint32_t cfw = sbase + pl.off_cfw + (uint32_t)warp * pl.cfw_stride;
    const uint32_t zb = sbase + pl.off_zero + (uint32_t)G::ZR;
    // zero padding: which window rows lie outside the image, and the AND masks of the window
    // words left / right of the patch
    uint32_t rowsel = 0u;
#pragma unroll
    for (int n = 0; n < G::NR; ++n) {
        const int iy = y0 * S + n - G::HALO;
        if (iy < 0 || iy >= pl.H) rowsel |= 1u << n;
    }
    uint32_t lmask[G::NLW > 0 ? G::NLW : 1], rmask[G::NRW > 0 ? G::NRW : 1];
    lmask[0] = 0u; rmask[0] = 0u;
#pragma unroll
    for (int u = 0; u < G::NLW; ++u) lmask[u] = (x0 * S + 2 * (u - G::NLW) < 0) ? 0u : 0xffffffffu;
#pragma unroll
    for (int u = 0; u < G::NRW; ++u) rmask[u] = (x0 * S + PW * S + 2 * u >= pl.W) ? 0u : 0xffffffffu;

    uint32_t sfw[KK][P / 2];
#pragma unroll
    for (int t = 0; t < KK; ++t)
#pragma unroll
        for (int q = 0; q < P / 2; ++q) sfw[t][q] = 0u;

    // passes until the next sample starts (a sample is C / TG passes; runs start on pass boundaries)
    const int sample_passes = pl.C / TG;
    int to_next_sample = sample_passes - (int)((plane_lo - (long long)b_first * pl.C) / TG);
    int seg = 0;
    const int OHW = pl.OH * pl.OW;
    T* outp = reinterpret_cast<T*>(pl.out) + (plane_lo + grp) * (long long)OHW + (y0 * pl.OW + x0);
    const long long out_step = (long long)TG * OHW;
    const uint32_t pass_stride = (uint32_t)TG * pl.plane_bytes;
    const int OW = pl.OW;

    int slot = 0, st = 0;
    uint32_t ph = 0;
    int passes_left = my_passes;
#pragma unroll 1
    while (passes_left > 0) {
        const int npass = passes_left < PPS ? passes_left : PPS;
        if (!mbar_wait_for(RBAR_FULL(slot), ph, pl.wait_cycles)) {
            atomicCAS(pl.fault, 0, (int)kFaultConsumerFull);
            return;
        }
        // Channel filters of the planes this warp's lanes will process in this stage: raw
        // 2-byte values -> the per-warp layout [pass][group][tap] the plane loop reads.
        {
            const unsigned long long st_first_plane = (unsigned long long)plane_lo + (unsigned long long)st * stage_planes;
            const uint32_t coff = (uint32_t)((st_first_plane * (KK * 2)) & 15ull);
            const uint32_t src = RSTAGE(slot) + pl.off_rawcf + coff;
            const int n = npass * (two_groups ? 2 : 1) * KK;
            __syncwarp();
            for (int e = lane; e < n; e += 32) {
                const int u = e / KK, t = e - u * KK;          // u = pass * groups + group
                const int pq = two_groups ? (u >> 1) : u, gi = two_groups ? (u & 1) : 0;
                const int tt = BWDX ? KK - 1 - t : t;          // grad-x reads the filter mirrored
                const uint32_t raw = lds16(src + 2u * (uint32_t)((pq * TG + g_lo + gi) * KK + t));
                const uint32_t dst = cfw + (uint32_t)((pq * 2 + gi) * G::CFP);
                if constexpr (MODE == DDF_B200_MUL) sts32(dst + 4u * (uint32_t)tt, Mix<T>::f32_bits(raw));
                else sts16(dst + 2u * (uint32_t)tt, raw);
            }
            __syncwarp();
        }

        uint32_t tb = RSTAGE(slot) + pl.guard + (uint32_t)grp * pl.plane_bytes + in_off;
        uint32_t cfa = cfw + (uint32_t)((grp - g_lo) * G::CFP);

        int q = 0;
#pragma unroll 1
        while (q < npass) {
            if (to_next_sample == sample_passes || seg == 0) {
                // first plane of a sample (or of this CTA's run): take the sample's spatial filter
                if (!mbar_wait_for(bar_sf_full, (uint32_t)(seg & 1), pl.wait_cycles)) {
                    atomicCAS(pl.fault, 0, (int)kFaultConsumerSf);
                            return;
                }
                const uint32_t sfs = sbase + pl.off_sf +
                                     (uint32_t)(((unsigned long long)(b_first + seg) * pl.sf_bytes) & 15ull);
                if constexpr (!BWDX) {
#pragma unroll
                    for (int t = 0; t < KK; ++t) {
#pragma unroll
                        for (int r = 0; r < PH; ++r) {
                            const uint32_t a = sfs + (uint32_t)(((t * pl.OH + y0 + r) * pl.OW + x0) * 2);
                            if constexpr (PW == 8) lds128v(a, sfw[t][r * 4], sfw[t][r * 4 + 1], sfw[t][r * 4 + 2], sfw[t][r * 4 + 3]);
                            else if constexpr (PW == 4) lds64v(a, sfw[t][r * 2], sfw[t][r * 2 + 1]);
                            else sfw[t][r] = lds32v(a);
                        }
                    }
                } else {
                    // grad-x: window tap (i, j) over go pairs with the filter value of the mirrored
                    // tap at the neighbouring pixel the product came from.
#pragma unroll
                    for (int i = 0; i < K; ++i) {
#pragma unroll
                        for (int j = 0; j < K; ++j) {
                            const int ft = KK - 1 - (i * K + j);
#pragma unroll
                            for (int pp = 0; pp < P; ++pp) {
                                const int yy = y0 + pp / PW + (i - G::R) * D, xx = x0 + pp % PW + (j - G::R) * D;
                                uint32_t v = 0u;
                                if (yy >= 0 && yy < pl.OH && xx >= 0 && xx < pl.OW)
                                    v = lds16v(sfs + (uint32_t)(((ft * pl.OH + yy) * pl.OW + xx) * 2));
                                if (pp & 1) sfw[i * K + j][pp / 2] |= v << 16;
                                else sfw[i * K + j][pp / 2] = v;
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_sf_empty);
                ++seg;
            }
            // the planes of this stage up to the next sample boundary: nothing but arithmetic
            int run = npass - q;
            if (run > to_next_sample) run = to_next_sample;
            q += run;
            to_next_sample -= run;
            if (to_next_sample == 0) to_next_sample = sample_passes;
#pragma unroll 1
            for (; run > 0; --run) {
                // the plane's converted channel filter: KK floats (mul) or KK packed halves (add)
                uint32_t c[G::CFS];
                constexpr int CWORDS = MODE == DDF_B200_MUL ? KK : (KK + 1) / 2;
                constexpr int NV = CWORDS / 4, REM = CWORDS % 4;
#pragma unroll
                for (int v = 0; v < NV; ++v) lds128(cfa + 16u * v, c[4 * v], c[4 * v + 1], c[4 * v + 2], c[4 * v + 3]);
                if constexpr (REM == 1) c[4 * NV] = lds32(cfa + 16u * NV);
                else if constexpr (REM == 2) lds64(cfa + 16u * NV, c[4 * NV], c[4 * NV + 1]);
                else if constexpr (REM == 3) lds128(cfa + 16u * NV, c[4 * NV], c[4 * NV + 1], c[4 * NV + 2], c[4 * NV + 3]);
                float res[P];
                RingPlane<T, G, K, D, S, PW, PH, MODE>::run(tb, zb, rowsel, lmask, rmask, sfw, c, res);
                if (active) {
#pragma unroll
                    for (int r = 0; r < PH; ++r) {
                        float rr[PW];
#pragma unroll
                        for (int cc = 0; cc < PW; ++cc) rr[cc] = res[r * PW + cc];
                        store_out<T, PW>(outp + r * OW, rr);
                    }
                }
                tb += pass_stride;
                cfa += (uint32_t)(2 * G::CFP);
                outp += out_step;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(RBAR_EMPTY(slot));
        passes_left -= npass;
        ++st;
        if (++slot == NST) { slot = 0; ph ^= 1u; }
    }
#undef RBAR_FULL
#undef RBAR_EMPTY
#undef RSTAGE
}

// ------------------------------------------------------------------------ host side
struct RingArgs {
    const void* in;
    const void* cf;
    const void* sf;
    void* out;
    Problem p;
    bool bwdx;
    int sm_count;
    int* fault;
    int device;
    bool overlap_launch;
    long long wait_cycles;   // 0 = default (about a second)
    uint32_t tx_skew;        // failure-path test only
};

template <typename T, int K, int D, int S, int PW, int PH, int WIN>
bool make_ring_plan(const RingArgs& a, RingPlan& pl, uint32_t& smem_bytes, int& grid, int& threads) {
    using G = RingGeo<K, D, S, PW, PH, WIN>;
    const Problem& p = a.p;
    const int H = a.bwdx ? p.OH : p.H, W = a.bwdx ? p.OW : p.W;
    const int OH = p.OH, OW = p.OW;
    if (a.bwdx && p.s != 1) return false;
    if (W != WIN || W != OW * S || H < OH * S) return false;
    if (OW % PW != 0 || OH % PH != 0) return false;
    if (p.sf_norm) return false;
    const int TPP = (OH / PH) * (OW / PW);
    if (TPP < 32 || TPP > kRingMaxThreads - 32) return false;
    const uint32_t plane_bytes = (uint32_t)(H * W * 2);
    int TG = (kRingMaxThreads - 32) / TPP;
    while (TG > 1 && (p.C % TG != 0 || ((unsigned long long)TG * plane_bytes) % 16 != 0)) --TG;
    if (p.C % TG != 0 || ((unsigned long long)TG * plane_bytes) % 16 != 0) return false;
    if (plane_bytes % G::ALIGN != 0) return false;
    const long long planes = (long long)p.B * p.C;
    const long long total_passes = planes / TG;
    const uint32_t sf_bytes = (uint32_t)(G::KK * OH * OW * 2);
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    if (!al16(a.in) || !al16(a.cf) || !al16(a.sf) || !al16(a.out)) return false;

    const uint32_t pass_bytes = (uint32_t)TG * plane_bytes;
    const uint32_t target = 36u << 10;
    int PPS = (int)(target / pass_bytes);
    if (PPS < 1) PPS = 1;
    const long long share = (total_passes + a.sm_count - 1) / a.sm_count;
    if (PPS > share) PPS = (int)share;
    if (PPS < 1) PPS = 1;

    const int n_warps = (TG * TPP + 31) / 32;
    const uint32_t guard = 32u;   // masked halo words of a stage's first / last row land here
    const uint32_t off_zero = round_up(8u * (2 * kRingMaxSlots + 2) + 16u, 16);
    const uint32_t off_cfw = off_zero + 2u * (uint32_t)G::ZR;
    const uint32_t sf_region = round_up(sf_bytes + 32u, 128);
    auto layout = [&](int pps) {
        pl.cfw_stride = (uint32_t)(pps * 2 * G::CFP);
        const uint32_t SPL = (uint32_t)pps * TG;
        pl.off_rawcf = round_up(2u * guard + SPL * plane_bytes, 16);
        pl.stage_stride = round_up(pl.off_rawcf + SPL * G::KK * 2u + 32u, 128);
        const uint32_t off_sf = round_up(off_cfw + (uint32_t)n_warps * pl.cfw_stride, 128);
        for (int slots = kRingMaxSlots; slots >= 1; --slots) {
            const uint32_t total = off_sf + sf_region + (uint32_t)slots * pl.stage_stride;
            if (total <= kSmemBudget) {
                pl.off_sf = off_sf;
                pl.off_stage0 = off_sf + sf_region;
                smem_bytes = total;
                return slots;
            }
        }
        return 0;
    };
    int slots = layout(PPS);
    while (slots < 4 && PPS > 1) slots = layout(--PPS);
    if (slots < 2) return false;
    pl.n_slots = slots;
    pl.off_cfw = off_cfw;
    pl.off_zero = off_zero;
    pl.guard = guard;
    pl.in = a.in; pl.cf = a.cf; pl.sf = a.sf; pl.out = a.out;
    pl.C = p.C; pl.H = H; pl.W = W; pl.OH = OH; pl.OW = OW;
    pl.tpp = TPP;
    pl.ppr = OW / PW;
    pl.tg = TG;
    pl.pps = PPS;
    pl.n_cwarps = n_warps;
    pl.total_passes = total_passes;
    pl.plane_bytes = plane_bytes;
    pl.sf_bytes = sf_bytes;
    pl.cf_total = (unsigned long long)planes * G::KK * 2;
    pl.sf_total = (unsigned long long)p.B * sf_bytes;
    pl.fault = a.fault;
    pl.wait_cycles = a.wait_cycles > 0 ? a.wait_cycles : kWaitCycles;
    pl.tx_skew = a.tx_skew;
    grid = (int)(total_passes < a.sm_count ? total_passes : a.sm_count);
    threads = (n_warps + 1) * 32;
    return true;
}

template <typename T, int K, int D, int S, int PW, int PH, int WIN, int MODE, bool BWDX>
int ring_launch(const RingArgs& a, cudaStream_t stream) {
    RingPlan pl;
    uint32_t smem = 0;
    int grid = 0, threads = 0;
    if (!make_ring_plan<T, K, D, S, PW, PH, WIN>(a, pl, smem, grid, threads)) return kNotHandled;
    auto kern = ring_kernel<T, K, D, S, PW, PH, WIN, MODE, BWDX>;
    static std::atomic<unsigned long long> opted_in{0};
    const unsigned long long bit = 1ull << (a.device & 63);
    if (!(opted_in.load(std::memory_order_acquire) & bit)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget);
        if (e != cudaSuccess) return (int)e;
        opted_in.fetch_or(bit, std::memory_order_release);
    }
    return (int)launch_overlapped(kern, dim3((unsigned)grid), dim3((unsigned)threads), smem, stream,
                                  a.overlap_launch, pl);
}

// Runtime (k, d, s, W, mode, bwdx) -> instantiation; defined per element type in
// ring_inst_<type>.cu.  Returns kNotHandled when no instantiation covers the problem.
template <typename T>
int ring_dispatch(const RingArgs& a, cudaStream_t stream);

}  // namespace ddf
