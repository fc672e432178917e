// Row kernel: DDF forward (and grad-x at stride 1) for square planes of the ddf_resnet stages,
// k = 3, dilation 1: outputs 7, 14, 28 or 56 pixels wide at stride 1 and, for the 2-byte element
// types, 7, 14 or 28 wide at stride 2.  Written for the 2-byte types (the text below); float
// elements run the same structure with one element per word, 7-pixel segments and plain float
// multiply / FMA, where that measured faster than the plane-streaming kernel.
//
// The op costs 18 FMA-pipe operations per output, which at 2-byte I/O is as much time as the
// HBM traffic; what decides a launch is the number of *other* instructions per output and the
// time until the first arithmetic starts.  Hence:
//
//  * A thread owns one output row, or a 14-pixel (stride 1) / 7-pixel (stride 2) segment of a
//    row, at a fixed position for the whole kernel, and does one plane of every chunk of
//    planes: the 9 x 14 (or 9 x 7) spatial-filter values of its pixels stay in registers,
//    packed two to a word, across all planes of a sample.  With that many pixels per thread
//    the window loads, the channel-filter loads, the stores and the loop cost about 10
//    instructions per output next to the 18 FMAs (the 4-pixel patches of the plane-ring
//    kernel: 20).
//  * Whole rows (7 or 14 wide) know their left and right zero padding at compile time: those
//    taps are simply not emitted (57 instead of 63 taps at 7 pixels), and no halo masks
//    exist.  Segments AND the first word of a row's first window and the last word of its
//    last window with per-thread constant masks.  Rows above and below the plane are
//    redirected by one address select to a zeroed area.  Zero padding is exact in both modes.
//  * Rows of 7 two-byte elements start on odd element offsets in every other row.  Such a row
//    is read as four aligned words and brought into a fixed register layout by funnel shifts
//    whose shift amount (0 or 16) is a per-thread constant; the arithmetic then selects
//    fixed halves of fixed registers (mixed-precision FMA, see ring_fwd.cuh).  Rows of 14
//    or more elements are word aligned and need no shifts.  Outputs of 7 pixels leave as
//    three word stores and one 2-byte store; a warp's stores cover a contiguous run.
//  * Persistent CTA per SM; chunks of planes (plus their channel filters) arrive through a
//    ring of shared-memory slots filled by untiled TMA bulk copies from one producer lane; a
//    conversion warp turns each landed chunk's channel filters into the per-plane vector
//    layout and announces them on a third mbarrier per slot; 14 compute warps of 32 threads
//    (448 = 64 x 7 = 32 x 14 = 8 x 56 = 2 x 224 threads cover whole planes at every width).
//    The spatial filters of two consecutive samples are double-buffered.
//
// Every mbarrier wait is bounded by the plan's wait_cycles (fault word + return, as in the
// other streaming kernels).
#pragma once

#include <atomic>

#include "common.cuh"
#include "ring_fwd.cuh"

namespace ddf {

struct RowPlan {
    const void* in;
    const void* cf;
    const void* sf;
    void* out;
    int chunks_per_sample;    // C / planes per chunk
    int n_slots;
    long long total_chunks;   // B * C / planes per chunk
    int chunks_q, chunks_r;   // total_chunks = grid * q + r: CTA i takes q (+1 if i < r) chunks
    uint32_t chunk_bytes;     // one chunk of input planes
    uint32_t sf_bytes;        // 9 * OW * OW * 2
    unsigned long long sf_total, cf_total;
    uint32_t off_zero, off_sf, sf_stride, off_stage0, stage_stride, off_rawcf, off_conv;
    int* fault;
    long long wait_cycles;
};

constexpr int kRowCompute = 448;              // compute threads: one per (plane, output row) of a chunk
constexpr int kRowThreads = kRowCompute + 64; // + producer warp + conversion warp
constexpr int kRowMaxSlots = 16;
constexpr int kRowCFP = 48;                   // bytes per plane of the converted channel filter

__device__ __forceinline__ void stg32(void* p, uint32_t v) {
    asm volatile("st.global.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void stg16(void* p, uint32_t v) {
    asm volatile("st.global.b16 [%0], %1;" ::"l"(p), "h"((uint16_t)v) : "memory");
}

// NSEG = 1: a thread owns a whole output row (OW = 7 or 14).  NSEG > 1: a row is cut into NSEG
// segments of 14 pixels (stride 1) or 7 pixels (stride 2), one per thread; a thread's input
// window then starts two elements left of its segment's first input element (a word
// boundary) and, at stride 1, ends two elements right of the last one.  The window's first
// word of a row's first segment and last word of its last segment are ANDed with per-thread
// constant masks (true zero padding, as in the plane-ring kernel).
// TPC: tasks (planes) a thread does per chunk; 2 halves the per-chunk barrier traffic where a
// CTA's share is many chunks.
// BWDX: grad-x at stride 1 -- the same kernel over go with the channel filter's taps mirrored
// and, for window tap (i, j), the spatial filter of the mirrored tap at the neighbouring
// pixel the product came from.
template <typename T, int S, int OW, int NSEG, int TPC, int MODE, bool BWDX>
__global__ void __launch_bounds__(kRowThreads, 1)
row_kernel(const __grid_constant__ RowPlan pl) {
    constexpr int K = 3, KK = 9;
    constexpr int SEG = OW / NSEG;                  // output pixels per thread
    constexpr int TPP = OW * NSEG;                  // threads per plane
    constexpr int CHT = kRowCompute / TPP;          // planes the compute threads cover at once
    constexpr int CH = CHT * TPC;                   // planes per chunk
    constexpr int W = OW * S;                       // input row length in elements
    constexpr int ES = (int)sizeof(T);
    constexpr bool F32 = ES == 4;                   // float: one element per word, plain FMUL / FFMA
    constexpr int PLANE = W * W * ES;               // input plane bytes
    constexpr bool XSHIFT = !F32 && W % 2 != 0;     // input rows start on odd elements: funnel shifts
    constexpr bool OSHIFT = !F32 && SEG % 2 != 0;   // the same for a thread's output and spatial-filter run
    // words of an input row a thread holds (2-byte: a segment's window starts two elements left
    // of it, float: one element left)
    constexpr int NW = F32 ? (NSEG > 1 ? SEG + 2 : W)
                           : (NSEG > 1 ? (S == 1 ? SEG / 2 + 2 : SEG + 1) : (W + 1) / 2);
    constexpr int NSW = F32 ? SEG : (SEG + 1) / 2;  // words of a thread's spatial-filter / output run
    // buffers for the samples' spatial filters: two (the next sample's filter arrives while this one is
    // in use), except for 56 x 56 float planes, where one sample's filter is 113 KB
    constexpr int NSFB = (F32 && OW == 56) ? 1 : 2;
    static_assert(S == 1 || S == 2, "stride 1 or 2");
    static_assert(F32 ? (S == 1 && SEG == 7)
                      : (NSEG == 1 ? (W == 7 || W == 14) : (S == 1 ? SEG == 14 : SEG == 7)), "row or segment geometry");
    static_assert(kRowCompute % TPP == 0, "whole planes per chunk");
    static_assert(!BWDX || S == 1, "grad-x at stride 1 only");
    static_assert(ES == 2 || ES == 4, "2- and 4-byte element types");

    extern __shared__ __align__(128) unsigned char smem_raw[];
    const uint32_t sbase = smem_u32(smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int NST = pl.n_slots;
    constexpr int NCW = kRowCompute / 32;           // 14 compute warps

#define WBAR_FULL(s) (sbase + 8u * (uint32_t)(s))
#define WBAR_EMPTY(s) (sbase + 8u * (uint32_t)(kRowMaxSlots + (s)))
#define WBAR_CF(s) (sbase + 8u * (uint32_t)(2 * kRowMaxSlots + (s)))
#define WBAR_SF_FULL(i) (sbase + 8u * (uint32_t)(3 * kRowMaxSlots + (i)))
#define WBAR_SF_EMPTY(i) (sbase + 8u * (uint32_t)(3 * kRowMaxSlots + 2 + (i)))
#define WSTAGE(s) (sbase + pl.off_stage0 + (uint32_t)(s) * pl.stage_stride)

    if (tid == 0) {
        for (int s = 0; s < NST; ++s) {
            mbar_init(WBAR_FULL(s), 1);
            mbar_init(WBAR_EMPTY(s), (uint32_t)NCW);
            mbar_init(WBAR_CF(s), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(WBAR_SF_FULL(i), 1);
            mbar_init(WBAR_SF_EMPTY(i), (uint32_t)NCW);
        }
        mbar_fence_init();
    }
    if (tid < 4) sts128(sbase + pl.off_zero + 16u * (uint32_t)tid, 0u, 0u, 0u, 0u);
    __syncthreads();
    // Programmatic dependent launch: this grid may have started while the previous one was still
    // running.  Everything that does not touch global memory (index arithmetic, register set-up)
    // comes before griddepcontrol.wait, which every role executes just before its main loop.
    asm volatile("griddepcontrol.launch_dependents;");

    const int bid = (int)blockIdx.x;
    const long long chunk_lo = (long long)bid * pl.chunks_q + (bid < pl.chunks_r ? bid : pl.chunks_r);
    const int my_chunks = pl.chunks_q + (bid < pl.chunks_r ? 1 : 0);
    if (my_chunks == 0) return;
    const int CPS = pl.chunks_per_sample;

    if (warp == NCW) {
        // ------------------------------------------------------------- producer lane
        if (lane != 0) return;
        bool ok = true;
        int seg = 0, issued = 0;
        int b = (int)chunk_lo / CPS;               // (the launcher keeps the chunk count below 2^31)
        int left_in_sample = 0;                    // chunks of sample b still to issue (0: start a sample)
        int first_left = CPS - (int)(chunk_lo - (long long)b * CPS);
        int slot = 0, round = 0;                   // chunk i uses slot i % NST in round i / NST
        asm volatile("griddepcontrol.wait;" ::: "memory");
        for (int i = 0; i < my_chunks && ok; ++i) {
            const long long g = chunk_lo + i;
            if (left_in_sample == 0) {
                // this sample's spatial filter, into the buffer the sample before the previous one used
                const int buf = NSFB == 2 ? (seg & 1) : 0;
                const int use = NSFB == 2 ? (seg >> 1) : seg;   // how often the buffer was used before
                if (use >= 1) ok = mbar_wait_for(WBAR_SF_EMPTY(buf), (uint32_t)((use - 1) & 1), pl.wait_cycles);
                if (!ok) break;
                const unsigned long long g0 = (unsigned long long)b * pl.sf_bytes;
                const Span sp = span_prepare(sbase + pl.off_sf + (uint32_t)buf * pl.sf_stride, pl.sf, g0,
                                             g0 + pl.sf_bytes, pl.sf_total);
                mbar_arrive_expect_tx(WBAR_SF_FULL(buf), sp.bytes);
                span_issue(sp, WBAR_SF_FULL(buf));
                ++seg;
                left_in_sample = i == 0 ? first_left : CPS;
            }
            if (--left_in_sample == 0) ++b;
            if (round > 0) ok = mbar_wait_for(WBAR_EMPTY(slot), (uint32_t)((round - 1) & 1), pl.wait_cycles);
            if (!ok) break;
            // the chunk's planes (a multiple of 16 bytes from a 16-byte aligned start) and their
            // channel filters (any byte range: aligned superset, clamped to the tensor's end)
            constexpr unsigned long long cfb = (unsigned long long)(CH * KK * ES);
            const Span sc = span_prepare(WSTAGE(slot) + pl.off_rawcf, pl.cf, (unsigned long long)g * cfb,
                                         (unsigned long long)(g + 1) * cfb, pl.cf_total);
            mbar_arrive_expect_tx(WBAR_FULL(slot), pl.chunk_bytes + sc.bytes);
            bulk_g2s(WSTAGE(slot) + 16u, (const char*)pl.in + (unsigned long long)g * pl.chunk_bytes, pl.chunk_bytes,
                     WBAR_FULL(slot));
            span_issue(sc, WBAR_FULL(slot));
            issued = i + 1;
            if (++slot == NST) { slot = 0; ++round; }
        }
        if (!ok) atomicCAS(pl.fault, 0, (int)kFaultService);
        // do not leave while requested copies may still be in flight (bounded)
        bool landed = true;
        for (int j = (issued > NST ? issued - NST : 0); j < issued; ++j)
            landed &= mbar_wait_for(WBAR_FULL(j % NST), (uint32_t)((j / NST) & 1), pl.wait_cycles);
        for (int s2 = (seg > NSFB ? seg - NSFB : 0); s2 < seg; ++s2)
            landed &= mbar_wait_for(WBAR_SF_FULL(NSFB == 2 ? (s2 & 1) : 0),
                                    (uint32_t)((NSFB == 2 ? (s2 >> 1) : s2) & 1), pl.wait_cycles);
        if (!landed) atomicCAS(pl.fault, 0, (int)kFaultDrain);
        return;
    }
    if (warp == NCW + 1) {
        // ------------------------------------------------- channel-filter conversion warp
        // raw 2-byte filters of a landed chunk -> per plane: KK floats (mul) or KK aligned
        // 2-byte values (add) every kRowCFP bytes
        int slot = 0;
        uint32_t ph = 0u;
        asm volatile("griddepcontrol.wait;" ::: "memory");
        for (int i = 0; i < my_chunks; ++i) {
            if (!mbar_wait_for(WBAR_FULL(slot), ph, pl.wait_cycles)) {
                atomicCAS(pl.fault, 0, (int)kFaultConsumerFull);
                return;
            }
            const uint32_t src = WSTAGE(slot) + pl.off_rawcf +
                                 (uint32_t)(((unsigned long long)(chunk_lo + i) * (CH * KK * ES)) & 15ull);
            const uint32_t dst = WSTAGE(slot) + pl.off_conv;
#pragma unroll 3
            for (int e = lane; e < CH * KK; e += 32) {
                const int u = e / KK, t = e - u * KK;
                const int tt = BWDX ? KK - 1 - t : t;
                if constexpr (F32) {
                    sts32(dst + (uint32_t)(u * kRowCFP + 4 * tt), lds32(src + 4u * (uint32_t)e));
                } else {
                    const uint32_t raw = lds16(src + 2u * (uint32_t)e);
                    if constexpr (MODE == DDF_B200_MUL) sts32(dst + (uint32_t)(u * kRowCFP + 4 * tt), Mix<T>::f32_bits(raw));
                    else sts16(dst + (uint32_t)(u * kRowCFP + 2 * tt), raw);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(WBAR_CF(slot));
            if (++slot == NST) { slot = 0; ph ^= 1u; }
        }
        return;
    }

    // ------------------------------------------------------------------- compute warps
    // plane within the chunk, output row, segment of the row
    const int j = tid / TPP, y = (tid - TPP * j) / NSEG, g = tid - TPP * j - NSEG * y;
    // Input rows of this thread relative to the chunk's first plane: byte offset of the aligned
    // word its window starts at, funnel shift that brings the window's element 0 to the low half
    // of word 0, and whether the row lies outside the plane.
    uint32_t rowoff[K], rowsh[K];
    bool rowout[K];
#pragma unroll
    for (int r = 0; r < K; ++r) {
        const int iy = y * S - 1 + r;
        rowout[r] = iy < 0 || iy >= W;
        // (wraps for iy < 0: unused then)
        // (a segment's window starts 4 bytes left of its first input element)
        const uint32_t a = 16u + (uint32_t)(j * PLANE + iy * W * ES + (NSEG > 1 ? g * SEG * S * ES - 4 : 0));
        rowoff[r] = XSHIFT ? (a & ~3u) : a;
        rowsh[r] = XSHIFT ? (a & 2u) * 8u : 0u;
    }
    // masks of the window's first / last word (segments only)
    uint32_t lmask = (NSEG > 1 && g == 0) ? 0u : 0xffffffffu;
    uint32_t rmask = (NSEG > 1 && S == 1 && g == NSEG - 1) ? 0u : 0xffffffffu;
    if constexpr (NSEG > 1) {
        asm volatile("" : "+r"(lmask));
        asm volatile("" : "+r"(rmask));
    }
    const uint32_t zaddr = sbase + pl.off_zero + (S == 2 ? 4u : 0u);   // same alignment class as the rows it replaces
    const uint32_t cfoff = pl.off_conv + (uint32_t)(j * kRowCFP);
    // output: SEG elements at element offset plane * OW * OW + OW * y + SEG * g; for odd SEG its word
    // parity is a thread constant (a chunk starts on an even element)
    const uint32_t opar = OSHIFT ? (uint32_t)((j * OW * OW + y * OW + g * SEG) & 1) : 0u;
    const uint32_t osh = opar * 16u;
    char* outp = reinterpret_cast<char*>(pl.out) +
                 ((unsigned long long)chunk_lo * CH + (unsigned long long)j) * (OW * OW * ES) +
                 (unsigned long long)((y * OW + g * SEG) * ES);

    uint32_t sfw[KK][NSW];
#pragma unroll
    for (int t = 0; t < KK; ++t)
#pragma unroll
        for (int q = 0; q < NSW; ++q) sfw[t][q] = 0u;

    int seg = 0, slot = 0;
    uint32_t ph = 0u;
    int b = (int)chunk_lo / CPS;
    int left_in_sample = 0;   // chunks of the current sample still to come (0: the next chunk starts a sample)
    const int first_left = CPS - (int)(chunk_lo - (long long)b * CPS);
    asm volatile("griddepcontrol.wait;" ::: "memory");   // (before the first store to global memory)
#pragma unroll 1
    for (int i = 0; i < my_chunks; ++i) {
        if (left_in_sample == 0) {
            // a new sample: its spatial filter (requested before the chunk, hence taken first; at the
            // start of a launch the registers fill while the first chunk is still in flight), 9 taps
            // x SEG pixels as (p0,p1) (p2,p3) ... per tap
            const int buf = NSFB == 2 ? (seg & 1) : 0;
            if (!mbar_wait_for(WBAR_SF_FULL(buf), (uint32_t)((NSFB == 2 ? (seg >> 1) : seg) & 1), pl.wait_cycles)) {
                atomicCAS(pl.fault, 0, (int)kFaultConsumerSf);
                return;
            }
            const uint32_t sfs = sbase + pl.off_sf + (uint32_t)buf * pl.sf_stride +
                                 (uint32_t)(((unsigned long long)b * pl.sf_bytes) & 15ull) +
                                 (uint32_t)((y * OW + g * SEG) * ES);
#pragma unroll
            for (int t = 0; t < KK; ++t) {
                if constexpr (!BWDX) {
                    const uint32_t a = sfs + (uint32_t)(t * OW * OW * ES);
                    if constexpr (OSHIFT) {
                        const uint32_t aw = a & ~3u, sh = (a & 2u) * 8u;
                        const uint32_t w0 = lds32v(aw), w1 = lds32v(aw + 4), w2 = lds32v(aw + 8), w3 = lds32v(aw + 12);
                        sfw[t][0] = __funnelshift_r(w0, w1, sh);
                        sfw[t][1] = __funnelshift_r(w1, w2, sh);
                        sfw[t][2] = __funnelshift_r(w2, w3, sh);
                        sfw[t][3] = w3 >> sh;
                    } else {
#pragma unroll
                        for (int q = 0; q < NSW; ++q) sfw[t][q] = lds32v(a + 4u * q);
                    }
                } else {
                    // window tap (ti, tj): filter plane KK-1-t, row y + ti - 1, elements
                    // g*SEG + tj - 1 + p (p = 0..SEG-1); what lies outside the plane is zero
                    const int ti = t / K, tj = t % K;
                    const int yy = y + ti - 1;
                    const uint32_t a = sfs + (uint32_t)(((KK - 1 - t) * OW * OW + (ti - 1) * OW + (tj - 1)) * ES);
                    if constexpr (F32) {
#pragma unroll
                        for (int q = 0; q < NSW; ++q) sfw[t][q] = lds32v(a + 4u * q);
                        if (tj == 0 && g == 0) sfw[t][0] = 0u;                     // column -1
                        if (tj == 2 && g == NSEG - 1) sfw[t][NSW - 1] = 0u;        // column OW
                    } else {
                        const uint32_t aw = a & ~3u, sh = (a & 2u) * 8u;
                        uint32_t wv[NSW + 1];
#pragma unroll
                        for (int q = 0; q <= NSW; ++q) wv[q] = lds32v(aw + 4u * q);
#pragma unroll
                        for (int q = 0; q < NSW; ++q) sfw[t][q] = __funnelshift_r(wv[q], wv[q + 1], sh);
                        if (SEG % 2 != 0) sfw[t][NSW - 1] &= 0x0000ffffu;          // the half past the run
                        if (tj == 0 && g == 0) sfw[t][0] &= 0xffff0000u;           // column -1
                        if (tj == 2 && g == NSEG - 1)                              // column OW
                            sfw[t][NSW - 1] &= (SEG % 2 != 0) ? 0u : 0x0000ffffu;
                    }
                    if (yy < 0 || yy >= OW) {
#pragma unroll
                        for (int q = 0; q < NSW; ++q) sfw[t][q] = 0u;
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(WBAR_SF_EMPTY(buf));
            ++seg;
            left_in_sample = i == 0 ? first_left : CPS;
        }
        // the chunk has landed (full) and its channel filters are converted (cf)
        if (!mbar_wait_for(WBAR_CF(slot), ph, pl.wait_cycles) ||
            !mbar_wait_for(WBAR_FULL(slot), ph, pl.wait_cycles)) {
            atomicCAS(pl.fault, 0, (int)kFaultConsumerFull);
            return;
        }
        if (--left_in_sample == 0) ++b;

#pragma unroll 1
        for (int u = 0; u < TPC; ++u) {
            // task u of the chunk: plane u * CHT + j
            const uint32_t st = WSTAGE(slot) + (uint32_t)(u * CHT * PLANE);
            const uint32_t ca0 = WSTAGE(slot) + cfoff + (uint32_t)(u * CHT * kRowCFP);
            char* op = outp + u * (CHT * OW * OW * ES);
            // ---- the plane's input rows
            uint32_t xw[K][NW];
#pragma unroll
            for (int r = 0; r < K; ++r) {
                const uint32_t a = rowout[r] ? zaddr : st + rowoff[r];
                if constexpr (XSHIFT) {
                    const uint32_t w0 = lds32(a), w1 = lds32(a + 4), w2 = lds32(a + 8), w3 = lds32(a + 12);
                    xw[r][0] = __funnelshift_r(w0, w1, rowsh[r]);
                    xw[r][1] = __funnelshift_r(w1, w2, rowsh[r]);
                    xw[r][2] = __funnelshift_r(w2, w3, rowsh[r]);
                    xw[r][3] = w3 >> rowsh[r];
                } else if constexpr (S == 2 && NSEG == 1) {
                    // 14 elements = 7 aligned words; input row 2y (r = 1) is 8-byte aligned, its
                    // neighbours are not
                    if (r == 1) {
                        lds64(a, xw[r][0], xw[r][1]);
                        lds64(a + 8, xw[r][2], xw[r][3]);
                        lds64(a + 16, xw[r][4], xw[r][5]);
                        xw[r][6] = lds32(a + 24);
                    } else {
                        xw[r][0] = lds32(a);
                        lds64(a + 4, xw[r][1], xw[r][2]);
                        lds64(a + 12, xw[r][3], xw[r][4]);
                        lds64(a + 20, xw[r][5], xw[r][6]);
                    }
                } else {
#pragma unroll
                    for (int q = 0; q < NW; ++q) xw[r][q] = lds32(a + 4u * q);
                    if constexpr (NSEG > 1) {
                        xw[r][0] &= lmask;
                        if constexpr (S == 1) xw[r][NW - 1] &= rmask;
                    }
                }
            }
            // ---- the plane's channel filter
            uint32_t c[12];
            {
                const uint32_t ca = ca0;
                if constexpr (MODE == DDF_B200_MUL || F32) {
                    lds128(ca, c[0], c[1], c[2], c[3]);
                    lds128(ca + 16, c[4], c[5], c[6], c[7]);
                    c[8] = lds32(ca + 32);
                } else {
                    lds128(ca, c[0], c[1], c[2], c[3]);
                    c[4] = lds32(ca + 16);
                }
            }
            // ---- the taps (those that fall left or right of the plane are not emitted), tap-major
            float acc[SEG];
#pragma unroll
            for (int p = 0; p < SEG; ++p) acc[p] = 0.f;
#pragma unroll
            for (int t = 0; t < KK; ++t) {
                const int ti = t / K, tj = t % K;
                // element of the thread's window for pixel p: whole rows start at the row's element 0
                // and drop the taps outside it; segments start two elements left of the segment
                // Pixels are taken HB at a time: whole rows (NSEG = 1) measured faster seven at a time
                // (14 x 14, mul: 13.0 -> 9.8 us), segments all fourteen at once (56 x 56, mul: 34.7 against 37.4 us).
                constexpr int HB = (NSEG == 1 && SEG > 7) ? 7 : SEG;
                if constexpr (F32) {
                    // float: window element p + tj (a segment's window starts one element left of it).
                    // mul: the filter product sf * cf first, then one FMA per pixel; add: two FMAs per pixel.
                    // Pixels in pairs through the packed f32x2 instructions (one issue slot for two
                    // FMAs), a last odd pixel and pairs with a dropped tap in scalar form.
                    const float cv = __uint_as_float(c[t]);
                    const unsigned long long cc = f2_pack(cv, cv);
#pragma unroll
                    for (int p = 0; p < SEG; p += 2) {
                        const int e0 = NSEG > 1 ? p + tj : p + tj - 1;
                        const int e1 = e0 + 1;
                        const bool v0 = NSEG > 1 || (e0 >= 0 && e0 < W);
                        const bool v1 = p + 1 < SEG && (NSEG > 1 || (e1 >= 0 && e1 < W));
                        if (v0 && v1) {
                            const unsigned long long xp = f2_pack(__uint_as_float(xw[ti][e0]), __uint_as_float(xw[ti][e1]));
                            const unsigned long long sp = f2_pack(__uint_as_float(sfw[t][p]), __uint_as_float(sfw[t][p + 1]));
                            unsigned long long ap = f2_pack(acc[p], acc[p + 1]);
                            if constexpr (MODE == DDF_B200_MUL) {
                                ap = f2_fma(xp, f2_mul(sp, cc), ap);
                            } else {
                                ap = f2_fma(xp, sp, ap);
                                ap = f2_fma(xp, cc, ap);
                            }
                            f2_unpack(ap, acc[p], acc[p + 1]);
                        } else {
                            if (v0) {
                                const float xv = __uint_as_float(xw[ti][e0]), sv = __uint_as_float(sfw[t][p]);
                                if constexpr (MODE == DDF_B200_MUL) acc[p] = fmaf(xv, sv * cv, acc[p]);
                                else acc[p] = fmaf(xv, cv, fmaf(xv, sv, acc[p]));
                            }
                            if (v1) {
                                const float xv = __uint_as_float(xw[ti][e1]), sv = __uint_as_float(sfw[t][p + 1]);
                                if constexpr (MODE == DDF_B200_MUL) acc[p + 1] = fmaf(xv, sv * cv, acc[p + 1]);
                                else acc[p + 1] = fmaf(xv, cv, fmaf(xv, sv, acc[p + 1]));
                            }
                        }
                    }
                } else
#pragma unroll
                for (int p0 = 0; p0 < SEG; p0 += HB) {
                    if constexpr (MODE == DDF_B200_MUL) {
                        // the exact products of the tap first, then the FMAs that share c[t]
                        float yv[HB];
#pragma unroll
                        for (int q = 0; q < HB; ++q) {
                            const int p = p0 + q;
                            const int e = NSEG > 1 ? p * S + tj + 1 : p * S + tj - 1;
                            if (NSEG == 1 && (e < 0 || e >= W)) continue;
                            yv[q] = Mix<T>::fmaw(e & 1, p & 1, xw[ti][e >> 1], sfw[t][p >> 1], 0.f);
                        }
                        // two pixels per instruction where both take part (fma.rn.f32x2 is the same
                        // IEEE fma per lane and half the issue slots: 56 x 56, 34.9 -> 28.9 us)
                        const unsigned long long cc = f2_pack(__uint_as_float(c[t]), __uint_as_float(c[t]));
#pragma unroll
                        for (int q = 0; q < HB; q += 2) {
                            const int p = p0 + q;
                            const int e0 = NSEG > 1 ? p * S + tj + 1 : p * S + tj - 1;
                            const int e1 = e0 + S;
                            const bool v0 = NSEG > 1 || (e0 >= 0 && e0 < W);
                            const bool v1 = q + 1 < HB && (NSEG > 1 || (e1 >= 0 && e1 < W));
                            if (v0 && v1) {
                                const unsigned long long r =
                                    f2_fma(f2_pack(yv[q], yv[q + 1]), cc, f2_pack(acc[p], acc[p + 1]));
                                f2_unpack(r, acc[p], acc[p + 1]);
                            } else {
                                if (v0) acc[p] = fmaf(yv[q], __uint_as_float(c[t]), acc[p]);
                                if (v1) acc[p + 1] = fmaf(yv[q + 1], __uint_as_float(c[t]), acc[p + 1]);
                            }
                        }
                    } else {
                        // x * sf for every pixel, then x * cf (consecutive FMAs are independent and the
                        // second group shares the channel-filter word)
#pragma unroll
                        for (int q = 0; q < HB; ++q) {
                            const int p = p0 + q;
                            const int e = NSEG > 1 ? p * S + tj + 1 : p * S + tj - 1;
                            if (NSEG == 1 && (e < 0 || e >= W)) continue;
                            acc[p] = Mix<T>::fmaw(e & 1, p & 1, xw[ti][e >> 1], sfw[t][p >> 1], acc[p]);
                        }
#pragma unroll
                        for (int q = 0; q < HB; ++q) {
                            const int p = p0 + q;
                            const int e = NSEG > 1 ? p * S + tj + 1 : p * S + tj - 1;
                            if (NSEG == 1 && (e < 0 || e >= W)) continue;
                            acc[p] = Mix<T>::fmaw(e & 1, t & 1, xw[ti][e >> 1], c[t >> 1], acc[p]);
                        }
                    }
                }
            }
            // ---- store the row
            if constexpr (F32) {
#pragma unroll
                for (int q = 0; q < SEG; ++q) stg32(op + 4 * q, __float_as_uint(acc[q]));
            } else if constexpr (OSHIFT) {
                // 7 results: three words and one half, arranged by the row's word parity
                const uint32_t w0 = Word<T>::put(acc[0], acc[1]), w1 = Word<T>::put(acc[2], acc[3]);
                const uint32_t w2 = Word<T>::put(acc[4], acc[5]), w3 = Word<T>::put(acc[6], 0.f);
                const uint32_t v0 = __funnelshift_r(w0, w1, osh), v1 = __funnelshift_r(w1, w2, osh);
                const uint32_t v2 = __funnelshift_r(w2, w3, osh);
                char* pw = op + 2u * opar;
                stg32(pw, v0);
                stg32(pw + 4, v1);
                stg32(pw + 8, v2);
                stg16(op + (opar ? 0 : 12), opar ? w0 : w3);
            } else {
#pragma unroll
                for (int q = 0; q < NSW; ++q) stg32(op + 4 * q, Word<T>::put(acc[2 * q], acc[2 * q + 1]));
            }
        }
        outp += CH * OW * OW * ES;
        __syncwarp();
        if (lane == 0) mbar_arrive(WBAR_EMPTY(slot));
        if (++slot == NST) { slot = 0; ph ^= 1u; }
    }
#undef WBAR_FULL
#undef WBAR_EMPTY
#undef WBAR_CF
#undef WBAR_SF_FULL
#undef WBAR_SF_EMPTY
#undef WSTAGE
}

// ------------------------------------------------------------------------ host side
struct RowArgs {
    const void* in;   // x for the forward, go for grad-x
    const void* cf;
    const void* sf;
    void* out;        // out for the forward, gx for grad-x
    Problem p;
    bool bwdx;
    int sm_count;
    int* fault;
    int device;
};

template <typename T, int S, int OW, int NSEG, int TPC, int MODE, bool BWDX>
int row_launch(const RowArgs& a, cudaStream_t stream) {
    const Problem& p = a.p;
    constexpr int W = OW * S;
    constexpr int ES = (int)sizeof(T);
    constexpr int kRowChunk = TPC * (kRowCompute / (OW * NSEG));
    RowPlan pl;
    pl.in = a.in; pl.cf = a.cf; pl.sf = a.sf; pl.out = a.out;
    pl.chunks_per_sample = p.C / kRowChunk;
    pl.total_chunks = (long long)p.B * pl.chunks_per_sample;
    if (pl.total_chunks > 0x7fffffffll) return kNotHandled;
    pl.chunk_bytes = (uint32_t)(kRowChunk * W * W * ES);
    pl.sf_bytes = (uint32_t)(9 * OW * OW * ES);
    pl.sf_total = (unsigned long long)p.B * pl.sf_bytes;
    pl.cf_total = (unsigned long long)p.B * p.C * (9ull * ES);
    pl.off_zero = round_up(8u * (3 * kRowMaxSlots + 4), 16);
    pl.off_sf = round_up(pl.off_zero + 64u, 128);
    pl.sf_stride = round_up(pl.sf_bytes + 48u, 128);
    // spatial-filter buffers: as the kernel's NSFB
    constexpr uint32_t kSfBufs = (ES == 4 && OW == 56) ? 1u : 2u;
    pl.off_stage0 = pl.off_sf + kSfBufs * pl.sf_stride;
    // [16 bytes: a first segment's window starts 4 bytes early][planes][16 bytes: a last row's or
    // last segment's window runs up to 14 bytes over][raw channel filters + alignment slack]
    pl.off_rawcf = round_up(16u + pl.chunk_bytes + 16u, 16);
    pl.off_conv = round_up(pl.off_rawcf + (uint32_t)(kRowChunk * 9 * ES) + 32u, 16);
    pl.stage_stride = round_up(pl.off_conv + (uint32_t)(kRowChunk * kRowCFP), 128);
    const long long share = (pl.total_chunks + a.sm_count - 1) / a.sm_count;
    if (pl.off_stage0 + pl.stage_stride > kSmemBudget) return kNotHandled;
    int slots = (int)((kSmemBudget - pl.off_stage0) / pl.stage_stride);
    if (slots > kRowMaxSlots) slots = kRowMaxSlots;
    if (slots > share) slots = (int)share;
    if (slots < 2) slots = share < 2 ? 1 : 2;
    if (pl.off_stage0 + (uint32_t)slots * pl.stage_stride > kSmemBudget) return kNotHandled;
    pl.n_slots = slots;
    pl.fault = a.fault;
    pl.wait_cycles = kWaitCycles;
    const uint32_t smem = pl.off_stage0 + (uint32_t)slots * pl.stage_stride;
    const int grid = (int)(pl.total_chunks < a.sm_count ? pl.total_chunks : a.sm_count);
    pl.chunks_q = (int)(pl.total_chunks / grid);
    pl.chunks_r = (int)(pl.total_chunks % grid);
    auto kern = row_kernel<T, S, OW, NSEG, TPC, MODE, BWDX>;
    static std::atomic<unsigned long long> opted_in{0};
    const unsigned long long bit = 1ull << (a.device & 63);
    if (!(opted_in.load(std::memory_order_acquire) & bit)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget);
        if (e != cudaSuccess) return (int)e;
        opted_in.fetch_or(bit, std::memory_order_release);
    }
    return (int)launch_overlapped(kern, dim3((unsigned)grid), dim3((unsigned)kRowThreads), smem, stream, true, pl);
}

// The problems the row kernel is built for: returns the number of planes its compute threads
// cover at once (a chunk is one or two of those; C must be a multiple of the chunk), 0 if the
// problem is not covered.
inline int row_planes_at_once(const RowArgs& a) {
    const Problem& p = a.p;
    if (p.dtype != DDF_B200_F16 && p.dtype != DDF_B200_BF16 && p.dtype != DDF_B200_F32) return 0;
    if (p.k != 3 || p.d != 1 || (p.s != 1 && p.s != 2) || p.sf_norm) return 0;
    if (a.bwdx && p.s != 1) return 0;
    if (p.OH != p.OW || p.H != p.OH * p.s || p.W != p.OW * p.s) return 0;
    int tpp;   // threads per plane
    if (p.dtype == DDF_B200_F32) {
        // float: 7-pixel segments, stride 1
        if (p.s != 1 || (p.OW != 7 && p.OW != 14 && p.OW != 28 && p.OW != 56)) return 0;
        // (measured against the plane-streaming kernel, B = 128, us at 56 / 28 / 14 / 7 pixels:
        // mul 41.8 / 21.1 / 15.5 / 10.6 and add 48.3 / 23.9 / 14.0 / 10.3 against 60.6 / 28.1 / 20.8 / 13.3)
        tpp = p.OW * (p.OW / 7);
    } else if (p.OW == 7) tpp = 7;
    else if (p.s == 1 && (p.OW == 14 || p.OW == 28 || p.OW == 56)) tpp = p.OW * (p.OW / 14);
    else if (p.s == 2 && (p.OW == 14 || p.OW == 28)) tpp = p.OW * (p.OW / 7);
    else return 0;
    const int cht = kRowCompute / tpp;
    if (p.C % cht != 0) return 0;
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    return (al16(a.in) && al16(a.cf) && al16(a.sf) && al16(a.out)) ? cht : 0;
}

// Defined per element type in row_inst_<type>.cu.
template <typename T>
int row_dispatch(const RowArgs& a, cudaStream_t stream);

}  // namespace ddf
