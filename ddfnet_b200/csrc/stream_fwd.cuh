// Plane-streaming DDF kernel for sm_100a (forward, and grad-x at stride 1).
//
// Work decomposition.  The (b, c) planes of the input are one contiguous run of
// B*C planes in memory.  The grid is persistent (one CTA per SM); CTA n owns an
// equal, contiguous share of that run and streams it through shared memory:
//
//   service warp   one elected lane issues untiled bulk async copies (TMA,
//                  cp.async.bulk) of the next stage -- a few whole planes plus
//                  their channel filters -- into a ring of shared-memory slots,
//                  each guarded by a full / empty mbarrier pair, and of the
//                  spatial filter of the next sample into its own buffer.  The
//                  same warp converts each landed stage's channel filters to
//                  float and then raises the stage's `ready` barrier.
//   compute warps  every thread owns P adjacent output pixels of one plane
//                  position for the whole kernel.  The k*k spatial-filter values
//                  of those pixels live in registers (they are the same for all
//                  channels of a sample) and are re-read only when the run
//                  crosses into the next sample.  Per plane a thread reads its
//                  k input rows from shared memory as vectors, forms
//                  w = cf (.) sf in float, accumulates in float and writes P
//                  results with one vector store.
//
// Zero padding costs nothing in the inner loop: rows outside the plane are
// redirected to a zeroed shared-memory row by an address select, and the halo
// words left / right of the plane are ANDed with a per-thread constant mask.
//
// Bulk copies must start on 16-byte boundaries.  Plane runs start anywhere, so
// every copy fetches the 16-byte-aligned superset of the bytes it needs and the
// readers add the remainder (< 16 bytes) to their shared-memory addresses.  A copy
// never reads past the tensor's last whole 16 bytes: what is left of a ragged end
// is fetched with plain loads.  The launcher declines (kNotHandled) only when a
// tensor's base address is not 16-byte aligned.
//
// Every wait on an mbarrier is bounded; a wait that runs out records a fault
// code in global memory and the thread leaves the kernel.
#pragma once

#include <atomic>
#include <cstdlib>

#include "common.cuh"

namespace ddf {

constexpr int kMaxSlots = 16;          // ring depth upper bound
constexpr int kMaxComputeThreads = 448;  // 14 warps; + 1 service warp = 480 threads
// 15 warps = 4 per SM sub-partition at most; each sub-partition has 16K registers,
// so a thread may use up to 128 (the launch bound below makes ptxas keep to that).
constexpr int kStreamThreads = kMaxComputeThreads + 32;
constexpr uint32_t kSmemBudget = 225 * 1024;

struct StreamPlan {
    const void* in;   // x for the forward, go for grad-x
    const void* cf;
    const void* sf;
    void* out;
    int C, H, W, OH, OW;
    int tasks_per_plane;   // OH*OW / P
    int groups_per_row;    // OW / P
    int planes_per_pass;   // NP: planes the compute threads cover at once (= thread_groups * PPT)
    int thread_groups;     // groups of tasks_per_plane threads; each thread does PPT planes per pass
    int passes_per_stage;  // PPS
    int n_slots;           // ring depth
    int n_compute_warps;
    long long total_passes;  // B*C / NP
    uint32_t plane_bytes;    // H*W*sizeof(T)
    uint32_t sf_bytes;       // k*k*OH*OW*sizeof(T): one sample's spatial filter
    unsigned long long in_total, cf_total, sf_total;   // byte sizes of the whole tensors
    uint32_t off_zero, off_cfc, cfc_stride, off_sf, off_stage0, stage_stride, off_rawcf;
    int* fault;
    float sf_scale;  // NORM kernels: output scale of the spatial FilterNorm (gain / k)
};

template <typename T, int K, int D, int S, int P>
struct Geo {
    static constexpr int KK = K * K;
    static constexpr int R = (K - 1) / 2;
    static constexpr int HALO = R * D;
    static constexpr int ES = (int)sizeof(T);
    static constexpr int EPW = 4 / ES;
    static constexpr int MAINN = P * S;          // elements read as the aligned main vector
    static constexpr int MAINB = MAINN * ES;
    // Element-wise path: every input element is fetched with its own shared load.  Used
    // where a thread's row segment is not a power-of-two vector: P = 1 with 2-byte
    // elements, and P = 7 (planes 7 or 14 wide: a thread then owns a whole or half row,
    // which spreads the per-plane overhead over 7 outputs instead of 1 or 2).
    static constexpr bool SUBWORD = MAINB < 4 || P == 7;
    static constexpr int MAINW = SUBWORD ? 1 : MAINB / 4;
    static constexpr bool PAIRS = (P >= 2) && (P % 2 == 0);  // pixels pair up for f32x2 math
    static constexpr int NCOL = (P - 1) * S + 2 * HALO + 1;  // input columns a thread touches
    static constexpr int NRE = ((P - 1) * S + HALO + 1 - MAINN) > 0 ? ((P - 1) * S + HALO + 1 - MAINN) : 0;
    static constexpr int NLW = (HALO + EPW - 1) / EPW;   // halo words left of the main vector
    static constexpr int NRW = (NRE + EPW - 1) / EPW;    // halo words right of it
    static constexpr int OUTB = P * ES;
    static_assert(K == 3 || K == 5, "streaming kernel is instantiated for k = 3, 5");
    static constexpr int NLM = NLW > 0 ? NLW : 1;        // sizes of the halo mask arrays
    static constexpr int NRM = NRW > 0 ? NRW : 1;
    static_assert(!SUBWORD || HALO <= 1, "the element-wise path covers a halo of one only");
    static_assert(ES == 2 || ES == 4, "2- and 4-byte element types only");
};

// VOL: volatile loads, for values that are kept in registers after their buffer has been
// handed back (see lds32v in common.cuh).
template <int NB, bool VOL = false>
__device__ __forceinline__ void lds_vec(uint32_t a, uint32_t (&w)[NB / 4]) {
    if constexpr (NB == 4) {
        w[0] = VOL ? lds32v(a) : lds32(a);
    } else if constexpr (NB == 8) {
        if constexpr (VOL) lds64v(a, w[0], w[1]);
        else lds64(a, w[0], w[1]);
    } else if constexpr (NB == 16) {
        if constexpr (VOL) lds128v(a, w[0], w[1], w[2], w[3]);
        else lds128(a, w[0], w[1], w[2], w[3]);
    } else {
        static_assert(NB == 32, "vector width");
        if constexpr (VOL) {
            lds128v(a, w[0], w[1], w[2], w[3]);
            lds128v(a + 16, w[4], w[5], w[6], w[7]);
        } else {
            lds128(a, w[0], w[1], w[2], w[3]);
            lds128(a + 16, w[4], w[5], w[6], w[7]);
        }
    }
}

// One input row of a thread's window, as floats.  rp = shared address of the
// first main element (input column ox0*S of that row).
template <typename T, bool VOL = false>
__device__ __forceinline__ uint32_t lds_elem_bits(uint32_t a) {
    if constexpr (sizeof(T) == 4) return VOL ? lds32v(a) : lds32(a);
    else return VOL ? lds16v(a) : lds16(a);
}

template <typename T, typename G>
__device__ __forceinline__ void load_row(uint32_t rp, const uint32_t (&lmask)[G::NLM],
                                         const uint32_t (&rmask)[G::NRM], float (&xr)[G::NCOL]) {
    if constexpr (G::SUBWORD) {
#pragma unroll
        for (int c = 0; c < G::NCOL; ++c) {
            const int e = c - G::HALO;  // element index relative to the segment's first column
            uint32_t w = lds_elem_bits<T>(rp + e * G::ES);
            if (e < 0) w &= lmask[0];
            if (e >= G::MAINN) w &= rmask[0];
            xr[c] = Word<T>::get(w, 0);
        }
    } else {
        uint32_t lw[G::NLW > 0 ? G::NLW : 1];
        uint32_t mw[G::MAINW];
        uint32_t rw[G::NRW > 0 ? G::NRW : 1];
#pragma unroll
        for (int a = 0; a < G::NLW; ++a) lw[a] = lds32(rp - 4 * (G::NLW - a)) & lmask[a];
        lds_vec<G::MAINB>(rp, mw);
#pragma unroll
        for (int a = 0; a < G::NRW; ++a) rw[a] = lds32(rp + G::MAINB + 4 * a) & rmask[a];
#pragma unroll
        for (int c = 0; c < G::NCOL; ++c) {
            const int e = c - G::HALO;
            if (e < 0) {
                const int idx = e + G::NLW * G::EPW;
                xr[c] = Word<T>::get(lw[idx / G::EPW], idx % G::EPW);
            } else if (e < G::MAINN) {
                xr[c] = Word<T>::get(mw[e / G::EPW], e % G::EPW);
            } else {
                const int idx = e - G::MAINN;
                xr[c] = Word<T>::get(rw[idx / G::EPW], idx % G::EPW);
            }
        }
    }
}

// Per-thread halo masks: all ones where the halo word lies inside the row, zero
// where it hangs over the left / right edge of the plane (those reads land on
// neighbouring data in shared memory and are cleared by the AND).  A word is
// never half inside: its first column is a multiple of the elements per word
// and the row width is even whenever a word holds two elements.
template <typename G>
__device__ __forceinline__ void halo_masks(int ox0, int S, int W, uint32_t (&lmask)[G::NLM],
                                           uint32_t (&rmask)[G::NRM]) {
    if constexpr (G::SUBWORD) {
        lmask[0] = ox0 > 0 ? 0xffffffffu : 0u;
        rmask[0] = (ox0 * S + G::MAINN) < W ? 0xffffffffu : 0u;
    } else {
        lmask[0] = 0u;
        rmask[0] = 0u;
#pragma unroll
        for (int a = 0; a < G::NLW; ++a)
            lmask[a] = (ox0 * S - (G::NLW - a) * G::EPW >= 0) ? 0xffffffffu : 0u;
#pragma unroll
        for (int a = 0; a < G::NRW; ++a)
            rmask[a] = (ox0 * S + G::MAINN + a * G::EPW + (G::EPW - 1) <= W - 1) ? 0xffffffffu : 0u;
    }
}

template <typename T, int P>
__device__ __forceinline__ void store_out(T* gp, const float (&acc)[P]) {
    constexpr int ES = (int)sizeof(T);
    if constexpr (P == 7) {
#pragma unroll
        for (int pp = 0; pp < 7; ++pp) Elem<T>::store(gp + pp, acc[pp]);
    } else if constexpr (ES == 4) {
        if constexpr (P == 1) {
            *reinterpret_cast<float*>(gp) = acc[0];
        } else if constexpr (P == 2) {
            *reinterpret_cast<float2*>(gp) = make_float2(acc[0], acc[1]);
        } else {
#pragma unroll
            for (int v = 0; v < P / 4; ++v)
                reinterpret_cast<float4*>(gp)[v] =
                    make_float4(acc[4 * v], acc[4 * v + 1], acc[4 * v + 2], acc[4 * v + 3]);
        }
    } else {
        if constexpr (P == 1) {
            Elem<T>::store(gp, acc[0]);
        } else if constexpr (P == 2) {
            *reinterpret_cast<uint32_t*>(gp) = Word<T>::put(acc[0], acc[1]);
        } else if constexpr (P == 4) {
            *reinterpret_cast<uint2*>(gp) =
                make_uint2(Word<T>::put(acc[0], acc[1]), Word<T>::put(acc[2], acc[3]));
        } else {
            static_assert(P == 8, "pixels per thread");
            *reinterpret_cast<uint4*>(gp) =
                make_uint4(Word<T>::put(acc[0], acc[1]), Word<T>::put(acc[2], acc[3]),
                           Word<T>::put(acc[4], acc[5]), Word<T>::put(acc[6], acc[7]));
        }
    }
}

// scale / (sqrt(v) + 1e-10) for v >= 0 without the library's out-of-line slow paths (a call
// inside the kernel would force spills around it): reciprocal square root refined by one
// Newton step, then a fast division; a few float ulps in all.
__device__ __forceinline__ float norm_gain(float v, float scale) {
    float r = rsqrtf(v);
    r = r * (1.5f - 0.5f * v * r * r);
    const float sd = v > 0.f ? v * r : 0.f;
    return __fdividef(scale, sd + 1e-10f);
}

__device__ __forceinline__ bool warp_test(uint32_t bar, uint32_t parity, int lane) {
    int ok = 0;
    if (lane == 0) ok = mbar_test(bar, parity) ? 1 : 0;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

// BWDX = false: out = DDF forward of `in` (= x).
// BWDX = true : out = grad-x computed from `in` (= go); stride must be 1.
// PACK        : accumulate with packed f32x2 FMAs (two pixels per instruction).
// PPT         : planes each thread processes per pass (1 or 2).  With 2 the two planes'
//               loads and arithmetic are independent and interleave, which hides the
//               shared-load and dependent-issue latencies that bound the kernel at 14
//               warps per SM; it needs registers, so it is used where P <= 4.
// NORM        : forward only: the values taken from `sf` are raw and the spatial FilterNorm
//               is applied to them in registers.
template <typename T, int K, int D, int S, int P, int MODE, bool BWDX, bool PACK, int PPT, bool NORM>
__global__ void __launch_bounds__(kStreamThreads, 1)
stream_kernel(const __grid_constant__ StreamPlan pl) {
    using G = Geo<T, K, D, S, P>;
    constexpr int KK = G::KK;
    constexpr int ES = G::ES;
    static_assert(!BWDX || S == 1, "grad-x streaming kernel is stride 1 only");

    extern __shared__ __align__(128) unsigned char smem_raw[];
    const uint32_t sbase = smem_u32(smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int NST = pl.n_slots;
    const int NCW = pl.n_compute_warps;
    const int NP = pl.planes_per_pass;
    const int PPS = pl.passes_per_stage;

    const uint32_t bar_sf_full = sbase + 8u * (3 * kMaxSlots);
    const uint32_t bar_sf_empty = bar_sf_full + 8u;
#define BAR_FULL(s) (sbase + 8u * (uint32_t)(s))
#define BAR_EMPTY(s) (sbase + 8u * (uint32_t)(kMaxSlots + (s)))
#define BAR_READY(s) (sbase + 8u * (uint32_t)(2 * kMaxSlots + (s)))
#define STAGE_BASE(s) (sbase + pl.off_stage0 + (uint32_t)(s) * pl.stage_stride)

    if (tid == 0) {
        for (int s = 0; s < NST; ++s) {
            mbar_init(BAR_FULL(s), 1);
            mbar_init(BAR_EMPTY(s), (uint32_t)NCW);
            mbar_init(BAR_READY(s), 1);
        }
        mbar_init(bar_sf_full, 1);
        mbar_init(bar_sf_empty, (uint32_t)NCW);
        mbar_fence_init();
    }
    if (tid < 64) sts32(sbase + pl.off_zero + 4u * tid, 0u);  // 256 zero bytes
    __syncthreads();
    // Programmatic dependent launch.  When the launch carries the attribute, this grid
    // may have started while the previous grid in the stream was still finishing: let
    // the next one do the same, and touch no global memory before the previous grid
    // has completed and its writes are visible.  Without the attribute both are no-ops.
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // This CTA's share of the passes (a pass = NP consecutive planes).
    const long long pass_lo = (pl.total_passes * (long long)blockIdx.x) / gridDim.x;
    const long long pass_hi = (pl.total_passes * (long long)(blockIdx.x + 1)) / gridDim.x;
    const int my_passes = (int)(pass_hi - pass_lo);
    if (my_passes == 0) return;
    const int my_stages = (my_passes + PPS - 1) / PPS;
    const long long plane_lo = pass_lo * NP, plane_hi = pass_hi * NP;
    const int stage_planes = PPS * NP;

    if (warp == NCW) {
        // ------------------------------------------------------------- service warp
        int issue_i = 0, conv_j = 0, seg_k = 0;
        long long seg_b = plane_lo / pl.C;
        long long seg_plane = plane_lo;  // first plane of the next sample segment
        long long idle_since = -1;
        bool gave_up = false;
        // Runs until every stage has been converted AND the spatial filter of every
        // sample that starts inside this CTA's run has been requested.
        while (conv_j < my_stages || seg_plane < plane_hi) {
            bool progress = false;
            // (1) Spatial filter of the next sample: requested once its first plane lies
            // within the stages issued so far or the one about to be issued, and the
            // buffer is free, i.e. every compute warp has copied the previous sample's
            // values into registers.
            {
                const int ahead = issue_i + 1 < my_stages ? issue_i + 1 : my_stages;
                long long horizon = plane_lo + (long long)ahead * stage_planes;
                if (horizon > plane_hi) horizon = plane_hi;
                if (seg_plane < horizon &&
                    (seg_k == 0 || warp_test(bar_sf_empty, (uint32_t)((seg_k - 1) & 1), lane))) {
                    if (lane == 0) {
                        const unsigned long long g0 = (unsigned long long)seg_b * pl.sf_bytes;
                        const Span sp = span_prepare(sbase + pl.off_sf, pl.sf, g0, g0 + pl.sf_bytes, pl.sf_total);
                        mbar_arrive_expect_tx(bar_sf_full, sp.bytes);
                        span_issue(sp, bar_sf_full);
                    }
                    ++seg_k;
                    ++seg_b;
                    seg_plane = seg_b * pl.C;
                    progress = true;
                }
            }
            // (2) Next stage, as soon as its slot has been released.
            if (issue_i < my_stages) {
                const int slot = issue_i % NST;
                const bool free_slot =
                    issue_i < NST ||
                    warp_test(BAR_EMPTY(slot), (uint32_t)((issue_i / NST - 1) & 1), lane);
                if (free_slot) {
                    const long long st_first = plane_lo + (long long)issue_i * stage_planes;
                    long long st_end = st_first + stage_planes;
                    if (st_end > plane_hi) st_end = plane_hi;
                    if (lane == 0) {
                        const unsigned long long g0 = (unsigned long long)st_first * pl.plane_bytes;
                        const unsigned long long g1 = (unsigned long long)st_end * pl.plane_bytes;
                        const unsigned long long c0 = (unsigned long long)st_first * (KK * ES);
                        const unsigned long long c1 = (unsigned long long)st_end * (KK * ES);
                        const Span sx = span_prepare(STAGE_BASE(slot) + 32u, pl.in, g0, g1, pl.in_total);
                        const Span sc = span_prepare(STAGE_BASE(slot) + pl.off_rawcf, pl.cf, c0, c1, pl.cf_total);
                        mbar_arrive_expect_tx(BAR_FULL(slot), sx.bytes + sc.bytes);
                        span_issue(sx, BAR_FULL(slot));
                        span_issue(sc, BAR_FULL(slot));
                    }
                    ++issue_i;
                    progress = true;
                }
            }
            if (conv_j < issue_i) {
                const int slot = conv_j % NST;
                if (warp_test(BAR_FULL(slot), (uint32_t)((conv_j / NST) & 1), lane)) {
                    // Channel filters of this stage: raw elements -> float.
                    const long long st_first = plane_lo + (long long)conv_j * stage_planes;
                    long long st_end = st_first + stage_planes;
                    if (st_end > plane_hi) st_end = plane_hi;
                    const int n = (int)(st_end - st_first) * KK;
                    const uint32_t coff = (uint32_t)(((unsigned long long)st_first * (KK * ES)) & 15ull);
                    const uint32_t src = STAGE_BASE(slot) + pl.off_rawcf + coff;
                    const uint32_t dst = sbase + pl.off_cfc + (uint32_t)slot * pl.cfc_stride;
                    // Four loads in flight per lane: the loop is latency-bound otherwise and
                    // the first stage's conversion sits on the kernel's start-up path.
                    for (int e0 = lane; e0 < n; e0 += 128) {
                        uint32_t raw[4];
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int e = e0 + 32 * u;
                            raw[u] = 0u;
                            if (e < n) raw[u] = ES == 4 ? lds32(src + 4u * e) : lds16(src + 2u * e);
                        }
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const int e = e0 + 32 * u;
                            const uint32_t v = __float_as_uint(Word<T>::get(raw[u], 0));
                            if (e < n) sts64(dst + 8u * e, v, v);  // (cf, cf): ready for the two-wide multiply
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(BAR_READY(slot));
                    ++conv_j;
                    progress = true;
                }
            }
            if (progress) {
                idle_since = -1;
            } else if (idle_since < 0) {
                idle_since = clock64();
            } else if (clock64() - idle_since > kWaitCycles) {
                gave_up = true;
                break;
            }
        }
        if (gave_up) {
            // Record the fault, then let every copy already issued land (bounded)
            // before this warp leaves.
            if (lane == 0) atomicCAS(pl.fault, 0, (int)kFaultService);
            bool drained = true;
            for (int j = conv_j; j < issue_i; ++j)
                drained &= mbar_wait(BAR_FULL(j % NST), (uint32_t)((j / NST) & 1));
            if (seg_k > 0) drained &= mbar_wait(bar_sf_full, (uint32_t)((seg_k - 1) & 1));
            if (!drained && lane == 0) atomicExch(pl.fault, (int)kFaultDrain);
        }
        return;
    }
    if (warp > NCW) return;

    // ----------------------------------------------------------------- compute warps
    const int TP = pl.tasks_per_plane;
    int pip = tid / TP;  // plane within the pass
    int task = tid - pip * TP;
    const int TG = pl.thread_groups;
    const bool active = pip < TG;
    if (!active) { pip = 0; task = 0; }
    const int oy = task / pl.groups_per_row;
    const int ox0 = (task - oy * pl.groups_per_row) * P;

    bool rowok[K];
    uint32_t rowoff[K];
#pragma unroll
    for (int i = 0; i < K; ++i) {
        const int iy = oy * S + (i - G::R) * D;
        rowok[i] = iy >= 0 && iy < pl.H;
        rowoff[i] = (uint32_t)((iy * pl.W + ox0 * S) * ES);
    }
    uint32_t lmask[G::NLM], rmask[G::NRM];
    halo_masks<G>(ox0, S, pl.W, lmask, rmask);
    const uint32_t zero_row = sbase + pl.off_zero + 64u;

    // Spatial-filter values of this thread's pixels.  With packed arithmetic they are
    // kept as (pixel q, pixel q + P/2) pairs, the operand layout of mul/fma.f32x2.
    // An odd P pairs up as well: the upper half of the last pair is a dummy pixel whose
    // result is dropped.
    constexpr bool PK = PACK && P >= 2;
    constexpr int PH = (P + 1) / 2;  // pairs per thread
    float sfr[PK ? 1 : KK][PK ? 1 : P];
    unsigned long long sf2[PK ? KK : 1][PK ? PH : 1];
    auto set_sf = [&](int t, int pp, float v) {
        if constexpr (PK) {
            float lo, hi;
            f2_unpack(sf2[t][pp % PH], lo, hi);
            if (pp < PH) lo = v; else hi = v;
            sf2[t][pp % PH] = f2_pack(lo, hi);
        } else {
            sfr[t][pp] = v;
        }
    };
#pragma unroll
    for (int t = 0; t < KK; ++t)
#pragma unroll
        for (int pp = 0; pp < P; ++pp) set_sf(t, pp, 0.f);

    long long b = plane_lo / pl.C;
    int c_in_b = (int)(plane_lo - b * pl.C);
    bool need_sf = true;
    int seg = 0;
    const long long out_plane = (long long)pl.OH * pl.OW;
    T* outp = reinterpret_cast<T*>(pl.out) + (plane_lo + pip) * out_plane + (long long)oy * pl.OW + ox0;
    const long long out_step = (long long)NP * out_plane;

    int slot = -1;
    uint32_t ph = 1;  // becomes slot 0, phase 0 on the first stage; no division per stage
    for (int st = 0; st < my_stages; ++st) {
        if (++slot == NST) slot = 0;
        if (slot == 0) ph ^= 1u;
        const int first_pass = st * PPS;
        const int npass = (my_passes - first_pass) < PPS ? (my_passes - first_pass) : PPS;
        const unsigned long long st_first_plane = (unsigned long long)plane_lo + (unsigned long long)first_pass * NP;
        const uint32_t xoff = (uint32_t)((st_first_plane * pl.plane_bytes) & 15ull);
        uint32_t plane_s = STAGE_BASE(slot) + 32u + xoff + (uint32_t)pip * pl.plane_bytes;
        uint32_t cfc_s = sbase + pl.off_cfc + (uint32_t)slot * pl.cfc_stride + (uint32_t)pip * (KK * 8);

        for (int q = 0; q < npass; ++q) {
            if (need_sf) {
                if (!mbar_wait(bar_sf_full, (uint32_t)(seg & 1))) {
                    atomicCAS(pl.fault, 0, (int)kFaultConsumerSf);
                    return;
                }
                const uint32_t sfs =
                    sbase + pl.off_sf + (uint32_t)(((unsigned long long)b * pl.sf_bytes) & 15ull);
                if constexpr (!BWDX) {
#pragma unroll
                    for (int t = 0; t < KK; ++t) {
                        const uint32_t a = sfs + (uint32_t)(((t * pl.OH + oy) * pl.OW + ox0) * ES);
                        if constexpr (G::SUBWORD || G::OUTB < 4) {
#pragma unroll
                            for (int pp = 0; pp < P; ++pp)
                                set_sf(t, pp, Word<T>::get(lds_elem_bits<T, true>(a + pp * ES), 0));
                        } else {
                            uint32_t w[G::OUTB / 4];
                            lds_vec<G::OUTB, true>(a, w);
#pragma unroll
                            for (int pp = 0; pp < P; ++pp)
                                set_sf(t, pp, Word<T>::get(w[pp / G::EPW], pp % G::EPW));
                        }
                    }
                    // Fused spatial FilterNorm (ddf/ddf.py:146-157): each pixel's k*k raw values
                    // become (v - mean) / (unbiased std + 1e-10) * scale, in registers, once
                    // per sample.  The dummy pixel of an odd P holds zeros and stays zero.
                    if constexpr (NORM) {
                        constexpr float inv_n = 1.f / (float)KK;
                        constexpr float inv_n1 = 1.f / (float)(KK > 1 ? KK - 1 : 1);
                        if constexpr (PK) {
#pragma unroll
                            for (int q2 = 0; q2 < PH; ++q2) {
                                unsigned long long sum2 = sf2[0][q2];
#pragma unroll
                                for (int t = 1; t < KK; ++t) sum2 = f2_add(sum2, sf2[t][q2]);
                                const unsigned long long nmean2 =
                                    f2_mul(sum2, f2_pack(-inv_n, -inv_n));
                                unsigned long long var2 = 0ull;
#pragma unroll
                                for (int t = 0; t < KK; ++t) {
                                    sf2[t][q2] = f2_add(sf2[t][q2], nmean2);
                                    var2 = f2_fma(sf2[t][q2], sf2[t][q2], var2);
                                }
                                float v0, v1;
                                f2_unpack(var2, v0, v1);
                                const unsigned long long inv2 =
                                    f2_pack(norm_gain(v0 * inv_n1, pl.sf_scale),
                                            norm_gain(v1 * inv_n1, pl.sf_scale));
#pragma unroll
                                for (int t = 0; t < KK; ++t) sf2[t][q2] = f2_mul(sf2[t][q2], inv2);
                            }
                        } else {
#pragma unroll
                            for (int pp = 0; pp < P; ++pp) {
                                float sum = 0.f;
#pragma unroll
                                for (int t = 0; t < KK; ++t) sum += sfr[t][pp];
                                const float mean = sum * inv_n;
                                float var = 0.f;
#pragma unroll
                                for (int t = 0; t < KK; ++t) {
                                    sfr[t][pp] -= mean;
                                    var = fmaf(sfr[t][pp], sfr[t][pp], var);
                                }
                                const float inv = norm_gain(var * inv_n1, pl.sf_scale);
#pragma unroll
                                for (int t = 0; t < KK; ++t) sfr[t][pp] *= inv;
                            }
                        }
                    }
                } else {
                    // grad-x: window tap (i,j) over go pairs with the filter value of
                    // the mirrored tap taken at the neighbouring pixel it came from.
#pragma unroll
                    for (int i = 0; i < K; ++i) {
#pragma unroll
                        for (int j = 0; j < K; ++j) {
                            const int ft = KK - 1 - (i * K + j);
                            const int yy = oy + (i - G::R) * D;
#pragma unroll
                            for (int pp = 0; pp < P; ++pp) {
                                const int xx = ox0 + pp + (j - G::R) * D;
                                float v = 0.f;
                                if (yy >= 0 && yy < pl.OH && xx >= 0 && xx < pl.OW) {
                                    const uint32_t a = sfs + (uint32_t)(((ft * pl.OH + yy) * pl.OW + xx) * ES);
                                    if constexpr (ES == 4) v = __uint_as_float(lds32v(a));
                                    else v = Word<T>::get(lds16v(a), 0);
                                }
                                set_sf(i * K + j, pp, v);
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_sf_empty);
                ++seg;
                need_sf = false;
            }
            // The stage is awaited after the spatial filter so that, at the start of the
            // kernel, taking the filter into registers overlaps the stage's arrival.
            if (q == 0 && (!mbar_wait(BAR_FULL(slot), ph) || !mbar_wait(BAR_READY(slot), ph))) {
                atomicCAS(pl.fault, 0, (int)kFaultConsumerFull);
                return;
            }

            float acc[PPT][PK ? 1 : P];
            unsigned long long acc2[PPT][PK ? PH : 1];
#pragma unroll
            for (int u = 0; u < PPT; ++u) {
                if constexpr (PK) {
#pragma unroll
                    for (int q2 = 0; q2 < PH; ++q2) acc2[u][q2] = 0ull;
                } else {
#pragma unroll
                    for (int pp = 0; pp < P; ++pp) acc[u][pp] = 0.f;
                }
            }
            // plane u of this thread within the pass is plane (u * TG + pip) of the pass
            const uint32_t plane_u = (uint32_t)TG * pl.plane_bytes;
            const uint32_t cfc_u = (uint32_t)TG * (KK * 8);

#pragma unroll
            for (int i = 0; i < K; ++i) {
                float xr[PPT][G::NCOL];
#pragma unroll
                for (int u = 0; u < PPT; ++u) {
                    const uint32_t rp = rowok[i] ? (plane_s + (uint32_t)u * plane_u + rowoff[i]) : zero_row;
                    load_row<T, G>(rp, lmask, rmask, xr[u]);
                }
#pragma unroll
                for (int j = 0; j < K; ++j) {
                    const int t = i * K + j;
#pragma unroll
                    for (int u = 0; u < PPT; ++u) {
                        const uint32_t ca = cfc_s + (uint32_t)u * cfc_u + 8u * (uint32_t)(BWDX ? (KK - 1 - t) : t);
                        if constexpr (PK) {
                            const unsigned long long c2 = lds64_pair(ca);
#pragma unroll
                            for (int q2 = 0; q2 < PH; ++q2) {
                                const unsigned long long w2 =
                                    MODE == DDF_B200_MUL ? f2_mul(c2, sf2[t][q2]) : f2_add(c2, sf2[t][q2]);
                                // the dummy pixel of an odd P re-reads the last column
                                constexpr int last = G::NCOL - 1;
                                const int hi_col = (q2 + PH) * S + j * D;
                                acc2[u][q2] = f2_fma(
                                    w2, f2_pack(xr[u][q2 * S + j * D], xr[u][hi_col < last ? hi_col : last]),
                                    acc2[u][q2]);
                            }
                        } else {
                            const float c = ldsf(ca);
#pragma unroll
                            for (int pp = 0; pp < P; ++pp)
                                acc[u][pp] = fmaf(combine_w<MODE, float>(c, sfr[t][pp]), xr[u][pp * S + j * D],
                                                  acc[u][pp]);
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < PPT; ++u) {
                float res[P];
                if constexpr (PK) {
#pragma unroll
                    for (int q2 = 0; q2 < PH; ++q2) {
                        float lo, hi;
                        f2_unpack(acc2[u][q2], lo, hi);
                        res[q2] = lo;
                        if (q2 + PH < P) res[q2 + PH] = hi;
                    }
                } else {
#pragma unroll
                    for (int pp = 0; pp < P; ++pp) res[pp] = acc[u][pp];
                }
                if (active) store_out<T, P>(outp + (long long)u * TG * out_plane, res);
            }

            plane_s += (uint32_t)NP * pl.plane_bytes;
            cfc_s += (uint32_t)NP * (KK * 8);
            outp += out_step;
            c_in_b += NP;
            if (c_in_b >= pl.C) {
                c_in_b = 0;
                ++b;
                need_sf = true;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(BAR_EMPTY(slot));
    }
#undef BAR_FULL
#undef BAR_EMPTY
#undef BAR_READY
#undef STAGE_BASE
}

// ------------------------------------------------------------------------ host side
// Launch with programmatic stream serialization: the grid may start while the previous
// kernel in the stream is finishing.  Only for kernels that execute griddepcontrol.wait
// before their first global-memory access.
template <typename... KArgs, typename... Args>
cudaError_t launch_overlapped(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, bool overlap, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1u : 0u;
    return cudaLaunchKernelEx(&cfg, kern, args...);
}

struct StreamArgs {
    const void* in;
    const void* cf;
    const void* sf;
    void* out;
    Problem p;
    bool bwdx;
    int sm_count;
    int* fault;
    int P;       // pixels per thread chosen by the dispatcher
    int device;  // current CUDA device index
    int ppt;     // planes per thread per pass to try first (2 or 1)
    int stage_bytes;  // target size of one ring stage; 0 = chosen from the plane size
    bool overlap_launch;  // launch with programmatic stream serialization
};

inline uint32_t round_up(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

// Fills the plan; returns false when the problem does not fit this kernel.
template <typename T, int K, int D, int S, int P, int PPT>
bool make_stream_plan(const StreamArgs& a, StreamPlan& pl, uint32_t& smem_bytes, int& grid) {
    using G = Geo<T, K, D, S, P>;
    const Problem& p = a.p;
    // Input / output plane geometry as the kernel sees it.
    const int H = a.bwdx ? p.OH : p.H, W = a.bwdx ? p.OW : p.W;
    const int OH = a.bwdx ? p.OH : p.OH, OW = a.bwdx ? p.OW : p.OW;
    if (a.bwdx && (p.s != 1)) return false;
    if (OW % P != 0 || W != OW * S) return false;
    if ((long long)H * W * G::ES > (1ll << 20)) return false;
    const int TP = OH * OW / P;
    if (TP < 1 || TP > kMaxComputeThreads) return false;
    int TG = kMaxComputeThreads / TP;  // thread groups
    while (TG > 1 && p.C % (TG * PPT) != 0) --TG;
    if (p.C % (TG * PPT) != 0) return false;
    const int NP = TG * PPT;  // planes per pass
    const long long planes = (long long)p.B * p.C;
    // Two planes per thread only while every CTA still gets a fair number of passes.
    if (PPT > 1 && planes / NP < 8ll * a.sm_count) return false;
    const uint32_t plane_bytes = (uint32_t)(H * W * G::ES);
    const uint32_t sf_bytes = (uint32_t)(G::KK * OH * OW * G::ES);
    // 16-byte rules of the bulk copies.
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    if (!al16(a.in) || !al16(a.cf) || !al16(a.sf) || !al16(a.out)) return false;

    // Stage size.  The service warp does a fixed amount of serial work per stage, so
    // large planes (>= 3 KB) want stages of two or more passes and about 48 KB;
    // small planes run best with about 16 KB.  a.stage_bytes > 0 overrides the target.
    const bool large_plane = plane_bytes >= 3072u;
    const uint32_t target = a.stage_bytes > 0 ? (uint32_t)a.stage_bytes
                                              : (large_plane ? 48u << 10 : 16u << 10);
    int PPS = (int)(target / ((uint32_t)NP * plane_bytes));
    if (a.stage_bytes <= 0 && large_plane && PPS < 2) PPS = 2;
    const long long total_passes = planes / NP;
    // Do not make stages longer than a CTA's share.
    const long long share = (total_passes + a.sm_count - 1) / a.sm_count;
    if (PPS > share) PPS = (int)share;
    if (PPS < 1) PPS = 1;

    pl.off_zero = 512;
    pl.off_cfc = pl.off_zero + 256;
    const uint32_t sf_region = round_up(sf_bytes + 32u, 128);
    // Ring slots that fit with PPS passes per stage (fills the layout fields).
    auto layout = [&](int pps) {
        const uint32_t SPL = (uint32_t)pps * NP;
        pl.cfc_stride = round_up(SPL * G::KK * 8u, 16);
        const uint32_t x_region = 32u + SPL * plane_bytes + 16u + 32u;
        pl.off_rawcf = round_up(x_region, 16);
        pl.stage_stride = round_up(pl.off_rawcf + SPL * G::KK * G::ES + 32u, 128);
        for (int slots = kMaxSlots; slots >= 1; --slots) {
            const uint32_t off_sf = round_up(pl.off_cfc + (uint32_t)slots * pl.cfc_stride, 128);
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
    // Shorten the stages until at least three fit (two when a stage is a single pass).
    int slots = layout(PPS);
    while (slots < 3 && PPS > 1) slots = layout(--PPS);
    if (slots < 2) return false;
    pl.n_slots = slots;
    pl.in = a.in; pl.cf = a.cf; pl.sf = a.sf; pl.out = a.out;
    pl.C = p.C; pl.H = H; pl.W = W; pl.OH = OH; pl.OW = OW;
    pl.tasks_per_plane = TP;
    pl.groups_per_row = OW / P;
    pl.planes_per_pass = NP;
    pl.thread_groups = TG;
    pl.passes_per_stage = PPS;
    pl.n_compute_warps = (TG * TP + 31) / 32;
    pl.total_passes = total_passes;
    pl.plane_bytes = plane_bytes;
    pl.sf_bytes = sf_bytes;
    pl.in_total = (unsigned long long)planes * plane_bytes;
    pl.cf_total = (unsigned long long)planes * G::KK * G::ES;
    pl.sf_total = (unsigned long long)p.B * sf_bytes;
    pl.fault = a.fault;
    if (a.bwdx && p.sf_norm) return false;  // grad-x takes the normalised filter
    pl.sf_scale = (float)p.sf_scale;
    grid = (int)(total_passes < a.sm_count ? total_passes : a.sm_count);
    return true;
}

template <typename T, int K, int D, int S, int P, int MODE, bool BWDX, int PPT = 1, bool NORM = false>
int stream_launch(const StreamArgs& a, cudaStream_t stream) {
    StreamPlan pl;
    uint32_t smem = 0;
    int grid = 0;
    if (!make_stream_plan<T, K, D, S, P, PPT>(a, pl, smem, grid)) return kNotHandled;
    constexpr bool PACK = sizeof(T) == 2 && P >= 2 && (P % 2 == 0 || PPT == 1);
    if (NORM != (a.p.sf_norm != 0)) return kNotHandled;
    auto kern = stream_kernel<T, K, D, S, P, MODE, BWDX, PACK, PPT, NORM>;
    // Opt in to the large dynamic shared-memory carve-out once per device and
    // kernel; steady-state launches (and launches under stream capture) then make
    // no call besides the launch itself.
    static std::atomic<unsigned long long> opted_in{0};
    const unsigned long long bit = 1ull << (a.device & 63);
    if (!(opted_in.load(std::memory_order_acquire) & bit)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)kSmemBudget);
        if (e != cudaSuccess) return (int)e;
        opted_in.fetch_or(bit, std::memory_order_release);
    }
    return (int)launch_overlapped(kern, dim3((unsigned)grid), dim3((unsigned)((pl.n_compute_warps + 1) * 32)),
                                  smem, stream, a.overlap_launch, pl);
}

// Runtime (k, d, s, P, mode, bwdx) -> instantiation.  Defined once per element
// type in stream_inst_<type>.cu.
template <typename T>
int stream_dispatch(const StreamArgs& a, cudaStream_t stream);

}  // namespace ddf
