// Plane-streaming kernel for the two filter gradients of the DDF op:
//
//   gcf[b,c,t]   = sum_{y,x} go[b,c,y,x] * x[b,c,y*s+oi,x*s+oj] * (sf[b,t,y,x] | 1)
//   gsf[b,t,y,x] = sum_c     go[b,c,y,x] * x[b,c,y*s+oi,x*s+oj] * (cf[b,c,t]   | 1)
//
// (the factor in parentheses is present for 'mul' and absent for 'add').  Both
// share the product go * x, so one pass over go and x produces both.
//
// The structure is that of the forward streaming kernel (stream_fwd.cuh): a
// persistent grid, each CTA owning a contiguous run of (b, c) planes; a service
// warp feeds go planes, x planes and channel filters through a ring of
// shared-memory stages with bulk async copies; every compute thread owns P output
// pixels for the whole kernel.
//
//   gsf  is a sum over channels at fixed pixel: each thread accumulates its
//        k*k*P values in registers while its CTA walks the channels of a sample
//        and writes them, as float partial sums, to a scratch slot when the run
//        leaves the sample (or ends).  A sample's channels may be split over a
//        few CTAs; gsf_reduce_kernel adds the slots in a fixed order (no atomics,
//        so the result is deterministic) and rounds to the element type.
//   gcf  is a sum over pixels at fixed channel: each thread forms k*k partial
//        sums per plane, a warp folds them with a multi-value butterfly (12
//        shuffles for 9 values instead of 45) and leaves one value per warp and
//        tap in the stage's shared-memory slot; when a stage is released the
//        service warp adds the per-warp values and stores gcf.
//
// Threads of one plane are padded to whole warps so that a warp never mixes
// two planes.
#pragma once

#include "stream_fwd.cuh"

namespace ddf {

constexpr int kBwdComputeThreads = 448;  // 14 warps; + 1 service warp = 480 threads
constexpr int kBwdThreads = kBwdComputeThreads + 32;

struct BwdPlan {
    const void* go;
    const void* x;
    const void* cf;
    const void* sf;
    void* gcf;       // may be null
    float* scratch;  // gsf partial sums; null when gsf is not wanted
    int C, H, W, OH, OW;
    int tasks_per_plane;   // OH*OW / P
    int tasks_padded;      // rounded up to a multiple of 32
    int groups_per_row;
    int planes_per_pass;
    int passes_per_stage;
    int n_slots;
    int n_compute_warps;
    int warps_per_plane;
    long long total_passes;
    uint32_t xplane_bytes, gplane_bytes, sf_bytes;
    unsigned long long x_total, go_total, cf_total, sf_total;   // byte sizes of the whole tensors
    uint32_t off_zero, off_cfc, cfc_stride, off_sf, off_stage0, stage_stride;
    uint32_t off_x, off_rawcf, off_gpart;  // inside a stage
    int* fault;
};

// Folds GROUP per-lane values across the warp.  On return lanes whose `slot`
// (precomputed by butterfly_slot) is >= 0 hold in v[0] the warp total of value
// number `slot`.
template <int GROUP>
__device__ __forceinline__ void butterfly_reduce(float (&v)[GROUP], int lane) {
    int n = GROUP;
#pragma unroll
    for (int lvl = 0; lvl < 5; ++lvl) {
        const int o = 16 >> lvl;
        const int lo = (n + 1) / 2;
        const bool upper = (lane & o) != 0;
#pragma unroll
        for (int i = 0; i < lo; ++i) {
            const float keep_lo = v[i];
            const float keep_hi = (lo + i < n) ? v[lo + i] : 0.f;
            const float recv = __shfl_xor_sync(0xffffffffu, upper ? keep_lo : keep_hi, o);
            v[i] = (upper ? keep_hi : keep_lo) + recv;
        }
        n = lo;
    }
}

// Which of the GROUP values ends up in this lane (-1: none).  Mirrors the
// splits butterfly_reduce makes: every level halves the (compile-time) array
// length n; `cnt` is how many of this lane's array entries are real values.
template <int GROUP>
__device__ __forceinline__ int butterfly_slot(int lane) {
    int n = GROUP, first = 0, cnt = GROUP;
#pragma unroll
    for (int lvl = 0; lvl < 5; ++lvl) {
        const int lo = (n + 1) / 2;
        if (lane & (16 >> lvl)) {
            first += lo;
            cnt = cnt > lo ? cnt - lo : 0;
        } else {
            cnt = cnt < lo ? cnt : lo;
        }
        n = lo;
    }
    return cnt > 0 ? first : -1;
}

// WHICH: 0 = both gradients in one pass; 1 = grad-cf only; 2 = grad-sf only.  The two
// single-gradient forms need half the registers (either the spatial-filter values or the
// grad-sf accumulators), which is what lets a thread own 8 pixels and a CTA's threads cover
// a 56 x 56 plane; the launcher then runs them one after the other.
template <typename T, int K, int D, int S, int P, int MODE, int WHICH>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_filters_kernel(const __grid_constant__ BwdPlan pl) {
    using G = Geo<T, K, D, S, P>;
    constexpr int KK = G::KK;
    constexpr int ES = G::ES;
    constexpr bool MUL = MODE == DDF_B200_MUL;
    constexpr bool DO_CF = WHICH != 2, DO_SF = WHICH != 1;
    // values folded per butterfly: all taps at once for k = 3, one tap row for k = 5
    constexpr int GROUP = (K == 3) ? KK : K;
    constexpr int ROWS_PER_GROUP = GROUP / K;

    extern __shared__ __align__(128) unsigned char smem_raw[];
    const uint32_t sbase = smem_u32(smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int NST = pl.n_slots;
    const int NCW = pl.n_compute_warps;
    const int NP = pl.planes_per_pass;
    const int PPS = pl.passes_per_stage;
    const int WPP = pl.warps_per_plane;

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
    if (tid < 64) sts32(sbase + pl.off_zero + 4u * tid, 0u);
    __syncthreads();
    // Programmatic dependent launch (see stream_kernel): no global access before this.
    asm volatile("griddepcontrol.launch_dependents;");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    const long long pass_lo = (pl.total_passes * (long long)blockIdx.x) / gridDim.x;
    const long long pass_hi = (pl.total_passes * (long long)(blockIdx.x + 1)) / gridDim.x;
    const int my_passes = (int)(pass_hi - pass_lo);
    if (my_passes == 0) return;
    const int my_stages = (my_passes + PPS - 1) / PPS;
    const long long plane_lo = pass_lo * NP, plane_hi = pass_hi * NP;
    const int stage_planes = PPS * NP;

    if (warp == NCW) {
        // ------------------------------------------------------------- service warp
        int issue_i = 0, conv_j = 0, red_r = 0, seg_k = 0;
        long long seg_b = plane_lo / pl.C;
        long long seg_plane = plane_lo;
        long long idle_since = -1;
        bool gave_up = false;
        while (red_r < my_stages || (MUL && seg_plane < plane_hi)) {
            bool progress = false;
            // (1) spatial filter of the next sample ('mul' only), see stream_fwd.cuh
            if constexpr (MUL) {
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
            // (2) next stage: its slot is reusable once the stage that used it has been
            // released by the compute warps AND its channel-filter-gradient partials
            // have been folded (red_r counts folded stages).
            if (issue_i < my_stages && (issue_i < NST || red_r > issue_i - NST)) {
                const int slot = issue_i % NST;
                const long long st_first = plane_lo + (long long)issue_i * stage_planes;
                long long st_end = st_first + stage_planes;
                if (st_end > plane_hi) st_end = plane_hi;
                if (lane == 0) {
                    const unsigned long long n0 = (unsigned long long)st_first, n1 = (unsigned long long)st_end;
                    // a copy never reads past its tensor's last whole 16 bytes (see span_prepare)
                    const Span sg = span_prepare(STAGE_BASE(slot) + 32u, pl.go, n0 * pl.gplane_bytes,
                                                 n1 * pl.gplane_bytes, pl.go_total);
                    const Span sx = span_prepare(STAGE_BASE(slot) + pl.off_x, pl.x, n0 * pl.xplane_bytes,
                                                 n1 * pl.xplane_bytes, pl.x_total);
                    Span sc{0u, nullptr, 0u};
                    if constexpr (MUL)
                        sc = span_prepare(STAGE_BASE(slot) + pl.off_rawcf, pl.cf, n0 * (KK * ES), n1 * (KK * ES),
                                          pl.cf_total);
                    mbar_arrive_expect_tx(BAR_FULL(slot), sg.bytes + sx.bytes + sc.bytes);
                    span_issue(sg, BAR_FULL(slot));
                    span_issue(sx, BAR_FULL(slot));
                    span_issue(sc, BAR_FULL(slot));
                }
                ++issue_i;
                progress = true;
            }
            if (conv_j < issue_i) {
                const int slot = conv_j % NST;
                if (warp_test(BAR_FULL(slot), (uint32_t)((conv_j / NST) & 1), lane)) {
                    if constexpr (MUL) {
                        const long long st_first = plane_lo + (long long)conv_j * stage_planes;
                        long long st_end = st_first + stage_planes;
                        if (st_end > plane_hi) st_end = plane_hi;
                        const int n = (int)(st_end - st_first) * KK;
                        const uint32_t coff = (uint32_t)(((unsigned long long)st_first * (KK * ES)) & 15ull);
                        const uint32_t src = STAGE_BASE(slot) + pl.off_rawcf + coff;
                        const uint32_t dst = sbase + pl.off_cfc + (uint32_t)slot * pl.cfc_stride;
                        for (int e = lane; e < n; e += 32) {
                            float v;
                            if constexpr (ES == 4) v = ldsf(src + 4u * e);
                            else v = Word<T>::get(lds16(src + 2u * e), 0);
                            sts32(dst + 8u * e, __float_as_uint(v));       // (cf, cf) for the
                            sts32(dst + 8u * e + 4u, __float_as_uint(v));  // two-wide FMA
                        }
                        __syncwarp();
                    }
                    if (lane == 0) mbar_arrive(BAR_READY(slot));
                    ++conv_j;
                    progress = true;
                }
            }
            if (red_r < conv_j) {
                const int slot = red_r % NST;
                if (warp_test(BAR_EMPTY(slot), (uint32_t)((red_r / NST) & 1), lane)) {
                    // Fold the per-warp partial sums of this stage and store gcf.
                    const long long st_first = plane_lo + (long long)red_r * stage_planes;
                    long long st_end = st_first + stage_planes;
                    if (st_end > plane_hi) st_end = plane_hi;
                    const int n = (int)(st_end - st_first) * KK;
                    if (pl.gcf != nullptr) {
                        T* dst = reinterpret_cast<T*>(pl.gcf) + st_first * KK;
                        const uint32_t src = STAGE_BASE(slot) + pl.off_gpart;
                        for (int e = lane; e < n; e += 32) {
                            const int plane = e / KK, t = e - plane * KK;
                            float tot = 0.f;
                            for (int w = 0; w < WPP; ++w)
                                tot += ldsf(src + 4u * (uint32_t)((plane * WPP + w) * KK + t));
                            Elem<T>::store(dst + e, tot);
                        }
                    }
                    __syncwarp();
                    ++red_r;
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
            if (lane == 0) atomicCAS(pl.fault, 0, (int)kFaultService);
            bool drained = true;
            for (int j = conv_j; j < issue_i; ++j)
                drained &= mbar_wait(BAR_FULL(j % NST), (uint32_t)((j / NST) & 1));
            if (MUL && seg_k > 0) drained &= mbar_wait(bar_sf_full, (uint32_t)((seg_k - 1) & 1));
            if (!drained && lane == 0) atomicExch(pl.fault, (int)kFaultDrain);
        }
        return;
    }
    if (warp > NCW) return;

    // ----------------------------------------------------------------- compute warps
    const int TP = pl.tasks_per_plane;
    const int TPW = pl.tasks_padded;
    const int pip = tid / TPW;  // plane within the pass; a warp never straddles two
    int task = tid - pip * TPW;
    const bool active = task < TP;
    if (!active) task = 0;
    const int wip = (tid - pip * TPW) >> 5;  // warp within the plane
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
    const uint32_t go_off = (uint32_t)((oy * pl.OW + ox0) * ES);
    const int my_slot = butterfly_slot<GROUP>(lane);

    // With P >= 2 the arithmetic is two-wide (mul/fma.f32x2): pixel pp pairs with
    // pixel pp + P/2 in the spatial-filter registers, the gsf accumulators, the
    // upstream gradient and the partial sums.
    // (2-byte element types only: their unpack can target any register, so pairs form
    // for free; float elements arrive in load order and pairing them costs moves.)
    constexpr bool PK = P >= 2 && sizeof(T) == 2;
    constexpr int HP = PK ? P / 2 : 1;
    float sfr[(MUL && !PK && DO_CF) ? KK : 1][(PK || !DO_CF) ? 1 : P];
    float gsf[(PK || !DO_SF) ? 1 : KK][(PK || !DO_SF) ? 1 : P];
    unsigned long long sf2[(MUL && PK && DO_CF) ? KK : 1][DO_CF ? HP : 1];
    unsigned long long gsf2[(PK && DO_SF) ? KK : 1][DO_SF ? HP : 1];
    if constexpr (DO_SF) {
#pragma unroll
        for (int t = 0; t < KK; ++t) {
            if constexpr (PK) {
#pragma unroll
                for (int q2 = 0; q2 < HP; ++q2) gsf2[t][q2] = 0ull;
            } else {
#pragma unroll
                for (int pp = 0; pp < P; ++pp) gsf[t][pp] = 0.f;
            }
        }
    }

    long long b = plane_lo / pl.C;
    int c_in_b = (int)(plane_lo - b * pl.C);
    bool need_sf = true;
    int seg = 0;
    const long long opl = (long long)pl.OH * pl.OW;

    auto flush = [&](long long sample) {
        if constexpr (DO_SF) {
        if (pl.scratch != nullptr && active) {
            float* dst = pl.scratch + (((sample + blockIdx.x) * NP + pip) * KK) * opl +
                         (long long)oy * pl.OW + ox0;
#pragma unroll
            for (int t = 0; t < KK; ++t) {
                float v[P];
                if constexpr (PK) {
#pragma unroll
                    for (int q2 = 0; q2 < HP; ++q2) f2_unpack(gsf2[t][q2], v[q2], v[q2 + HP]);
                } else {
#pragma unroll
                    for (int pp = 0; pp < P; ++pp) v[pp] = gsf[t][pp];
                }
                if constexpr (P == 1) {
                    dst[t * opl] = v[0];
                } else if constexpr (P == 2) {
                    *reinterpret_cast<float2*>(dst + t * opl) = make_float2(v[0], v[1]);
                } else {
#pragma unroll
                    for (int u = 0; u < P / 4; ++u)
                        reinterpret_cast<float4*>(dst + t * opl)[u] =
                            make_float4(v[4 * u], v[4 * u + 1], v[4 * u + 2], v[4 * u + 3]);
                }
            }
        }
#pragma unroll
        for (int t = 0; t < KK; ++t) {
            if constexpr (PK) {
#pragma unroll
                for (int q2 = 0; q2 < HP; ++q2) gsf2[t][q2] = 0ull;
            } else {
#pragma unroll
                for (int pp = 0; pp < P; ++pp) gsf[t][pp] = 0.f;
            }
        }
        }
    };

    int slot = -1;
    uint32_t ph = 1;  // becomes slot 0, phase 0 on the first stage; no division per stage
    for (int st = 0; st < my_stages; ++st) {
        if (++slot == NST) slot = 0;
        if (slot == 0) ph ^= 1u;
        if (!mbar_wait(BAR_FULL(slot), ph) || !mbar_wait(BAR_READY(slot), ph)) {
            atomicCAS(pl.fault, 0, (int)kFaultConsumerFull);
            return;
        }
        const int first_pass = st * PPS;
        const int npass = (my_passes - first_pass) < PPS ? (my_passes - first_pass) : PPS;
        const unsigned long long sfp = (unsigned long long)plane_lo + (unsigned long long)first_pass * NP;
        const uint32_t xoff = (uint32_t)((sfp * pl.xplane_bytes) & 15ull);
        const uint32_t goff = (uint32_t)((sfp * pl.gplane_bytes) & 15ull);
        uint32_t xplane_s = STAGE_BASE(slot) + pl.off_x + xoff + (uint32_t)pip * pl.xplane_bytes;
        uint32_t gplane_s = STAGE_BASE(slot) + 32u + goff + (uint32_t)pip * pl.gplane_bytes + go_off;
        uint32_t cfc_s = sbase + pl.off_cfc + (uint32_t)slot * pl.cfc_stride + (uint32_t)pip * (KK * 8);
        uint32_t gpart_s = STAGE_BASE(slot) + pl.off_gpart + 4u * (uint32_t)((pip * WPP + wip) * KK);

        for (int q = 0; q < npass; ++q) {
            if constexpr (MUL) {
                if (need_sf) {
                    if (!mbar_wait(bar_sf_full, (uint32_t)(seg & 1))) {
                        atomicCAS(pl.fault, 0, (int)kFaultConsumerSf);
                        return;
                    }
                    const uint32_t sfs =
                        sbase + pl.off_sf + (uint32_t)(((unsigned long long)b * pl.sf_bytes) & 15ull);
#pragma unroll
                    for (int t = 0; t < (DO_CF ? KK : 0); ++t) {
                        const uint32_t a = sfs + (uint32_t)(((t * pl.OH + oy) * pl.OW + ox0) * ES);
                        if constexpr (G::OUTB < 4) {
                            sfr[t][0] = Word<T>::get(lds16v(a), 0);
                        } else {
                            uint32_t w[G::OUTB / 4];
                            lds_vec<G::OUTB, true>(a, w);
                            if constexpr (PK) {
#pragma unroll
                                for (int q2 = 0; q2 < HP; ++q2)
                                    sf2[t][q2] = f2_pack(Word<T>::get(w[q2 / G::EPW], q2 % G::EPW),
                                                         Word<T>::get(w[(q2 + HP) / G::EPW], (q2 + HP) % G::EPW));
                            } else {
#pragma unroll
                                for (int pp = 0; pp < P; ++pp)
                                    sfr[t][pp] = Word<T>::get(w[pp / G::EPW], pp % G::EPW);
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_sf_empty);
                    ++seg;
                    need_sf = false;
                }
            }

            // upstream gradient at this thread's pixels
            float g[P];
            if constexpr (G::OUTB < 4) {
                g[0] = Word<T>::get(lds16(gplane_s), 0);
            } else {
                uint32_t w[G::OUTB / 4];
                lds_vec<G::OUTB>(gplane_s, w);
#pragma unroll
                for (int pp = 0; pp < P; ++pp) g[pp] = Word<T>::get(w[pp / G::EPW], pp % G::EPW);
            }

            unsigned long long g2[HP];
            if constexpr (PK) {
#pragma unroll
                for (int q2 = 0; q2 < HP; ++q2) g2[q2] = f2_pack(g[q2], g[q2 + HP]);
            }

#pragma unroll
            for (int i0 = 0; i0 < K; i0 += ROWS_PER_GROUP) {
                float part[GROUP];
                unsigned long long part2[PK ? GROUP : 1];
#pragma unroll
                for (int u = 0; u < GROUP; ++u) {
                    part[u] = 0.f;
                    if constexpr (PK) part2[u] = 0ull;
                }
#pragma unroll
                for (int ii = 0; ii < ROWS_PER_GROUP; ++ii) {
                    const int i = i0 + ii;
                    const uint32_t rp = rowok[i] ? (xplane_s + rowoff[i]) : zero_row;
                    float xr[G::NCOL];
                    load_row<T, G>(rp, lmask, rmask, xr);
#pragma unroll
                    for (int j = 0; j < K; ++j) {
                        const int t = i * K + j;
                        const int u = ii * K + j;
                        if constexpr (PK) {
                            unsigned long long c2 = 0ull;
                            if constexpr (MUL && DO_SF) c2 = lds64_pair(cfc_s + 8u * t);
#pragma unroll
                            for (int q2 = 0; q2 < HP; ++q2) {
                                const unsigned long long prod2 =
                                    f2_mul(g2[q2], f2_pack(xr[q2 * S + j * D], xr[(q2 + HP) * S + j * D]));
                                if constexpr (MUL) {
                                    if constexpr (DO_SF) gsf2[t][q2] = f2_fma(prod2, c2, gsf2[t][q2]);
                                    if constexpr (DO_CF) part2[u] = f2_fma(prod2, sf2[t][q2], part2[u]);
                                } else {
                                    if constexpr (DO_SF) gsf2[t][q2] = f2_add(gsf2[t][q2], prod2);
                                    if constexpr (DO_CF) part2[u] = f2_add(part2[u], prod2);
                                }
                            }
                        } else {
                            float c = 1.f;
                            if constexpr (MUL && DO_SF) c = ldsf(cfc_s + 8u * t);
#pragma unroll
                            for (int pp = 0; pp < P; ++pp) {
                                const float prod = g[pp] * xr[pp * S + j * D];
                                if constexpr (MUL) {
                                    if constexpr (DO_SF) gsf[t][pp] = fmaf(prod, c, gsf[t][pp]);
                                    if constexpr (DO_CF) part[u] = fmaf(prod, sfr[t][pp], part[u]);
                                } else {
                                    if constexpr (DO_SF) gsf[t][pp] += prod;
                                    if constexpr (DO_CF) part[u] += prod;
                                }
                            }
                        }
                    }
                }
                if constexpr (DO_CF) {
                    if constexpr (PK) {
#pragma unroll
                        for (int u = 0; u < GROUP; ++u) {
                            float lo, hi;
                            f2_unpack(part2[u], lo, hi);
                            part[u] = lo + hi;
                        }
                    }
                    if (!active) {
#pragma unroll
                        for (int u = 0; u < GROUP; ++u) part[u] = 0.f;
                    }
                    butterfly_reduce<GROUP>(part, lane);
                    if (my_slot >= 0)
                        sts32(gpart_s + 4u * (uint32_t)(i0 * K + my_slot), __float_as_uint(part[0]));
                }
            }

            xplane_s += (uint32_t)NP * pl.xplane_bytes;
            gplane_s += (uint32_t)NP * pl.gplane_bytes;
            cfc_s += (uint32_t)NP * (KK * 8);
            gpart_s += 4u * (uint32_t)(NP * WPP * KK);
            c_in_b += NP;
            if (c_in_b >= pl.C) {
                flush(b);
                c_in_b = 0;
                ++b;
                need_sf = true;
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(BAR_EMPTY(slot));
    }
    if (c_in_b != 0) flush(b);
#undef BAR_FULL
#undef BAR_EMPTY
#undef BAR_READY
#undef STAGE_BASE
}

// gsf[b, e] = sum over the CTAs whose plane run touched sample b, and over the
// planes-per-pass lanes of each, of their float partials; fixed order.
template <typename T>
__global__ void __launch_bounds__(256)
gsf_reduce_kernel(const float* __restrict__ scratch, T* __restrict__ gsf, int B, int C, int NP,
                  long long n_per_sample, long long total_passes, int grid_main) {
    // May have been launched while the filter-gradient kernel was finishing.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __shared__ long long s_c0;
    __shared__ int s_nslot;
    for (long long b = blockIdx.y; b < B; b += gridDim.y) {
        // passes of sample b, and the CTAs of the main kernel that owned them: 64-bit
        // divisions, done by one thread per block instead of by every thread
        __syncthreads();
        if (threadIdx.x == 0) {
            const long long q0 = b * C / NP, q1 = (b + 1) * C / NP - 1;
            const long long c0 = ((q0 + 1) * grid_main - 1) / total_passes;
            const long long c1 = ((q1 + 1) * grid_main - 1) / total_passes;
            s_c0 = c0;
            s_nslot = (int)(c1 - c0 + 1) * NP;
        }
        __syncthreads();
        // The slots of those CTAs are consecutive: slot j holds n_per_sample floats.
        const int nslot = s_nslot;
        const float* base = scratch + (b + s_c0) * NP * n_per_sample;
        if ((n_per_sample & 3) == 0 && ((reinterpret_cast<uintptr_t>(scratch) | reinterpret_cast<uintptr_t>(gsf)) & 15u) == 0) {
            // four elements per thread: 16-byte loads, four slots in flight; the order of the
            // additions is fixed, so the result does not depend on scheduling
            const long long n4 = n_per_sample >> 2;
            for (long long e4 = blockIdx.x * (long long)blockDim.x + threadIdx.x; e4 < n4;
                 e4 += (long long)gridDim.x * blockDim.x) {
                float4 acc[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int j0 = 0; j0 < nslot; j0 += 4) {
                    float4 v[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        v[u] = (j0 + u < nslot)
                                   ? __ldg(reinterpret_cast<const float4*>(base + (long long)(j0 + u) * n_per_sample) + e4)
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        acc[u].x += v[u].x; acc[u].y += v[u].y; acc[u].z += v[u].z; acc[u].w += v[u].w;
                    }
                }
                float tot[4];
                tot[0] = (acc[0].x + acc[1].x) + (acc[2].x + acc[3].x);
                tot[1] = (acc[0].y + acc[1].y) + (acc[2].y + acc[3].y);
                tot[2] = (acc[0].z + acc[1].z) + (acc[2].z + acc[3].z);
                tot[3] = (acc[0].w + acc[1].w) + (acc[2].w + acc[3].w);
                T* dst = gsf + b * n_per_sample + 4 * e4;
                if constexpr (sizeof(T) == 4) {
                    *reinterpret_cast<float4*>(dst) = make_float4(tot[0], tot[1], tot[2], tot[3]);
                } else if constexpr (sizeof(T) == 2) {
                    *reinterpret_cast<uint2*>(dst) = make_uint2(Word<T>::put(tot[0], tot[1]), Word<T>::put(tot[2], tot[3]));
                } else {
#pragma unroll
                    for (int u = 0; u < 4; ++u) Elem<T>::store(dst + u, tot[u]);
                }
            }
            continue;
        }
        for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < n_per_sample;
             e += (long long)gridDim.x * blockDim.x) {
            // Eight loads in flight per thread; fixed order of additions.
            float acc[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) acc[u] = 0.f;
            for (int j0 = 0; j0 < nslot; j0 += 8) {
                float v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    v[u] = (j0 + u < nslot) ? __ldg(base + (long long)(j0 + u) * n_per_sample + e) : 0.f;
#pragma unroll
                for (int u = 0; u < 8; ++u) acc[u] += v[u];
            }
            const float tot = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
            Elem<T>::store(gsf + b * n_per_sample + e, tot);
        }
    }
}

// ------------------------------------------------------------------------ host side
struct BwdArgs {
    const void* go;
    const void* x;
    const void* cf;
    const void* sf;
    void* gcf;
    void* gsf;
    void* workspace;
    Problem p;
    int sm_count;
    int* fault;
    int P;
    int device;
    bool overlap_launch;  // launch with programmatic stream serialization
};

struct BwdGeometry {
    int P, TP, TPW, NP, grid;
    long long total_passes;
};

// Thread layout shared by the launcher, the workspace query and the reducer.
inline bool bwd_geometry(const Problem& p, int P, int sm_count, BwdGeometry& g) {
    if (p.OW % P != 0 || p.W != p.OW * p.s) return false;
    const int TP = p.OH * p.OW / P;
    const int TPW = (TP + 31) / 32 * 32;
    if (TP < 1 || TPW > kBwdComputeThreads) return false;
    int NP = kBwdComputeThreads / TPW;
    while (NP > 1 && p.C % NP != 0) --NP;
    g.P = P; g.TP = TP; g.TPW = TPW; g.NP = NP;
    g.total_passes = (long long)p.B * p.C / NP;
    g.grid = (int)(g.total_passes < sm_count ? g.total_passes : sm_count);
    return true;
}

inline size_t bwd_workspace_bytes(const Problem& p, const BwdGeometry& g) {
    return (size_t)(p.B + g.grid) * g.NP * p.k * p.k * p.OH * p.OW * sizeof(float);
}

template <typename T, int K, int D, int S, int P>
bool make_bwd_plan(const BwdArgs& a, BwdPlan& pl, uint32_t& smem_bytes, BwdGeometry& g) {
    using G = Geo<T, K, D, S, P>;
    const Problem& p = a.p;
    if (!bwd_geometry(p, P, a.sm_count, g)) return false;
    const long long planes = (long long)p.B * p.C;
    const uint32_t xpb = (uint32_t)(p.H * p.W * G::ES);
    const uint32_t gpb = (uint32_t)(p.OH * p.OW * G::ES);
    const uint32_t sfb = (uint32_t)(G::KK * p.OH * p.OW * G::ES);
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    if (!al16(a.go) || !al16(a.x) || !al16(a.cf) || !al16(a.sf)) return false;
    if (a.workspace && !al16(a.workspace)) return false;

    // Stages of about 48 KB: the service warp's per-stage duties (expanding channel
    // filters, folding the grad-cf partials, three copies) are a serial chain; with
    // one pass per stage the compute warps end up waiting for it.
    int PPS = (int)(49152u / ((uint32_t)g.NP * (xpb + gpb)));
    if (PPS < 1) PPS = 1;
    const long long share = (g.total_passes + a.sm_count - 1) / a.sm_count;
    if (PPS > share) PPS = (int)share;
    if (PPS < 1) PPS = 1;
    const int SPL = PPS * g.NP;
    const int WPP = g.TPW / 32;

    pl.off_zero = 512;
    pl.off_cfc = pl.off_zero + 256;
    pl.cfc_stride = round_up((uint32_t)SPL * G::KK * 8u, 16);
    const uint32_t go_region = 32u + (uint32_t)SPL * gpb + 16u + 32u;
    pl.off_x = round_up(go_region, 16) + 32u;
    const uint32_t x_end = pl.off_x + (uint32_t)SPL * xpb + 16u + 32u;
    pl.off_rawcf = round_up(x_end, 16);
    pl.off_gpart = round_up(pl.off_rawcf + (uint32_t)SPL * G::KK * G::ES + 32u, 16);
    pl.stage_stride = round_up(pl.off_gpart + (uint32_t)SPL * WPP * G::KK * 4u, 128);
    const uint32_t sf_region = round_up(sfb + 32u, 128);
    int slots = kMaxSlots;
    for (;; --slots) {
        if (slots < 2) return false;
        const uint32_t off_sf = round_up(pl.off_cfc + (uint32_t)slots * pl.cfc_stride, 128);
        const uint32_t total = off_sf + sf_region + (uint32_t)slots * pl.stage_stride;
        if (total <= kSmemBudget) {
            pl.off_sf = off_sf;
            pl.off_stage0 = off_sf + sf_region;
            smem_bytes = total;
            break;
        }
    }
    pl.n_slots = slots;
    pl.go = a.go; pl.x = a.x; pl.cf = a.cf; pl.sf = a.sf;
    pl.gcf = a.gcf;
    pl.scratch = a.gsf ? reinterpret_cast<float*>(a.workspace) : nullptr;
    pl.C = p.C; pl.H = p.H; pl.W = p.W; pl.OH = p.OH; pl.OW = p.OW;
    pl.tasks_per_plane = g.TP;
    pl.tasks_padded = g.TPW;
    pl.groups_per_row = p.OW / P;
    pl.planes_per_pass = g.NP;
    pl.passes_per_stage = PPS;
    pl.n_compute_warps = g.NP * WPP;
    pl.warps_per_plane = WPP;
    pl.total_passes = g.total_passes;
    pl.xplane_bytes = xpb;
    pl.gplane_bytes = gpb;
    pl.sf_bytes = sfb;
    pl.x_total = (unsigned long long)planes * xpb;
    pl.go_total = (unsigned long long)planes * gpb;
    pl.cf_total = (unsigned long long)planes * G::KK * G::ES;
    pl.sf_total = (unsigned long long)p.B * sfb;
    pl.fault = a.fault;
    return true;
}

template <typename T, int K, int D, int S, int P, int MODE, int WHICH = 0>
int bwd_launch(const BwdArgs& a, cudaStream_t stream, int* launches) {
    BwdPlan pl;
    BwdGeometry g;
    uint32_t smem = 0;
    if (!make_bwd_plan<T, K, D, S, P>(a, pl, smem, g)) return kNotHandled;
    if (a.gsf && !a.workspace) return DDF_B200_E_WORKSPACE;
    auto kern = bwd_filters_kernel<T, K, D, S, P, MODE, WHICH>;
    static std::atomic<unsigned long long> opted_in{0};
    const unsigned long long bit = 1ull << (a.device & 63);
    if (!(opted_in.load(std::memory_order_acquire) & bit)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)kSmemBudget);
        if (e != cudaSuccess) return (int)e;
        opted_in.fetch_or(bit, std::memory_order_release);
    }
    const int threads = (pl.n_compute_warps + 1) * 32;
    cudaError_t e = launch_overlapped(kern, dim3((unsigned)g.grid), dim3((unsigned)threads), smem, stream,
                                      a.overlap_launch, pl);
    if (e != cudaSuccess) return (int)e;
    ++*launches;
    if (a.gsf) {
        const long long n = (long long)a.p.k * a.p.k * a.p.OH * a.p.OW;
        // one thread per four elements where the sample's size allows 16-byte accesses
        const bool vec = (n & 3) == 0 &&
                         ((reinterpret_cast<uintptr_t>(a.workspace) | reinterpret_cast<uintptr_t>(a.gsf)) & 15u) == 0;
        const long long work = vec ? n / 4 : n;
        dim3 grid((unsigned)((work + 255) / 256 < 64 ? (work + 255) / 256 : 64),
                  (unsigned)(a.p.B < 32768 ? a.p.B : 32768));
        e = launch_overlapped(gsf_reduce_kernel<T>, grid, dim3(256), 0, stream, a.overlap_launch,
                              reinterpret_cast<const float*>(a.workspace), reinterpret_cast<T*>(a.gsf),
                              a.p.B, a.p.C, g.NP, n, g.total_passes, g.grid);
        if (e != cudaSuccess) return (int)e;
        ++*launches;
    }
    return 0;
}

// The two gradients as two launches of the single-gradient forms (8 pixels per thread).
template <typename T, int K, int D, int S, int P, int MODE>
int bwd_launch_split(const BwdArgs& a, cudaStream_t stream, int* launches) {
    if (a.gcf) {
        BwdArgs one = a;
        one.gsf = nullptr;
        const int rc = bwd_launch<T, K, D, S, P, MODE, 1>(one, stream, launches);
        if (rc) return rc;
    }
    if (a.gsf) {
        BwdArgs one = a;
        one.gcf = nullptr;
        const int rc = bwd_launch<T, K, D, S, P, MODE, 2>(one, stream, launches);
        if (rc) return rc;
    }
    return 0;
}

template <typename T>
int bwd_dispatch(const BwdArgs& a, cudaStream_t stream, int* launches);

}  // namespace ddf
