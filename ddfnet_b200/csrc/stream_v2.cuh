// Plane-streaming DDF kernel, second generation (k = 3, dilation 1; forward at
// stride 1 and 2, grad-x at stride 1).
//
// The first-generation kernel (stream_fwd.cuh) is bound by instruction issue,
// not by HBM: its compute warps spend more instructions unpacking 2-byte
// elements, masking halos and pairing registers for the two-wide FMA than on the
// arithmetic itself.  This kernel moves all of that out of the compute warps:
//
//   service warps (3)  Warp 0's lane 0 issues the bulk async copies (TMA) of raw
//                      planes, channel filters and spatial filters, as before.
//                      All three warps then CONVERT each landed plane, once per
//                      input element, into the layout the arithmetic wants:
//                      float, zero-padded, and already paired for f32x2 math.
//   compute warps      A thread owns two segments A and B of L adjacent output
//                      pixels in one output row (2L outputs).  Its inner loop is
//                      nothing but 128-bit shared loads and packed arithmetic:
//                      for every tap and pixel pair one mul.f32x2 (w = cf (.) sf)
//                      and one fma.f32x2, all operands aligned 64-bit register
//                      pairs that come straight out of the loads.
//
// Converted layout.  For input row r and pixel group g (2L output pixels) the
// record holds the pairs  P[m] = (xA[m-1], xB[m-1])  where xA / xB are the input
// row seen from segment A / B's first input column, m = 0 .. NPR-1, zero outside
// the plane.  Tap j of pixel pair k reads P[S*k + j].  Records are stored as
// 16-byte quads, quad-major (all records' quad 0, then all quad 1, ...), so every
// 128-bit load and store is unit-stride across a warp (no bank conflicts), and
// with one zero row above and below the plane so that vertical padding needs no
// test either.
#pragma once

#include <atomic>

#include "stream_fwd.cuh"

namespace ddf {

constexpr int kV2ServiceWarps = 3;
constexpr int kV2MaxComputeThreads = 416;                        // 13 warps
constexpr int kV2Threads = kV2MaxComputeThreads + 32 * kV2ServiceWarps;  // 512
constexpr int kV2MaxCSlots = 8;

struct V2Plan {
    const void* in;
    const void* cf;
    const void* sf;
    void* out;
    int C, H, W, OH, OW;
    int G;                 // pixel groups per output row = OW / (2L)
    int tasks_per_plane;   // OH * G
    int planes_per_pass;   // NP
    int passes_per_stage;  // PPS
    int n_slots;           // raw ring depth
    int n_cslots;          // converted ring depth
    int n_compute_warps;
    long long total_passes;
    uint32_t plane_bytes;   // raw input plane
    uint32_t sf_bytes;      // one sample's spatial filter (raw)
    uint32_t cplane_bytes;  // converted plane = NQ * (H + 2) * G * 16
    uint32_t quad_stride;   // (H + 2) * G * 16
    uint32_t off_ccf, ccf_stride, off_sf, off_stage0, stage_stride, off_rawcf, off_conv0, cslot_stride;
    int* fault;
};

template <typename T, int S, int L>
struct V2Geo {
    static constexpr int ES = (int)sizeof(T);
    static constexpr int EPW = 4 / ES;
    static constexpr int NPR = (S == 1) ? L + 2 : 2 * L + 1;  // pairs per record
    static constexpr int NQ = (NPR + 1) / 2;                  // 16-byte quads per record
    static constexpr int MAINN = S * 2 * L;                   // raw elements of a group's row
    static constexpr int MAINB = MAINN * ES;
    static constexpr int NV = S * L + NPR;                    // distinct input values per record
    static constexpr bool RIGHT_HALO = (S == 1);
    static constexpr int P = 2 * L;
    static constexpr int OUTB = P * ES;
    static_assert(S == 1 || S == 2, "stride 1 or 2");
    static_assert(L == 1 || L == 2 || L == 4, "segment length");
    static_assert(MAINB >= 4, "a group's row spans at least one 32-bit word");
};

__device__ __forceinline__ void sts128(uint32_t a, float x, float y, float z, float w) {
    asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(a), "f"(x), "f"(y), "f"(z), "f"(w)
                 : "memory");
}
__device__ __forceinline__ void lds128_u64(uint32_t a, unsigned long long& p, unsigned long long& q) {
    asm volatile("ld.shared.v2.b64 {%0, %1}, [%2];" : "=l"(p), "=l"(q) : "r"(a));
}
__device__ __forceinline__ unsigned long long lds64_u64(uint32_t a) {
    unsigned long long p;
    asm volatile("ld.shared.b64 %0, [%1];" : "=l"(p) : "r"(a));
    return p;
}
__device__ __forceinline__ void sts64(uint32_t a, float x, float y) {
    asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(a), "f"(x), "f"(y) : "memory");
}

template <typename T, int S, int L, int MODE, bool BWDX>
__global__ void __launch_bounds__(kV2Threads, 1)
stream2_kernel(const __grid_constant__ V2Plan pl) {
    using G_ = V2Geo<T, S, L>;
    constexpr int KK = 9;
    constexpr int ES = G_::ES;
    constexpr int NQ = G_::NQ;
    static_assert(!BWDX || S == 1, "grad-x is stride 1 only");

    extern __shared__ __align__(128) unsigned char smem_raw[];
    const uint32_t sbase = smem_u32(smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int NST = pl.n_slots, NC = pl.n_cslots, NCW = pl.n_compute_warps;
    const int NP = pl.planes_per_pass, PPS = pl.passes_per_stage;
    const int Gn = pl.G;

#define RFULL(s) (sbase + 8u * (uint32_t)(s))
#define REMPTY(s) (sbase + 8u * (uint32_t)(kMaxSlots + (s)))
#define CFULL(c) (sbase + 8u * (uint32_t)(2 * kMaxSlots + (c)))
#define CEMPTY(c) (sbase + 8u * (uint32_t)(2 * kMaxSlots + kV2MaxCSlots + (c)))
    const uint32_t bar_sf_full = sbase + 8u * (2 * kMaxSlots + 2 * kV2MaxCSlots);
    const uint32_t bar_sf_empty = bar_sf_full + 8u;
#define STAGE_BASE(s) (sbase + pl.off_stage0 + (uint32_t)(s) * pl.stage_stride)
#define CSLOT_BASE(c) (sbase + pl.off_conv0 + (uint32_t)(c) * pl.cslot_stride)

    if (tid == 0) {
        for (int s = 0; s < NST; ++s) {
            mbar_init(RFULL(s), 1);
            mbar_init(REMPTY(s), kV2ServiceWarps);
        }
        for (int c = 0; c < NC; ++c) {
            mbar_init(CFULL(c), kV2ServiceWarps);
            mbar_init(CEMPTY(c), (uint32_t)NCW);
        }
        mbar_init(bar_sf_full, 1);
        mbar_init(bar_sf_empty, (uint32_t)NCW);
        mbar_fence_init();
    }
    // Zero rows above and below every converted plane (never overwritten later).
    {
        const int per_plane = NQ * 2 * Gn;  // 16-byte units: NQ quads x {top, bottom} x G
        const int total = NC * NP * per_plane;
        for (int u = tid; u < total; u += blockDim.x) {
            const int plane = u / per_plane;
            const int r = u - plane * per_plane;
            const int q = r / (2 * Gn);
            const int r2 = r - q * 2 * Gn;
            const int bottom = r2 / Gn;
            const int g = r2 - bottom * Gn;
            const int c = plane / NP, pp = plane - c * NP;
            const uint32_t a = CSLOT_BASE(c) + (uint32_t)pp * pl.cplane_bytes + (uint32_t)q * pl.quad_stride +
                               (uint32_t)(((bottom ? pl.H + 1 : 0) * Gn + g) * 16);
            sts128(a, 0.f, 0.f, 0.f, 0.f);
        }
    }
    __syncthreads();

    const long long pass_lo = (pl.total_passes * (long long)blockIdx.x) / gridDim.x;
    const long long pass_hi = (pl.total_passes * (long long)(blockIdx.x + 1)) / gridDim.x;
    const int my_passes = (int)(pass_hi - pass_lo);
    if (my_passes == 0) return;
    const int my_stages = (my_passes + PPS - 1) / PPS;
    const long long plane_lo = pass_lo * NP, plane_hi = pass_hi * NP;
    const int stage_planes = PPS * NP;

    if (warp >= NCW) {
        // ------------------------------------------------------------- service warps
        const int sw = warp - NCW;  // 0: producer + converter, 1, 2: converters
        if (sw >= kV2ServiceWarps) return;
        // producer state (meaningful in service warp 0 only)
        int issue_i = 0, seg_k = 0;
        long long seg_b = plane_lo / pl.C;
        long long seg_plane = plane_lo;
        bool gave_up = false;

        auto producer_poll = [&]() {
            // spatial filter of the next sample
            {
                const int ahead = issue_i + 1 < my_stages ? issue_i + 1 : my_stages;
                long long horizon = plane_lo + (long long)ahead * stage_planes;
                if (horizon > plane_hi) horizon = plane_hi;
                if (seg_plane < horizon &&
                    (seg_k == 0 || warp_test(bar_sf_empty, (uint32_t)((seg_k - 1) & 1), lane))) {
                    if (lane == 0) {
                        const unsigned long long g0 = (unsigned long long)seg_b * pl.sf_bytes;
                        const unsigned long long a0 = g0 & ~15ull;
                        const unsigned long long a1 = (g0 + pl.sf_bytes + 15ull) & ~15ull;
                        mbar_arrive_expect_tx(bar_sf_full, (uint32_t)(a1 - a0));
                        bulk_g2s(sbase + pl.off_sf, (const char*)pl.sf + a0, (uint32_t)(a1 - a0),
                                 bar_sf_full);
                    }
                    ++seg_k;
                    ++seg_b;
                    seg_plane = seg_b * pl.C;
                }
            }
            // raw stages: as many as have a free slot
            while (issue_i < my_stages) {
                const int slot = issue_i % NST;
                if (!(issue_i < NST || warp_test(REMPTY(slot), (uint32_t)((issue_i / NST - 1) & 1), lane)))
                    break;
                const long long st_first = plane_lo + (long long)issue_i * stage_planes;
                long long st_end = st_first + stage_planes;
                if (st_end > plane_hi) st_end = plane_hi;
                if (lane == 0) {
                    const unsigned long long g0 = (unsigned long long)st_first * pl.plane_bytes;
                    const unsigned long long g1 = (unsigned long long)st_end * pl.plane_bytes;
                    const unsigned long long a0 = g0 & ~15ull, a1 = (g1 + 15ull) & ~15ull;
                    const unsigned long long c0 = (unsigned long long)st_first * (KK * ES);
                    const unsigned long long c1 = (unsigned long long)st_end * (KK * ES);
                    const unsigned long long ca0 = c0 & ~15ull, ca1 = (c1 + 15ull) & ~15ull;
                    mbar_arrive_expect_tx(RFULL(slot), (uint32_t)((a1 - a0) + (ca1 - ca0)));
                    bulk_g2s(STAGE_BASE(slot) + 32u, (const char*)pl.in + a0, (uint32_t)(a1 - a0),
                             RFULL(slot));
                    bulk_g2s(STAGE_BASE(slot) + pl.off_rawcf, (const char*)pl.cf + ca0,
                             (uint32_t)(ca1 - ca0), RFULL(slot));
                }
                ++issue_i;
            }
        };
        // Wait that keeps the producer's duties going (service warp 0) and is bounded.
        auto service_wait = [&](uint32_t bar, uint32_t parity) -> bool {
            if (warp_test(bar, parity, lane)) return true;
            const long long t0 = clock64();
            for (;;) {
                if (sw == 0) producer_poll();
                if (warp_test(bar, parity, lane)) return true;
                if (clock64() - t0 > kWaitCycles) return false;
            }
        };

        const int recs_per_plane = pl.H * Gn;
        const int recs_per_pass = NP * recs_per_plane;
        const int lanes_total = 32 * kV2ServiceWarps;
        const int step_g = lanes_total % Gn, step_y = lanes_total / Gn;

        for (int pidx = 0; pidx < my_passes && !gave_up; ++pidx) {
            if (sw == 0) producer_poll();
            const int st = pidx / PPS, q = pidx - st * PPS;
            const int rslot = st % NST, cslot = pidx % NC;
            if (q == 0 && !service_wait(RFULL(rslot), (uint32_t)((st / NST) & 1))) { gave_up = true; break; }
            if (pidx >= NC && !service_wait(CEMPTY(cslot), (uint32_t)((pidx / NC - 1) & 1))) { gave_up = true; break; }

            const unsigned long long st_first_plane =
                (unsigned long long)plane_lo + (unsigned long long)st * stage_planes;
            const uint32_t xoff = (uint32_t)((st_first_plane * pl.plane_bytes) & 15ull);
            const uint32_t raw0 = STAGE_BASE(rslot) + 32u + xoff + (uint32_t)(q * NP) * pl.plane_bytes;
            const uint32_t conv0 = CSLOT_BASE(cslot);

            // channel filters of this pass: (cf, cf) float pairs, 10 pairs (80 bytes) per plane
            if (sw == 0) {
                const uint32_t coff = (uint32_t)((st_first_plane * (KK * ES)) & 15ull);
                const uint32_t src = STAGE_BASE(rslot) + pl.off_rawcf + coff + (uint32_t)(q * NP * KK * ES);
                const uint32_t dst = sbase + pl.off_ccf + (uint32_t)cslot * pl.ccf_stride;
                for (int e = lane; e < NP * KK; e += 32) {
                    float v;
                    if constexpr (ES == 4) v = ldsf(src + 4u * e);
                    else v = Word<T>::get(lds16(src + 2u * e), 0);
                    const int plane = e / KK, t = e - plane * KK;
                    sts64(dst + (uint32_t)(plane * 80 + t * 8), v, v);
                }
            }

            // records of this pass, strided over the 96 service lanes
            int r = sw * 32 + lane;
            int ppl = r / recs_per_plane;
            int rem = r - ppl * recs_per_plane;
            int yy = rem / Gn, g = rem - yy * Gn;
            for (; r < recs_per_pass; r += lanes_total) {
                const uint32_t src = raw0 + (uint32_t)ppl * pl.plane_bytes +
                                     (uint32_t)((yy * pl.W + G_::MAINN * g) * ES);
                float val[G_::NV];
                // left halo element, main vector, right halo element
                {
                    float lh;
                    if constexpr (ES == 4) lh = ldsf(src - 4u);
                    else lh = Word<T>::get(lds16(src - 2u), 0);
                    val[0] = g > 0 ? lh : 0.f;
                    uint32_t mw[G_::MAINB / 4];
                    lds_vec<G_::MAINB>(src, mw);
#pragma unroll
                    for (int e = 0; e < G_::MAINN; ++e) val[1 + e] = Word<T>::get(mw[e / G_::EPW], e % G_::EPW);
                    if constexpr (G_::RIGHT_HALO) {
                        float rh;
                        if constexpr (ES == 4) rh = ldsf(src + G_::MAINB);
                        else rh = Word<T>::get(lds16(src + G_::MAINB), 0);
                        val[1 + G_::MAINN] = g + 1 < Gn ? rh : 0.f;
                    }
                }
                const uint32_t dst = conv0 + (uint32_t)ppl * pl.cplane_bytes + (uint32_t)(((yy + 1) * Gn + g) * 16);
#pragma unroll
                for (int qd = 0; qd < NQ; ++qd) {
                    const int m0 = 2 * qd, m1 = 2 * qd + 1;
                    const float a0 = val[m0], b0 = val[S * L + m0];
                    const float a1 = m1 < G_::NPR ? val[m1 < G_::NPR ? m1 : 0] : 0.f;
                    const float b1 = m1 < G_::NPR ? val[m1 < G_::NPR ? S * L + m1 : 0] : 0.f;
                    sts128(dst + (uint32_t)qd * pl.quad_stride, a0, b0, a1, b1);
                }
                // advance (ppl, yy, g) by 96 records
                g += step_g;
                yy += step_y;
                if (g >= Gn) { g -= Gn; ++yy; }
                while (yy >= pl.H) { yy -= pl.H; ++ppl; }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(CFULL(cslot));
            // last pass of the raw stage: this warp is done reading it
            if (q == PPS - 1 || pidx == my_passes - 1) {
                if (lane == 0) mbar_arrive(REMPTY(rslot));
            }
        }
        if (sw == 0 && !gave_up) {
            // spatial filters of samples that start after the last conversion was queued
            const long long t0 = clock64();
            while (seg_plane < plane_hi) {
                producer_poll();
                if (clock64() - t0 > kWaitCycles) { gave_up = true; break; }
            }
        }
        if (gave_up) {
            if (lane == 0) atomicCAS(pl.fault, 0, (int)kFaultService);
            if (sw == 0) {
                bool drained = true;
                const int first = issue_i > NST ? issue_i - NST : 0;
                for (int j = first; j < issue_i; ++j)
                    drained &= mbar_wait(RFULL(j % NST), (uint32_t)((j / NST) & 1));
                if (seg_k > 0) drained &= mbar_wait(bar_sf_full, (uint32_t)((seg_k - 1) & 1));
                if (!drained && lane == 0) atomicExch(pl.fault, (int)kFaultDrain);
            }
        }
        return;
    }

    // ----------------------------------------------------------------- compute warps
    const int TP = pl.tasks_per_plane;
    int pip = tid / TP;
    int task = tid - pip * TP;
    const bool active = pip < NP;
    if (!active) { pip = 0; task = 0; }
    const int oy = task / Gn;
    const int g = task - oy * Gn;

    // byte offsets of this thread's three converted rows (quad 0) inside a converted plane
    uint32_t rowoff[3];
#pragma unroll
    for (int i = 0; i < 3; ++i) rowoff[i] = (uint32_t)(((S * oy + i) * Gn + g) * 16);

    unsigned long long sf2[KK][L];
#pragma unroll
    for (int t = 0; t < KK; ++t)
#pragma unroll
        for (int k = 0; k < L; ++k) sf2[t][k] = 0ull;

    long long b = plane_lo / pl.C;
    int c_in_b = (int)(plane_lo - b * pl.C);
    bool need_sf = true;
    int seg = 0;
    const long long out_plane = (long long)pl.OH * pl.OW;
    T* outp = reinterpret_cast<T*>(pl.out) + (plane_lo + pip) * out_plane + (long long)oy * pl.OW + g * (2 * L);
    const long long out_step = (long long)NP * out_plane;

    for (int pidx = 0; pidx < my_passes; ++pidx) {
        const int cslot = pidx % NC;
        if (need_sf) {
            if (!mbar_wait(bar_sf_full, (uint32_t)(seg & 1))) {
                atomicCAS(pl.fault, 0, (int)kFaultConsumerSf);
                return;
            }
            const uint32_t sfs = sbase + pl.off_sf + (uint32_t)(((unsigned long long)b * pl.sf_bytes) & 15ull);
            if constexpr (!BWDX) {
#pragma unroll
                for (int t = 0; t < KK; ++t) {
                    const uint32_t a = sfs + (uint32_t)(((t * pl.OH + oy) * pl.OW + g * (2 * L)) * ES);
                    uint32_t w[G_::OUTB / 4];
                    lds_vec<G_::OUTB>(a, w);
#pragma unroll
                    for (int k = 0; k < L; ++k)
                        sf2[t][k] = f2_pack(Word<T>::get(w[k / G_::EPW], k % G_::EPW),
                                            Word<T>::get(w[(L + k) / G_::EPW], (L + k) % G_::EPW));
                }
            } else {
#pragma unroll
                for (int i = 0; i < 3; ++i) {
#pragma unroll
                    for (int j = 0; j < 3; ++j) {
                        const int ft = KK - 1 - (i * 3 + j);
                        const int yy = oy + i - 1;
#pragma unroll
                        for (int k = 0; k < L; ++k) {
                            float v[2];
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                const int xx = g * (2 * L) + h * L + k + j - 1;
                                v[h] = 0.f;
                                if (yy >= 0 && yy < pl.OH && xx >= 0 && xx < pl.OW) {
                                    const uint32_t a = sfs + (uint32_t)(((ft * pl.OH + yy) * pl.OW + xx) * ES);
                                    if constexpr (ES == 4) v[h] = ldsf(a);
                                    else v[h] = Word<T>::get(lds16(a), 0);
                                }
                            }
                            sf2[i * 3 + j][k] = f2_pack(v[0], v[1]);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_sf_empty);
            ++seg;
            need_sf = false;
        }

        if (!mbar_wait(CFULL(cslot), (uint32_t)((pidx / NC) & 1))) {
            atomicCAS(pl.fault, 0, (int)kFaultConsumerFull);
            return;
        }
        const uint32_t cplane = CSLOT_BASE(cslot) + (uint32_t)pip * pl.cplane_bytes;
        const uint32_t ccf = sbase + pl.off_ccf + (uint32_t)cslot * pl.ccf_stride + (uint32_t)pip * 80u;

        unsigned long long acc2[L];
#pragma unroll
        for (int k = 0; k < L; ++k) acc2[k] = 0ull;

#pragma unroll
        for (int i = 0; i < 3; ++i) {
            unsigned long long pr[2 * NQ];
#pragma unroll
            for (int qd = 0; qd < NQ; ++qd)
                lds128_u64(cplane + (uint32_t)qd * pl.quad_stride + rowoff[i], pr[2 * qd], pr[2 * qd + 1]);
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                const int t = i * 3 + j;
                const unsigned long long c2 = lds64_u64(ccf + (uint32_t)((BWDX ? KK - 1 - t : t) * 8));
#pragma unroll
                for (int k = 0; k < L; ++k) {
                    const unsigned long long w2 =
                        MODE == DDF_B200_MUL ? f2_mul(c2, sf2[t][k]) : f2_add(c2, sf2[t][k]);
                    acc2[k] = f2_fma(w2, pr[S * k + j], acc2[k]);
                }
            }
        }
        if (active) {
            float o[2 * L];
#pragma unroll
            for (int k = 0; k < L; ++k) f2_unpack(acc2[k], o[k], o[L + k]);
            store_out<T, 2 * L>(outp, o);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(CEMPTY(cslot));

        outp += out_step;
        c_in_b += NP;
        if (c_in_b >= pl.C) {
            c_in_b = 0;
            ++b;
            need_sf = true;
        }
    }
#undef RFULL
#undef REMPTY
#undef CFULL
#undef CEMPTY
#undef STAGE_BASE
#undef CSLOT_BASE
}

// ------------------------------------------------------------------------ host side
template <typename T, int S, int L>
bool make_v2_plan(const StreamArgs& a, V2Plan& pl, uint32_t& smem_bytes, int& grid) {
    using G_ = V2Geo<T, S, L>;
    const Problem& p = a.p;
    if (p.k != 3 || p.d != 1 || p.s != S) return false;
    if (a.bwdx && S != 1) return false;
    const int H = a.bwdx ? p.OH : p.H, W = a.bwdx ? p.OW : p.W;
    const int OH = p.OH, OW = p.OW;
    if (OW % (2 * L) != 0 || W != OW * S) return false;
    if (S == 2 && H != OH * 2) return false;  // odd heights: first-generation kernel
    const int Gn = OW / (2 * L);
    const int TP = OH * Gn;
    if (TP < 1 || TP > kV2MaxComputeThreads) return false;
    int NP = kV2MaxComputeThreads / TP;
    while (NP > 1 && p.C % NP != 0) --NP;
    const long long planes = (long long)p.B * p.C;
    const uint32_t plane_bytes = (uint32_t)(H * W * G_::ES);
    const uint32_t sf_bytes = (uint32_t)(9 * OH * OW * G_::ES);
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    if (!al16(a.in) || !al16(a.cf) || !al16(a.sf) || !al16(a.out)) return false;
    if ((planes * plane_bytes) % 16 != 0) return false;
    if ((planes * 9 * G_::ES) % 16 != 0) return false;
    if (((long long)p.B * sf_bytes) % 16 != 0) return false;

    const long long total_passes = planes / NP;
    int PPS = (int)(12288u / ((uint32_t)NP * plane_bytes));
    if (PPS < 1) PPS = 1;
    const long long share = (total_passes + a.sm_count - 1) / a.sm_count;
    if (PPS > share) PPS = (int)share;
    if (PPS < 1) PPS = 1;
    const int SPL = PPS * NP;

    pl.quad_stride = (uint32_t)((H + 2) * Gn * 16);
    pl.cplane_bytes = (uint32_t)G_::NQ * pl.quad_stride;
    pl.cslot_stride = round_up((uint32_t)NP * pl.cplane_bytes, 128);
    pl.ccf_stride = round_up((uint32_t)NP * 80u, 16);
    const uint32_t x_region = 32u + (uint32_t)SPL * plane_bytes + 16u + 32u;
    pl.off_rawcf = round_up(x_region, 16);
    pl.stage_stride = round_up(pl.off_rawcf + (uint32_t)SPL * 9 * G_::ES + 32u, 128);
    const uint32_t sf_region = round_up(sf_bytes + 32u, 128);

    // converted ring: 3 slots if they fit beside at least 3 raw stages, else 2
    int nc = 4, ns = 0;
    for (; nc >= 2; --nc) {
        const uint32_t fixed = 512u + round_up((uint32_t)nc * pl.ccf_stride, 128) + sf_region +
                               (uint32_t)nc * pl.cslot_stride;
        if (fixed >= kSmemBudget) continue;
        ns = (int)((kSmemBudget - fixed) / pl.stage_stride);
        if (ns >= 3 || nc == 2) break;
    }
    if (nc < 2 || ns < 2) return false;
    if (ns > 12) ns = 12;
    pl.n_cslots = nc;
    pl.n_slots = ns;
    pl.off_ccf = 512;
    pl.off_sf = round_up(pl.off_ccf + (uint32_t)nc * pl.ccf_stride, 128);
    pl.off_conv0 = pl.off_sf + sf_region;
    pl.off_stage0 = pl.off_conv0 + (uint32_t)nc * pl.cslot_stride;
    smem_bytes = pl.off_stage0 + (uint32_t)ns * pl.stage_stride;
    if (smem_bytes > kSmemBudget) return false;

    pl.in = a.in; pl.cf = a.cf; pl.sf = a.sf; pl.out = a.out;
    pl.C = p.C; pl.H = H; pl.W = W; pl.OH = OH; pl.OW = OW;
    pl.G = Gn;
    pl.tasks_per_plane = TP;
    pl.planes_per_pass = NP;
    pl.passes_per_stage = PPS;
    pl.n_compute_warps = (NP * TP + 31) / 32;
    pl.total_passes = total_passes;
    pl.plane_bytes = plane_bytes;
    pl.sf_bytes = sf_bytes;
    pl.fault = a.fault;
    grid = (int)(total_passes < a.sm_count ? total_passes : a.sm_count);
    return true;
}

template <typename T, int S, int L, int MODE, bool BWDX>
int stream2_launch(const StreamArgs& a, cudaStream_t stream) {
    V2Plan pl;
    uint32_t smem = 0;
    int grid = 0;
    if (!make_v2_plan<T, S, L>(a, pl, smem, grid)) return kNotHandled;
    auto kern = stream2_kernel<T, S, L, MODE, BWDX>;
    static std::atomic<unsigned long long> opted_in{0};
    const unsigned long long bit = 1ull << (a.device & 63);
    if (!(opted_in.load(std::memory_order_acquire) & bit)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)kSmemBudget);
        if (e != cudaSuccess) return (int)e;
        opted_in.fetch_or(bit, std::memory_order_release);
    }
    const int threads = (pl.n_compute_warps + kV2ServiceWarps) * 32;
    kern<<<grid, threads, smem, stream>>>(pl);
    return (int)cudaGetLastError();
}

// Largest segment length whose pixel groups tile the output row.  0 = not covered.
inline int v2_segment(const Problem& p, bool bwdx) {
    if (p.k != 3 || p.d != 1 || (p.s != 1 && p.s != 2) || p.dtype == DDF_B200_F64) return 0;
    if (bwdx && p.s != 1) return 0;
    if (p.W != p.OW * p.s || (p.s == 2 && p.H != p.OH * 2)) return 0;
    static const int cand[3] = {4, 2, 1};
    for (int ci = 0; ci < 3; ++ci) {
        const int L = cand[ci];
        if (p.s == 2 && L == 4) continue;  // not instantiated
        if (p.OW % (2 * L) != 0) continue;
        const long long tp = (long long)p.OH * (p.OW / (2 * L));
        if (tp > kV2MaxComputeThreads) continue;
        return L;
    }
    return 0;
}

template <typename T>
int stream2_dispatch(const StreamArgs& a, cudaStream_t stream);

}  // namespace ddf
