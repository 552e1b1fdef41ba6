// gemv.cu — single-row W4A8 GEMV (decode, one token) for sm_100a.
//
// Replaces x_gemv_w4a8_core and x_gemv_w4a8_fanout (xpu/src/kernels_dpas.cpp:586-675,
// 945-1102). HBM-bound: the packed weight stream (256 B per 16-row x K32 tile plus a
// 32 B scale line) is read exactly once; activations (40 B per k-tile) come from L2.
//
// Mapping. One warp owns one (row-group, K-split) task at a time, as the reference's
// sub-group does. Split weights launch one CTA of S warps per row-group (the hardware places
// them as SMs free up); unsplit ones and the fused-quantiser form run persistent 16-warp
// CTAs, two per SM. A 256-byte tile is 16 rows x 16 B, so a HALF-warp reads one tile with
// one 128-bit load per lane and the two halves of a warp walk the even and the odd tiles of
// the split. That is exactly the reference's two-accumulator order (acc0 takes the even
// offsets from kt_begin, acc1 the odd ones, leftover to acc0), so each lane keeps ONE
// accumulator and acc0+acc1 is a single shuffle. The fan-out order and the K16 tier (one
// serial accumulator) pass the odd half's product terms to the even half every pair.
// Weights, their scale lines and the matching activations reach the tile loop through
// per-warp cp.async rings in shared memory (see the kernel).
//
// Unpack. A row's 16 bytes hold k = 2b (low nibble) and 2b+1 (high nibble). Masking
// gives the even-k and the odd-k codes of a word as four bytes each; xor 8 turns a
// two's-complement nibble q into q+8 in [0,15], so dp4a against the matching
// activation bytes yields d + 8*asum and the exact int32 dot is recovered inside the
// zero-point term: d - z*asum == d' - (z+8)*asum. The activation scratch is stored
// already split into even-k / odd-k halves per tile.
#include "stream.cuh"

#include <algorithm>

namespace tq {

namespace {

constexpr int kW = 16;    // most warps per CTA (a launch may use fewer: blockDim.x / 32)
constexpr int kST = 8;    // tiles per ring stage
// Stage layout: codes (256 B per tile), scale lines (32 B per tile; 64 B in the K16 tier: one
// line per half tile), and - unless the kernel quantised the row itself - the tiles'
// activations: 32 bytes of codes (even-k half, odd-k half) per tile, the int32 code sums (one
// per tile; the two K16 half sums in the K16 tier), the fp32 scales.
struct StageLayout {
    int scales, act_codes, act_sums, act_scales, bytes;
};
__host__ __device__ constexpr StageLayout stage_layout(bool fuseq, bool k16) {
    const int scales = kST * 256;
    const int act_codes = scales + kST * (k16 ? 64 : 32);
    const int act_sums = act_codes + kST * 32;
    const int act_scales = act_sums + kST * (k16 ? 8 : 4);
    return StageLayout{scales, act_codes, act_sums, act_scales,
                       fuseq ? act_codes : act_scales + kST * 4};
}
__host__ __device__ constexpr int stage_bytes(bool fuseq, bool k16 = false) {
    return stage_layout(fuseq, k16).bytes;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}

// High nibbles in place: ((w & 0xF0F0F0F0) ^ 0x80808080) = four unsigned bytes 16 * (q + 8).
__device__ __forceinline__ uint32_t nib_hi_plus8_x16(uint32_t w) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(d) : "r"(w), "r"(0xF0F0F0F0u), "r"(0x80808080u));
    return d;
}
__device__ __forceinline__ int dp4a_u8s8(uint32_t ua, uint32_t sb, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(ua), "r"(sb), "r"(c));
    return d;
}

// sum over the tile row of (q + 8) * a. The odd-k codes stay in the high nibbles and are
// multiplied as 16 * (q + 8): that accumulator is an exact multiple of 16.
__device__ __forceinline__ int tile_dot_plus8(const uint4 &w, const uint4 &e, const uint4 &o) {
    int dlo = 0, dhi = 0;
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
    const uint32_t ee[4] = {e.x, e.y, e.z, e.w};
    const uint32_t oo[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        dlo = __dp4a((int)nib_plus8(ww[j]), (int)ee[j], dlo);
        dhi = dp4a_u8s8(nib_hi_plus8_x16(ww[j]), oo[j], dhi);
    }
    return dlo + (dhi >> 4);
}

// Persistent kernel: a team of S warps owns one 16-row group at a time (warp s = K-split
// s), walks the row-groups team, team + teams, ... and adds its partial sums in split order
// through shared memory behind a named barrier.
// Every warp streams its tiles through a private ring of NS shared-memory stages (kST tiles,
// their scale lines and - from the prepared scratch, which stays in L2 - the matching
// activation codes, sums and scales) filled with cp.async, so that NS-1 stages per warp are
// in flight while one is consumed and no load of the tile loop leaves the SM; the ring keeps
// running across the warp's units. In a stage the two half-warps take the even and the odd tiles (one 128-bit
// shared-memory load per lane = one row of a tile).
// FUSEQ: the fp32 activation row is quantised by every CTA into shared memory (the same
// per-block rule and code as quant_s8_kernel) after the wait on earlier kernels, instead of
// being read from the prepared scratch; CTA 0 also writes the scratch.
// K16: the K16 scale tier (x_gemv_w4a8_core_k16, xpu/src/kernels_dpas.cpp:683-767): two scale
// lines per tile, each half dot promoted with its own scale and K16 sum, and ONE accumulator
// per split (the halves of a warp pass their terms along as in the fan-out order).
template <bool SERIAL, bool DUMP, bool FUSEQ, int NS, bool K16 = false>
__global__ void __launch_bounds__(kW * 32, 2) gemv_w4a8_kernel(const GemvArgs a) {
    __shared__ float part[kW * 16];
    // ring[warps][NS][kStageBytes], then (FUSEQ) qp[K], as[K/32], sum32[K/32]
    const int nw = blockDim.x >> 5;
    constexpr StageLayout L = stage_layout(FUSEQ, K16);
    constexpr int kStageBytes = L.bytes;
    constexpr int kActCodes = L.act_codes, kActSums = L.act_sums, kActScales = L.act_scales;
    constexpr bool ORDERED = SERIAL || K16;      // one accumulator, terms added in tile order
    extern __shared__ __align__(16) unsigned char dyn[];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int h = lane >> 4;
    const int n = lane & 15;
    const int S = a.splits;
    const int tpc = nw / S;                            // teams per CTA
    const int team = warp / S;
    const int split = warp - team * S;
    const int g0 = blockIdx.x + gridDim.x * team;
    const int teams = gridDim.x * tpc;                 // row-group stride of this warp
    const int Kt = a.K >> 5;
    const int Ktg = Kt >> a.ksh;
    const int groups = a.goff[a.count];
    const int kt_begin = Kt * split / S;
    const int cnt = Kt * (split + 1) / S - kt_begin;
    unsigned char *ring = dyn + (size_t)warp * NS * kStageBytes;
    const uint32_t ring_s = smem_u32(ring);
    const uint64_t pol = l2_policy_evict_first();

    // Producer side of the ring: the next (row-group, tile offset) to fetch. The source
    // pointers of the row-group are kept per lane and only move by a stage per call.
    int pg = g0, pi0 = 0;
    uint32_t pdst = ring_s;
    const uint8_t *psrc = nullptr;        // this lane's first 16-byte piece of the next stage
    const uint16_t *pscl = nullptr;       // scale line 0 of the row-group, this lane's half
    auto producer_group = [&]() {
        if (pg < groups) {
            int wi = 0;
            while (wi + 1 < a.count && pg >= a.goff[wi + 1]) ++wi;
            const int lg = pg - a.goff[wi];
            psrc = a.codes[wi] + ((size_t)lg * Kt + kt_begin) * 256u + lane * 16;
            // K16: two 32-byte lines per tile, lane l copies piece l of the stage's 8 x 64 bytes
            pscl = K16 ? a.scales[wi] + (size_t)lg * (Kt * 2) * 16u + lane * 8
                       : a.scales[wi] + (size_t)lg * Ktg * 16u + (lane & 1) * 8;
        }
    };
    producer_group();
    // One stage = the weight part (codes and scale lines: may be fetched before the wait on
    // earlier kernels) and finish_stage (activations from the prepared scratch, which an
    // earlier kernel wrote; then the stage is committed and the producer moves on).
    auto issue_weights = [&]() {
        if (pg < groups && cnt > 0) {
            const int left = cnt - pi0;
            const uint16_t *sl =
                K16 ? pscl + (size_t)(kt_begin + pi0) * 32u
                    : pscl + (size_t)((kt_begin + pi0 + (lane >> 1)) >> a.ksh) * 16u;
            constexpr int kPieces = K16 ? 4 : 2;      // 16-byte scale pieces per tile
            if (left >= kST) {
#pragma unroll
                for (int p = 0; p < kST / 2; ++p)
                    cp_async16(pdst + lane * 16 + p * 512, psrc + p * 512, pol);
                if (lane < kPieces * kST) cp_async16(pdst + kST * 256 + lane * 16, sl, pol);
            } else {
#pragma unroll
                for (int p = 0; p < kST / 2; ++p)
                    if (lane + 32 * p < left * 16)
                        cp_async16(pdst + lane * 16 + p * 512, psrc + p * 512, pol);
                if (lane < kPieces * left) cp_async16(pdst + kST * 256 + lane * 16, sl, pol);
            }
        }
    };
    auto finish_stage = [&]() {
        if (pg < groups && cnt > 0) {
            if (!FUSEQ) {
                const int nt = min(kST, cnt - pi0);
                const int kt0 = kt_begin + pi0;
                if (lane < 16) {
                    // codes of tile lane/2, half lane%2
                    if (lane < 2 * nt)
                        cp_async16_plain(pdst + kActCodes + lane * 16, a.qp + (size_t)kt0 * 32 + lane * 16);
                } else if (K16) {
                    // lanes 16..31: the two K16 sums of tile (lane - 16) / 2
                    if (lane - 16 < 2 * nt)
                        cp_async4(pdst + kActSums + (lane - 16) * 4, a.sum16 + 2 * kt0 + (lane - 16));
                } else if ((lane & 7) < nt) {
                    // lanes 16..23: int32 sums, lanes 24..31: scales (adjacent in the stage)
                    const void *src = lane < 24 ? static_cast<const void *>(a.sum32 + kt0 + (lane - 16))
                                                : static_cast<const void *>(a.as + kt0 + (lane - 24));
                    cp_async4(pdst + kActSums + (lane - 16) * 4, src);
                }
                if (K16 && lane < nt) cp_async4(pdst + kActScales + lane * 4, a.as + kt0 + lane);
            }
            pi0 += kST;
            psrc += kST * 256;
            if (pi0 >= cnt) {
                pi0 = 0;
                pg += teams;
                producer_group();
            }
            pdst = (pdst + kStageBytes == ring_s + NS * kStageBytes) ? ring_s : pdst + kStageBytes;
        }
        cp_async_commit();
    };

    pdl_trigger();
    // Weights do not depend on earlier kernels: the ring starts filling before the wait.
    if (FUSEQ) {
#pragma unroll
        for (int i = 0; i < NS - 1; ++i) {
            issue_weights();
            finish_stage();
        }
        pdl_wait();
    } else {
        issue_weights();          // the first stage's weights cross the wait
        pdl_wait();
        finish_stage();
#pragma unroll
        for (int i = 1; i < NS - 1; ++i) {
            issue_weights();
            finish_stage();
        }
    }

    uint32_t fq_codes = 0, fq_scales = 0, fq_sums = 0;   // FUSEQ: the CTA's quantised row
    if (FUSEQ) {
        unsigned char *qbase = dyn + (size_t)nw * NS * kStageBytes;
        int8_t *sqp = reinterpret_cast<int8_t *>(qbase);
        float *sas = reinterpret_cast<float *>(qbase + a.K);
        int32_t *ssum = reinterpret_cast<int32_t *>(qbase + a.K + (size_t)Kt * 4);
        const bool scribe = blockIdx.x == 0;     // keeps the library's prepared scratch current
        for (int b = warp; b < Kt; b += nw) {
            const float v = a.x[b * 32 + lane];
            const float mx = warp_max(fabsf(v));
            const float sc = (mx > 0.0f) ? __fdiv_rn(mx, 127.0f) : 1.0f;
            const int qv = quantise_one(v, sc);
            const int hs = half_sum16(qv);
            const int other = __shfl_xor_sync(0xffffffffu, hs, 16);
            sqp[b * 32 + permuted_pos(lane)] = (int8_t)qv;
            if (lane == 0) {
                sas[b] = sc;
                ssum[b] = hs + other;
            }
            if (scribe) {
                a.sq[b * 32 + lane] = (int8_t)qv;
                a.sqp[b * 32 + permuted_pos(lane)] = (int8_t)qv;
                if ((lane & 15) == 0) a.ssum16[b * 2 + (lane >> 4)] = hs;
                if (lane == 0) {
                    a.sscale[b] = sc;
                    a.ssum32[b] = hs + other;
                }
            }
        }
        __syncthreads();
        fq_codes = smem_u32(sqp);
        fq_scales = smem_u32(sas);
        fq_sums = smem_u32(ssum);
    }

    // Consumer side. One stage: the half-warp h takes tiles h, h + 2, ... of the stage. A
    // pair step handles tile 2u + h on both half-warps; its shared-memory addresses are
    // constant offsets from the per-stage bases.
    uint32_t cst = ring_s;
    const uint32_t lane_w = h * 256 + n * 16;              // this lane's row in tile h
    const uint32_t lane_s = kST * 256 + h * (K16 ? 64 : 32) + n * 2;    // and its scale word
    // ea: even-k codes of the tile (odd-k at +16); sa / fa_: its int32 sum and fp32 scale
    auto pair_step = [&](uint32_t wl, uint32_t sl, uint32_t ea, uint32_t sa, uint32_t fa_,
                         int32_t *dmp, bool valid, bool odd_valid, float &acc) {
        float fa = 0.0f, fb = 0.0f, fa2 = 0.0f;      // fa2: the high half's term (K16)
        if (valid) {
            const uint4 wv = lds_v4(wl);
            const uint32_t sc = lds_u16(sl);
            const uint4 e = lds_v4(ea);
            const uint4 o = lds_v4(ea + 16);
            const int asum = (int)lds_u32(sa);
            fb = __uint_as_float(lds_u32(fa_));
            int zp;
            float ws;
            unpack_scale(sc, zp, ws);
            if (K16) {
                // k 0..15 = words x, y; k 16..31 = words z, w: each half has its own scale
                // line (the second one 32 bytes on) and its own K16 sum (4 bytes on)
                int lo = __dp4a((int)nib_plus8(wv.x), (int)e.x, 0);
                lo = __dp4a((int)nib_plus8(wv.y), (int)e.y, lo);
                int hi = dp4a_u8s8(nib_hi_plus8_x16(wv.x), o.x, 0);
                hi = dp4a_u8s8(nib_hi_plus8_x16(wv.y), o.y, hi);
                const float f = (float)(lo + (hi >> 4) - (zp + 8) * asum);
                fa = __fmul_rn(f, ws);
                int lo2 = __dp4a((int)nib_plus8(wv.z), (int)e.z, 0);
                lo2 = __dp4a((int)nib_plus8(wv.w), (int)e.w, lo2);
                int hi2 = dp4a_u8s8(nib_hi_plus8_x16(wv.z), o.z, 0);
                hi2 = dp4a_u8s8(nib_hi_plus8_x16(wv.w), o.w, hi2);
                int zp2;
                float ws2;
                unpack_scale(lds_u16(sl + 32), zp2, ws2);
                const int asum2 = (int)lds_u32(sa + 4);
                const float f2 = (float)(lo2 + (hi2 >> 4) - (zp2 + 8) * asum2);
                fa2 = __fmul_rn(f2, ws2);
            } else {
                const int dp = tile_dot_plus8(wv, e, o);
                if (DUMP) *dmp = dp - 8 * asum;
                const float f = (float)(dp - (zp + 8) * asum);
                fa = __fmul_rn(f, ws);
            }
        }
        if (!ORDERED) {
            if (valid) acc = fmaf(fa, fb, acc);
        } else {
            // pair (even tile on h == 0, odd tile on h == 1), added in tile order
            const float oa = __shfl_down_sync(0xffffffffu, fa, 16);
            const float ob = __shfl_down_sync(0xffffffffu, fb, 16);
            const float oa2 = K16 ? __shfl_down_sync(0xffffffffu, fa2, 16) : 0.0f;
            if (h == 0) {
                if (valid) {
                    acc = fmaf(fa, fb, acc);
                    if (K16) acc = fmaf(fa2, fb, acc);
                }
                if (odd_valid) {
                    acc = fmaf(oa, ob, acc);
                    if (K16) acc = fmaf(oa2, ob, acc);
                }
            }
        }
    };

    for (int g = g0; g < groups; g += teams) {
        int wi = 0;
        while (wi + 1 < a.count && g >= a.goff[wi + 1]) ++wi;
        const int lg = g - a.goff[wi];
        // FUSEQ: activations of tile kt_begin + h in the CTA's arrays; they move with the stages
        uint32_t fe = fq_codes + (kt_begin + h) * 32, fs = fq_sums + (kt_begin + h) * 4,
                 ff = fq_scales + (kt_begin + h) * 4;
        int32_t *dmp = DUMP ? a.dump + ((size_t)g * Kt + kt_begin + h) * 16 + n : nullptr;

        float acc = 0.0f;
        for (int left = cnt; left > 0; left -= kST) {
            cp_async_wait<NS - 2>();
            __syncwarp();                 // the stage is complete; the slot read last is free
            issue_weights();
            finish_stage();
            const uint32_t wl = cst + lane_w, sl = cst + lane_s;
            constexpr int kSclPair = K16 ? 128 : 64, kSumPair = K16 ? 16 : 8;   // per tile pair
            // activations of tile h of this stage, and the distance between tile pairs
            const uint32_t ea = FUSEQ ? fe : cst + kActCodes + h * 32;
            const uint32_t sa = FUSEQ ? fs : cst + kActSums + h * (K16 ? 8 : 4);
            const uint32_t fa_ = FUSEQ ? ff : cst + kActScales + h * 4;
            if (left >= kST) {
#pragma unroll
                for (int u = 0; u < kST / 2; ++u)
                    pair_step(wl + u * 512, sl + u * kSclPair, ea + u * 64, sa + u * kSumPair, fa_ + u * 8,
                              DUMP ? dmp + u * 32 : nullptr, true, true, acc);
            } else {
                // last, short stage of the split: the same steps behind warp-uniform tests,
                // only the last pair can be half
#pragma unroll
                for (int u = 0; u < kST / 2; ++u)
                    if (2 * u < left)
                        pair_step(wl + u * 512, sl + u * kSclPair, ea + u * 64, sa + u * kSumPair, fa_ + u * 8,
                                  DUMP ? dmp + u * 32 : nullptr, 2 * u + h < left, 2 * u + 1 < left,
                                  acc);
            }
            cst = (cst + kStageBytes == ring_s + NS * kStageBytes) ? ring_s : cst + kStageBytes;
            fe += kST * 32;
            fs += kST * 4;
            ff += kST * 4;
            if (DUMP) dmp += kST * 16;
        }
        if (DUMP) continue;
        if (!ORDERED) acc = __fadd_rn(acc, __shfl_down_sync(0xffffffffu, acc, 16));

        const int row = lg * 16 + n;
        if (S == 1) {
            // unsplit: the accumulator is stored as is; a residual is a separate add
            if (h == 0) a.y[wi][row] = a.residual ? __fadd_rn(acc, a.residual[row]) : acc;
            continue;
        }
        if (h == 0) part[warp * 16 + n] = acc;
        named_bar_sync(1 + team, S * 32);
        if (split == 0 && h == 0) {
            float sum = 0.0f;
            for (int i = 0; i < S; ++i) sum = __fadd_rn(sum, part[(warp + i) * 16 + n]);
            if (SERIAL)
                a.y[wi][row] = sum;
            else
                a.y[wi][row] = __fadd_rn(sum, a.residual ? a.residual[row] : 0.0f);
        }
        named_bar_sync(1 + team, S * 32);     // part is rewritten by the next row-group
    }
}

int g_sms = 0;

}  // namespace

void launch_gemv(const GemvArgs &a) {
    const int groups = a.goff[a.count];
    if (groups <= 0 || a.splits <= 0) return;
    if (!g_sms) {
        int dev = 0;
        TQ_CHECK(cudaGetDevice(&dev));
        TQ_CHECK(cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev));
        if (g_sms <= 0) g_sms = 148;
    }
    if (a.splits > kW || (kW % a.splits)) {
        fprintf(stderr, "launch_gemv: %d splits do not divide the %d warps of a CTA\n", a.splits, kW);
        note_error(cudaErrorInvalidValue, "launch_gemv");
        return;
    }
    const int tpc = kW / a.splits;
    const int grid = std::min(2 * g_sms, (groups + tpc - 1) / tpc);
    // prepared path: two stages that carry their activations; fused quantiser: the CTA's
    // quantised row sits beside the rings, three stages when that fits two CTAs per SM
    constexpr size_t kRingP = (size_t)kW * 2 * stage_bytes(false);
    constexpr size_t kRingF3 = (size_t)kW * 3 * stage_bytes(true), kRingF2 = (size_t)kW * 2 * stage_bytes(true);
    constexpr size_t kPerCta = (227 * 1024) / 2 - 1024 - kW * 16 * 4;   // two CTAs per SM
    static_assert(kRingP <= kPerCta, "ring too large for two CTAs per SM");
    const size_t qbytes = (size_t)a.K + (size_t)(a.K / 32) * 8;
    static bool attr = false;
    if (!attr) {
        TQ_CHECK(cudaFuncSetAttribute(gemv_w4a8_kernel<false, true, false, 2>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRingP));
        TQ_CHECK(cudaFuncSetAttribute(gemv_w4a8_kernel<true, false, false, 2>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRingP));
        TQ_CHECK(cudaFuncSetAttribute(gemv_w4a8_kernel<false, false, false, 2>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRingP));
        TQ_CHECK(cudaFuncSetAttribute(gemv_w4a8_kernel<false, false, false, 3>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)((size_t)kW * 3 * stage_bytes(false))));
        TQ_CHECK(cudaFuncSetAttribute(gemv_w4a8_kernel<false, false, true, 3>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPerCta));
        TQ_CHECK(cudaFuncSetAttribute(gemv_w4a8_kernel<false, false, true, 2>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPerCta));
        attr = true;
    }
    if (a.k16 && !a.dump) {
        // K16 tier: prepared activations only (a fused-quantiser call prepares first)
        constexpr size_t kRingK16 = (size_t)kW * 2 * stage_bytes(false, true);
        static_assert(kRingK16 <= kPerCta, "K16 ring too large for two CTAs per SM");
        static bool attr16 = false;
        if (!attr16) {
            TQ_CHECK(cudaFuncSetAttribute(gemv_w4a8_kernel<false, false, false, 2, true>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRingK16));
            attr16 = true;
        }
        if (a.splits >= 4)      // one row-group per CTA, as for the other tiers below
            launch_pdl(gemv_w4a8_kernel<false, false, false, 2, true>, dim3(groups),
                       dim3(a.splits * 32), (size_t)a.splits * 2 * stage_bytes(false, true), a);
        else
            launch_pdl(gemv_w4a8_kernel<false, false, false, 2, true>, dim3(grid), dim3(kW * 32),
                       kRingK16, a);
    } else if (a.dump)
        launch_pdl(gemv_w4a8_kernel<false, true, false, 2>, dim3(grid), dim3(kW * 32), kRingP, a);
    else if (a.serial && a.splits >= 4)
        launch_pdl(gemv_w4a8_kernel<true, false, false, 2>, dim3(groups), dim3(a.splits * 32),
                   (size_t)a.splits * 2 * stage_bytes(false), a);
    else if (a.serial)
        launch_pdl(gemv_w4a8_kernel<true, false, false, 2>, dim3(grid), dim3(kW * 32), kRingP, a);
    else if (a.x && kRingF3 + qbytes <= kPerCta)
        launch_pdl(gemv_w4a8_kernel<false, false, true, 3>, dim3(grid), dim3(kW * 32),
                   kRingF3 + qbytes, a);
    else if (a.x && kRingF2 + qbytes <= kPerCta)
        launch_pdl(gemv_w4a8_kernel<false, false, true, 2>, dim3(grid), dim3(kW * 32),
                   kRingF2 + qbytes, a);
    else if (a.splits >= 4) {
        // Split weights (fewer than 4096 row-groups): one team per CTA, one row-group per CTA,
        // so the hardware places CTAs as SMs free up instead of a fixed share per SM (5%
        // faster than the persistent split on 17408x5120), and the next launch's first CTAs
        // start while the last ones of this launch drain. Few row-groups (a long-K weight,
        // at most three CTAs per SM in flight) get three ring stages, else two (four CTAs
        // per SM).
        const int nw = a.splits;
        if (groups <= 3 * g_sms)
            launch_pdl(gemv_w4a8_kernel<false, false, false, 3>, dim3(groups), dim3(nw * 32),
                       (size_t)nw * 3 * stage_bytes(false), a);
        else
            launch_pdl(gemv_w4a8_kernel<false, false, false, 2>, dim3(groups), dim3(nw * 32),
                       (size_t)nw * 2 * stage_bytes(false), a);
    } else
        launch_pdl(gemv_w4a8_kernel<false, false, false, 2>, dim3(grid), dim3(kW * 32), kRingP, a);
    TQ_LAUNCH_CHECK("gemv_w4a8_kernel");
}

}  // namespace tq
