// gemv.cu — single-row W4A8 GEMV (decode, one token) for sm_100a.
//
// Replaces x_gemv_w4a8_core and x_gemv_w4a8_fanout (xpu/src/kernels_dpas.cpp:586-675,
// 945-1102). HBM-bound: the packed weight stream (256 B per 16-row x K32 tile plus a
// 32 B scale line) is read exactly once; activations (32 B per k-tile) stay in L1/L2.
//
// Mapping. One warp owns one (row-group, K-split) task at a time, as the reference's
// sub-group does; the kernel is persistent (two CTAs of 16 warps per SM). A 256-byte tile is 16 rows x 16 B, so a HALF-warp reads one tile with one
// 128-bit load per lane and the two halves of a warp walk the even and the odd tiles
// of the split. That is exactly the reference's two-accumulator order (acc0 takes the
// even offsets from kt_begin, acc1 the odd ones, leftover to acc0), so each lane keeps
// ONE accumulator and acc0+acc1 is a single shuffle. The fan-out order (one serial
// accumulator) passes the odd half's product terms to the even half every pair.
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

constexpr int kU = 5;     // 128-bit weight loads in flight per lane (one batch); more spills at 64 registers
constexpr int kW = 16;    // warps per CTA

__device__ __forceinline__ int tile_dot_plus8(const uint4 &w, const uint4 &e, const uint4 &o) {
    int d = 0;
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
    const uint32_t ee[4] = {e.x, e.y, e.z, e.w};
    const uint32_t oo[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        d = __dp4a((int)nib_plus8(ww[j]), (int)ee[j], d);
        d = __dp4a((int)nib_plus8(ww[j] >> 4), (int)oo[j], d);
    }
    return d;
}

__device__ __forceinline__ uint32_t ldg_stream_u16(const uint16_t *p) {
    uint16_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

// Persistent kernel: a team of S warps owns one 16-row group at a time (warp s = K-split
// s) and walks the row-groups team, team + teams, ... Each half-warp reads whole tiles
// (one 128-bit load per lane = one row of a tile), so a warp keeps up to 2 * kU tiles
// in flight per batch; a batch is loaded completely, scale words included, before
// it is consumed, and 32 warps per SM overlap each other's batches.
// FUSEQ: the fp32 activation row is quantised by every CTA into shared memory (the same
// per-block rule and code as quant_s8_kernel) after the wait on earlier kernels, instead of
// being read from the prepared scratch; CTA 0 also writes the scratch.
template <bool SERIAL, bool DUMP, bool FUSEQ>
__global__ void __launch_bounds__(kW * 32, 2) gemv_w4a8_kernel(const GemvArgs a) {
    __shared__ float part[kW * 16];
    extern __shared__ __align__(16) unsigned char dyn[];   // FUSEQ: qp[K], as[K/32], sum32[K/32]
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int h = lane >> 4;
    const int n = lane & 15;
    const int S = a.splits;
    const int tpc = kW / S;                       // teams per CTA
    const int team = warp / S;
    const int split = warp - team * S;
    const int Kt = a.K >> 5;
    const int Ktg = Kt >> a.ksh;
    const int groups = a.goff[a.count];
    const int teams = gridDim.x * tpc;
    const int kt_begin = Kt * split / S;
    const int cnt = Kt * (split + 1) / S - kt_begin;
    // tiles of this half-warp: offsets h, h+2, ... inside the split; balanced batches
    const int nper = (cnt + 1) >> 1;
    const int nb = (nper + kU - 1) / kU;
    const int ub = nb ? (nper + nb - 1) / nb : 0;

    pdl_trigger();
    {
        // Before waiting for earlier kernels: pull this warp's first weight span into L2.
        const int g = blockIdx.x + gridDim.x * team;
        if (g < groups && cnt > 0) {
            int wi = 0;
            while (wi + 1 < a.count && g >= a.goff[wi + 1]) ++wi;
            const int lg = g - a.goff[wi];
            const uint8_t *p = a.codes[wi] + ((size_t)lg * Kt + kt_begin) * 256u;
            for (int line = lane; line < cnt * 2; line += 32) prefetch_l2(p + line * 128);
        }
    }
    pdl_wait();

    const int8_t *qp = a.qp;
    const float *asv = a.as;
    const int32_t *sumv = a.sum32;
    if (FUSEQ) {
        int8_t *sqp = reinterpret_cast<int8_t *>(dyn);
        float *sas = reinterpret_cast<float *>(dyn + a.K);
        int32_t *ssum = reinterpret_cast<int32_t *>(dyn + a.K + (size_t)Kt * 4);
        const bool scribe = blockIdx.x == 0;     // keeps the library's prepared scratch current
        for (int b = warp; b < Kt; b += kW) {
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
        qp = sqp;
        asv = sas;
        sumv = ssum;
    }

    for (int g = blockIdx.x + gridDim.x * team; g < groups; g += teams) {
        int wi = 0;
        while (wi + 1 < a.count && g >= a.goff[wi + 1]) ++wi;
        const int lg = g - a.goff[wi];
        const uint8_t *bbase =
            a.codes[wi] + ((size_t)lg * Kt + kt_begin) * 256u + (size_t)n * 16u;
        const uint16_t *sbase = a.scales[wi] + (size_t)lg * Ktg * 16u + n;

        float acc = 0.0f;
        for (int b = 0; b < nb; ++b) {
            const int i0 = b * ub;
            uint4 wv[kU];
            uint32_t sc[kU];
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                const int idx = 2 * (i0 + u) + h;
                if (u < ub && idx < cnt) {
                    wv[u] = ldg_stream_v4(bbase + (size_t)idx * 256u);
                    sc[u] = ldg_stream_u16(sbase + (size_t)((kt_begin + idx) >> a.ksh) * 16u);
                }
            }
#pragma unroll
            for (int u = 0; u < kU; ++u) {
                if (u >= ub) break;
                const int idx = 2 * (i0 + u) + h;
                const bool valid = idx < cnt;
                float fa = 0.0f, fb = 0.0f;
                if (valid) {
                    const int kt = kt_begin + idx;
                    uint4 e, o;
                    if (FUSEQ) {
                        e = *reinterpret_cast<const uint4 *>(qp + (size_t)kt * 32);
                        o = *reinterpret_cast<const uint4 *>(qp + (size_t)kt * 32 + 16);
                    } else {
                        e = __ldg(reinterpret_cast<const uint4 *>(qp + (size_t)kt * 32));
                        o = __ldg(reinterpret_cast<const uint4 *>(qp + (size_t)kt * 32 + 16));
                    }
                    const int dp = tile_dot_plus8(wv[u], e, o);
                    int zp;
                    float ws;
                    unpack_scale(sc[u], zp, ws);
                    const int asum = FUSEQ ? sumv[kt] : __ldg(sumv + kt);
                    if (DUMP) a.dump[((size_t)g * Kt + kt) * 16 + n] = dp - 8 * asum;
                    const float f = (float)(dp - (zp + 8) * asum);
                    fa = __fmul_rn(f, ws);
                    fb = FUSEQ ? asv[kt] : __ldg(asv + kt);
                }
                if (!SERIAL) {
                    if (valid) acc = fmaf(fa, fb, acc);
                } else {
                    // pair (even tile on h == 0, odd tile on h == 1), added in tile order
                    const float oa = __shfl_down_sync(0xffffffffu, fa, 16);
                    const float ob = __shfl_down_sync(0xffffffffu, fb, 16);
                    if (h == 0) {
                        if (valid) acc = fmaf(fa, fb, acc);
                        if (idx + 1 < cnt) acc = fmaf(oa, ob, acc);
                    }
                }
            }
        }
        if (DUMP) continue;
        if (!SERIAL) acc = __fadd_rn(acc, __shfl_down_sync(0xffffffffu, acc, 16));

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
    const int tpc = kW / a.splits;
    const int grid = std::min(2 * g_sms, (groups + tpc - 1) / tpc);
    if (a.dump)
        launch_pdl(gemv_w4a8_kernel<false, true, false>, dim3(grid), dim3(kW * 32), 0, a);
    else if (a.serial)
        launch_pdl(gemv_w4a8_kernel<true, false, false>, dim3(grid), dim3(kW * 32), 0, a);
    else if (a.x && (size_t)a.K + (size_t)(a.K / 32) * 8 <= 40 * 1024)
        launch_pdl(gemv_w4a8_kernel<false, false, true>, dim3(grid), dim3(kW * 32),
                   (size_t)a.K + (size_t)(a.K / 32) * 8, a);
    else
        launch_pdl(gemv_w4a8_kernel<false, false, false>, dim3(grid), dim3(kW * 32), 0, a);
    TQ_LAUNCH_CHECK("gemv_w4a8_kernel");
}

}  // namespace tq
