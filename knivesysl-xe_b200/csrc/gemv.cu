// gemv.cu — single-row W4A8 GEMV (decode, one token) for sm_100a.
//
// Replaces x_gemv_w4a8_core and x_gemv_w4a8_fanout (xpu/src/kernels_dpas.cpp:586-675,
// 945-1102). HBM-bound: the packed weight stream (256 B per 16-row x K32 tile plus a
// 32 B scale line) is read exactly once; activations (32 B per k-tile) stay in L1/L2.
//
// Mapping. One warp owns one (row-group, K-split) task, as the reference's sub-group
// does. A 256-byte tile is 16 rows x 16 B, so a HALF-warp reads one tile with one
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
#include "common.cuh"

namespace tq {

namespace {

constexpr int kUnroll = 4;   // 128-bit weight loads in flight per lane

struct TileOperands {
    uint4 w;
};

__device__ __forceinline__ int tile_dot_plus8(const uint4 &w, const uint4 &e, const uint4 &o) {
    int d = 0;
    const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
    const uint32_t ee[4] = {e.x, e.y, e.z, e.w};
    const uint32_t oo[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t lo = (ww[j] & 0x0F0F0F0Fu) ^ 0x08080808u;
        const uint32_t hi = ((ww[j] >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;
        d = __dp4a((int)lo, (int)ee[j], d);
        d = __dp4a((int)hi, (int)oo[j], d);
    }
    return d;
}

template <int W, bool SERIAL, bool DUMP>
__global__ void __launch_bounds__(W * 32) gemv_w4a8_kernel(const GemvArgs a) {
    __shared__ float part[W * 16];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int h = lane >> 4;
    const int n = lane & 15;
    const int S = a.splits;
    const int Kt = a.K >> 5;
    const int groups = a.goff[a.count];
    const int tasks = groups * S;
    const int task = blockIdx.x * W + warp;

    float acc = 0.0f;
    if (task < tasks) {
        const int g = task / S;
        const int split = task - g * S;
        int wi = 0;
        while (wi + 1 < a.count && g >= a.goff[wi + 1]) ++wi;
        const int lg = g - a.goff[wi];
        const uint8_t *bbase = a.codes[wi] + (size_t)lg * Kt * 256u + (size_t)n * 16u;
        const uint16_t *sbase = a.scales[wi] + (size_t)lg * (Kt >> a.ksh) * 16u + n;
        const int kt_begin = Kt * split / S;
        const int cnt = Kt * (split + 1) / S - kt_begin;

        for (int i0 = 0; i0 < cnt; i0 += 2 * kUnroll) {
            uint4 wv[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int idx = i0 + 2 * u + h;
                if (idx < cnt) wv[u] = ldg_stream_v4(bbase + (size_t)(kt_begin + idx) * 256u);
            }
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                const int idx = i0 + 2 * u + h;
                const bool valid = idx < cnt;
                float fa = 0.0f, fb = 0.0f;
                if (valid) {
                    const int kt = kt_begin + idx;
                    const uint4 e = __ldg(reinterpret_cast<const uint4 *>(a.qp + (size_t)kt * 32));
                    const uint4 o =
                        __ldg(reinterpret_cast<const uint4 *>(a.qp + (size_t)kt * 32 + 16));
                    const int dp = tile_dot_plus8(wv[u], e, o);
                    const uint32_t packed = __ldg(sbase + (size_t)(kt >> a.ksh) * 16u);
                    int zp;
                    float ws;
                    unpack_scale(packed, zp, ws);
                    const int asum = __ldg(a.sum32 + kt);
                    if (DUMP) {
                        a.dump[((size_t)g * Kt + kt) * 16 + n] = dp - 8 * asum;
                    }
                    const float f = (float)(dp - (zp + 8) * asum);
                    fa = __fmul_rn(f, ws);
                    fb = __ldg(a.as + kt);
                }
                if (!SERIAL) {
                    if (valid) acc = fmaf(fa, fb, acc);
                } else {
                    // pair (even tile on h == 0, odd tile on h == 1), added in tile order
                    const float oa = __shfl_down_sync(0xffffffffu, fa, 16);
                    const float ob = __shfl_down_sync(0xffffffffu, fb, 16);
                    if (h == 0) {
                        if (valid) acc = fmaf(fa, fb, acc);
                        if (i0 + 2 * u + 1 < cnt) acc = fmaf(oa, ob, acc);
                    }
                }
            }
        }
        if (!SERIAL) acc = __fadd_rn(acc, __shfl_down_sync(0xffffffffu, acc, 16));
    }
    if (DUMP) return;

    if (S == 1) {
        if (task < tasks && h == 0) {
            int wi = 0;
            while (wi + 1 < a.count && task >= a.goff[wi + 1]) ++wi;
            const int row = (task - a.goff[wi]) * 16 + n;
            // unsplit: the accumulator is stored as is; a residual is a separate add
            a.y[wi][row] = a.residual ? __fadd_rn(acc, a.residual[row]) : acc;
        }
        return;
    }
    if (h == 0) part[warp * 16 + n] = acc;
    __syncthreads();
    const int gpw = W / S;                 // complete row-groups per block
    if (warp >= gpw || h != 0) return;
    const int g = blockIdx.x * gpw + warp;
    if (g >= groups) return;
    float sum = 0.0f;
    for (int i = 0; i < S; ++i) sum = __fadd_rn(sum, part[(warp * S + i) * 16 + n]);
    int wi = 0;
    while (wi + 1 < a.count && g >= a.goff[wi + 1]) ++wi;
    const int row = (g - a.goff[wi]) * 16 + n;
    if (SERIAL)
        a.y[wi][row] = sum;
    else
        a.y[wi][row] = __fadd_rn(sum, a.residual ? a.residual[row] : 0.0f);
}

template <int W>
void launch_w(const GemvArgs &a, int grid) {
    if (a.dump)
        gemv_w4a8_kernel<W, false, true><<<grid, W * 32, 0, stream()>>>(a);
    else if (a.serial)
        gemv_w4a8_kernel<W, true, false><<<grid, W * 32, 0, stream()>>>(a);
    else
        gemv_w4a8_kernel<W, false, false><<<grid, W * 32, 0, stream()>>>(a);
}

}  // namespace

void launch_gemv(const GemvArgs &a) {
    const int groups = a.goff[a.count];
    const int tasks = groups * a.splits;
    if (tasks <= 0) return;
    if (a.splits == 16) {
        launch_w<16>(a, (tasks + 15) / 16);
    } else {
        launch_w<8>(a, (tasks + 7) / 8);
    }
    TQ_LAUNCH_CHECK("gemv_w4a8_kernel");
}

}  // namespace tq
