// gemm_mma.cu — batched W4A8 GEMM for small token counts (decode batches, T = 8..64)
// and the general fallback for any T % 8 == 0, on sm_100a.
//
// Replaces x_gemm_w4a8's split path and gemm_rc16 (xpu/src/kernels_dpas.cpp:1255-1490).
// At T <= 64 the kernel is HBM-bound on the weight stream: one warp owns one
// (row-group, K-split) task for ALL token rows of its block (up to 64), so every
// weight byte is fetched once. One k-tile (16 rows x K32) against 8 tokens is exactly
// one mma.sync.m16n8k32.s8.s8.s32, giving the exact int32 tile dots the reference's
// dpas produces; the fp32 promote term = (float)(d - z*asum) * (ws*as) is applied per
// k-tile in ascending order into one accumulator per output, and the K-splits are
// added 0..S-1 through shared memory (an unsplit segment stores its accumulator
// untouched), so the summation order matches the reference.
//
// Operand mapping. mma A = weights (16 rows), B = activations (8 tokens). The k slots
// of the instruction are a fixed permutation of the tile's k (exact for an integer
// dot): lane (r = lane/4, c = lane%4) loads word c of rows r and r+8; its even-k
// nibbles fill k-slots 4c..4c+3 and its odd-k nibbles k-slots 16+4c..; the matching
// activation bytes are picked out of the token's 8 natural-order bytes with two byte
// permutes. Nibbles are used as q+8 (xor 8), the -8*asum is folded into the zero-point
// term: d - z*asum == d' - (z+8)*asum.
#include "common.cuh"

namespace tq {

namespace {

__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                       uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}

// Token block b of the launch -> first 8-token group, number of groups, segment index.
// Blocks never straddle a segment, because a segment owns its split count.
template <int NTG>
__device__ __forceinline__ void locate_block(const GemmSegments &s, int b, int &tg0, int &ntg,
                                             int &seg) {
    int start = 0;
    for (int i = 0; i < s.count; ++i) {
        const int len = s.end[i] - start;
        const int nb = (len + NTG - 1) / NTG;
        if (b < nb) {
            tg0 = start + b * NTG;
            ntg = min(NTG, s.end[i] - tg0);
            seg = i;
            return;
        }
        b -= nb;
        start = s.end[i];
    }
    tg0 = 0; ntg = 0; seg = 0;
}

template <int W, int NTG, bool DUMP>
__global__ void __launch_bounds__(W * 32) gemm_w4a8_mma_kernel(const GemmArgs a) {
    __shared__ float red[W * NTG * 4 * 32];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int r = lane >> 2;      // row inside the half tile / token inside the group
    const int c = lane & 3;
    const int S = a.max_splits;
    const int gpb = W / S;
    const int sub = warp / S;
    const int split = warp - sub * S;
    const int Kt = a.K >> 5;
    const int T = a.T;
    const int groups = a.goff[a.count];
    const int g = blockIdx.x * gpb + sub;
    const bool live = g < groups;

    int wi = 0;
    if (live)
        while (wi + 1 < a.count && g >= a.goff[wi + 1]) ++wi;
    const int lg = live ? g - a.goff[wi] : 0;
    int tg0, ntg, seg;
    locate_block<NTG>(a.seg[wi], blockIdx.y, tg0, ntg, seg);
    const int actual = a.seg[wi].split[seg];

    float acc[NTG][4];
#pragma unroll
    for (int t = 0; t < NTG; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[t][i] = 0.0f;

    if (live && split < actual) {
        const int kt_begin = Kt * split / actual;
        const int kt_end = Kt * (split + 1) / actual;
        const uint8_t *bptr = a.codes[wi] + (size_t)lg * Kt * 256u + (size_t)r * 16u + c * 4u;
        const uint16_t *sbase = a.scales[wi] + (size_t)lg * (Kt >> a.ksh) * 16u;
        for (int kt = kt_begin; kt < kt_end; ++kt) {
            const uint32_t w0 = ldg_stream_u32(bptr + (size_t)kt * 256u);
            const uint32_t w1 = ldg_stream_u32(bptr + (size_t)kt * 256u + 128u);
            const uint32_t a0 = (w0 & 0x0F0F0F0Fu) ^ 0x08080808u;
            const uint32_t a2 = ((w0 >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;
            const uint32_t a1 = (w1 & 0x0F0F0F0Fu) ^ 0x08080808u;
            const uint32_t a3 = ((w1 >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;
            int zp0, zp1;
            float ws0, ws1;
            unpack_scale(__ldg(sbase + (size_t)(kt >> a.ksh) * 16u + r), zp0, ws0);
            unpack_scale(__ldg(sbase + (size_t)(kt >> a.ksh) * 16u + r + 8), zp1, ws1);
            zp0 += 8;
            zp1 += 8;
#pragma unroll
            for (int t = 0; t < NTG; ++t) {
                if (t < ntg) {
                    const size_t arow = (size_t)kt * T + (size_t)(tg0 + t) * 8;
                    const uint2 bb =
                        __ldg(reinterpret_cast<const uint2 *>(a.aq + (arow + r) * 32 + c * 8));
                    const uint32_t b0 = __byte_perm(bb.x, bb.y, 0x6420);
                    const uint32_t b1 = __byte_perm(bb.x, bb.y, 0x7531);
                    int d[4];
                    mma_s8(d, a0, a1, a2, a3, b0, b1);
                    const float2 as2 = __ldg(reinterpret_cast<const float2 *>(a.as + arow + 2 * c));
                    const int2 sm2 = __ldg(reinterpret_cast<const int2 *>(a.asum + arow + 2 * c));
                    if (DUMP) {
                        const size_t M = (size_t)a.M[0];
                        const size_t row0 = (size_t)lg * 16 + r;
                        int32_t *o = a.dump + (arow + 2 * c) * M;
                        o[row0] = d[0] - 8 * sm2.x;
                        o[M + row0] = d[1] - 8 * sm2.y;
                        o[row0 + 8] = d[2] - 8 * sm2.x;
                        o[M + row0 + 8] = d[3] - 8 * sm2.y;
                    }
                    acc[t][0] = fmaf((float)(d[0] - zp0 * sm2.x), __fmul_rn(ws0, as2.x), acc[t][0]);
                    acc[t][1] = fmaf((float)(d[1] - zp0 * sm2.y), __fmul_rn(ws0, as2.y), acc[t][1]);
                    acc[t][2] = fmaf((float)(d[2] - zp1 * sm2.x), __fmul_rn(ws1, as2.x), acc[t][2]);
                    acc[t][3] = fmaf((float)(d[3] - zp1 * sm2.y), __fmul_rn(ws1, as2.y), acc[t][3]);
                }
            }
        }
    }
    if (DUMP) return;

    const int M = a.M[wi];
    if (S == 1) {
        if (live) {
            float *y = a.y[wi];
#pragma unroll
            for (int t = 0; t < NTG; ++t) {
                if (t < ntg) {
                    const size_t tok = (size_t)(tg0 + t) * 8 + 2 * c;
                    const size_t row = (size_t)lg * 16 + r;
                    y[tok * M + row] = acc[t][0];
                    y[(tok + 1) * M + row] = acc[t][1];
                    y[tok * M + row + 8] = acc[t][2];
                    y[(tok + 1) * M + row + 8] = acc[t][3];
                }
            }
        }
        return;
    }
#pragma unroll
    for (int t = 0; t < NTG; ++t)
#pragma unroll
        for (int i = 0; i < 4; ++i) red[((warp * NTG + t) * 4 + i) * 32 + lane] = acc[t][i];
    __syncthreads();
    if (!live || split != 0) return;
    float *y = a.y[wi];
#pragma unroll
    for (int t = 0; t < NTG; ++t) {
        if (t < ntg) {
            float out[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int base = (((sub * S) * NTG + t) * 4 + i) * 32 + lane;
                float sum;
                if (actual == 1) {
                    sum = red[base];   // unsplit segment: no extra "+0" rounding step
                } else {
                    sum = 0.0f;
                    for (int s = 0; s < actual; ++s)
                        sum = __fadd_rn(sum, red[base + s * NTG * 4 * 32]);
                }
                out[i] = sum;
            }
            const size_t tok = (size_t)(tg0 + t) * 8 + 2 * c;
            const size_t row = (size_t)lg * 16 + r;
            y[tok * M + row] = out[0];
            y[(tok + 1) * M + row] = out[1];
            y[tok * M + row + 8] = out[2];
            y[(tok + 1) * M + row + 8] = out[3];
        }
    }
}

int token_blocks(const GemmSegments &s, int ntg) {
    int start = 0, nb = 0;
    for (int i = 0; i < s.count; ++i) {
        nb += (s.end[i] - start + ntg - 1) / ntg;
        start = s.end[i];
    }
    return nb;
}

template <int W, int NTG>
void launch_one(const GemmArgs &a) {
    const int groups = a.goff[a.count];
    const int gpb = W / a.max_splits;
    dim3 grid((groups + gpb - 1) / gpb, token_blocks(a.seg[0], NTG));
    if (a.dump)
        gemm_w4a8_mma_kernel<W, NTG, true><<<grid, W * 32, 0, stream()>>>(a);
    else
        gemm_w4a8_mma_kernel<W, NTG, false><<<grid, W * 32, 0, stream()>>>(a);
}

}  // namespace

void launch_gemm_mma(const GemmArgs &a) {
    // Longest segment decides how many 8-token groups one warp carries.
    int longest = 0, start = 0;
    for (int i = 0; i < a.seg[0].count; ++i) {
        longest = max(longest, a.seg[0].end[i] - start);
        start = a.seg[0].end[i];
    }
    if (a.max_splits == 16) {
        if (longest <= 1) launch_one<16, 1>(a);
        else if (longest <= 2) launch_one<16, 2>(a);
        else launch_one<16, 4>(a);
    } else {
        if (longest <= 1) launch_one<8, 1>(a);
        else if (longest <= 2) launch_one<8, 2>(a);
        else if (longest <= 4) launch_one<8, 4>(a);
        else launch_one<8, 8>(a);
    }
    TQ_LAUNCH_CHECK("gemm_w4a8_mma_kernel");
}

}  // namespace tq
