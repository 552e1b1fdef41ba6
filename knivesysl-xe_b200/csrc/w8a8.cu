// w8a8.cu — the W8A8 tier (int8 weights with one plain FP16 scale per (row, K32), no zero
// point): the reference's high-fidelity fallback for the few matrices that need more than four
// weight bits, lm_head first (xpu/src/kernels_dpas.cpp:345-395 repack, 768-843 GEMV,
// 1578-1629 GEMM). Weights: codes[Mt][Kt][16 rows][32 B] (a row's 32 codes are contiguous),
// scales[Mt][Kt][16]. Activations are the W4A8 staging unchanged.
//
// Both kernels are HBM-bound streams of 512-byte tiles. The GEMV keeps the W4A8 GEMV's
// mapping (a half-warp per tile, the two halves of a warp = the reference's two accumulators,
// a team of S warps per row-group, partial sums added in split order through shared memory)
// with plain batched loads: the one weight this tier serves in practice is hundreds of
// megabytes, so ramp and tail do not matter. The GEMM gives a warp one (row-group, eight
// tokens) task, as the reference does, on mma.sync m16n8k32: its A fragment is word c and
// word 4 + c of rows r and r + 8 of the tile, read straight from global memory.
#include "stream.cuh"

#include <algorithm>

namespace tq {

namespace {

constexpr int kW = 16;     // warps per GEMV CTA
constexpr int kU = 4;      // tiles a half-warp loads per batch

__global__ void __launch_bounds__(kW * 32)
gemv_w8a8_kernel(const uint8_t *__restrict__ codes, const uint16_t *__restrict__ scales,
                 const int8_t *__restrict__ q, const float *__restrict__ as,
                 const float *__restrict__ residual, float *__restrict__ y, int groups, int Kt,
                 int S) {
    __shared__ float part[kW * 16];
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = lane >> 4, n = lane & 15;
    const int tpc = kW / S, team = warp / S, split = warp - team * S;
    const int kt_begin = Kt * split / S;
    const int cnt = Kt * (split + 1) / S - kt_begin;
    for (int g0 = blockIdx.x * tpc; g0 < groups; g0 += gridDim.x * tpc) {
        const int g = g0 + team;
        float acc = 0.0f;
        if (g < groups) {
            const uint8_t *bbase = codes + ((size_t)g * Kt + kt_begin) * 512u + (size_t)n * 32u;
            const uint16_t *sbase = scales + ((size_t)g * Kt + kt_begin) * 16u + n;
            // this half-warp's tiles: offsets h, h + 2, ... (even offsets = accumulator 0)
            for (int i0 = h; i0 < cnt; i0 += 2 * kU) {
                uint4 wa[kU], wb[kU];
                uint32_t sc[kU];
#pragma unroll
                for (int u = 0; u < kU; ++u) {
                    const int i = i0 + 2 * u;
                    if (i < cnt) {
                        wa[u] = ldg_stream_v4(bbase + (size_t)i * 512u);
                        wb[u] = ldg_stream_v4(bbase + (size_t)i * 512u + 16);
                        sc[u] = __ldg(sbase + (size_t)i * 16u);
                    }
                }
#pragma unroll
                for (int u = 0; u < kU; ++u) {
                    const int i = i0 + 2 * u;
                    if (i >= cnt) break;
                    const int kt = kt_begin + i;
                    const uint4 a0 = __ldg(reinterpret_cast<const uint4 *>(q + (size_t)kt * 32));
                    const uint4 a1 = __ldg(reinterpret_cast<const uint4 *>(q + (size_t)kt * 32) + 1);
                    int d = __dp4a((int)wa[u].x, (int)a0.x, 0);
                    d = __dp4a((int)wa[u].y, (int)a0.y, d);
                    d = __dp4a((int)wa[u].z, (int)a0.z, d);
                    d = __dp4a((int)wa[u].w, (int)a0.w, d);
                    d = __dp4a((int)wb[u].x, (int)a1.x, d);
                    d = __dp4a((int)wb[u].y, (int)a1.y, d);
                    d = __dp4a((int)wb[u].z, (int)a1.z, d);
                    d = __dp4a((int)wb[u].w, (int)a1.w, d);
                    const float ws = __half2float(__ushort_as_half((unsigned short)sc[u]));
                    acc = fmaf(__fmul_rn((float)d, ws), __ldg(as + kt), acc);
                }
            }
        }
        acc = __fadd_rn(acc, __shfl_down_sync(0xffffffffu, acc, 16));    // acc0 + acc1
        const int row = g * 16 + n;
        if (S == 1) {
            // unsplit: the accumulator is stored as is; a residual is a separate add
            if (g < groups && h == 0) y[row] = residual ? __fadd_rn(acc, residual[row]) : acc;
            continue;
        }
        if (h == 0) part[warp * 16 + n] = acc;
        __syncthreads();
        if (g < groups && split == 0 && h == 0) {
            float sum = 0.0f;
            for (int i = 0; i < S; ++i) sum = __fadd_rn(sum, part[(warp + i) * 16 + n]);
            y[row] = __fadd_rn(sum, residual ? residual[row] : 0.0f);
        }
        __syncthreads();      // part is rewritten by the next round
    }
}

constexpr int kGW = 8;     // warps per GEMM CTA

__global__ void __launch_bounds__(kGW * 32)
gemm_w8a8_kernel(const uint8_t *__restrict__ codes, const uint16_t *__restrict__ scales,
                 const int8_t *__restrict__ aq, const float *__restrict__ as,
                 float *__restrict__ y, int M, int Kt, int T) {
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = lane >> 2, c = lane & 3;
    const int tgroups = T / 8;
    const long tasks = (long)(M / 16) * tgroups;
    int czero[4];
    make_const_quad(czero, 0);
    for (long task = (long)blockIdx.x * kGW + warp; task < tasks; task += (long)gridDim.x * kGW) {
        const int rg = (int)(task / tgroups), tg = (int)(task - (long)rg * tgroups);
        const uint8_t *bbase = codes + (size_t)rg * Kt * 512u + (size_t)r * 32u + c * 4;
        const uint16_t *sbase = scales + (size_t)rg * Kt * 16u + r;
        const int8_t *abase = aq + ((size_t)tg * 8 + r) * 32 + c * 4;
        const float *asb = as + (size_t)tg * 8 + 2 * c;
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int kt = 0; kt < Kt; ++kt) {
            const uint8_t *t = bbase + (size_t)kt * 512u;
            const uint32_t a0 = ldg_stream_u32(t), a2 = ldg_stream_u32(t + 16);
            const uint32_t a1 = ldg_stream_u32(t + 256), a3 = ldg_stream_u32(t + 272);
            const int8_t *ab = abase + (size_t)kt * T * 32;
            const uint32_t b0 = __ldg(reinterpret_cast<const uint32_t *>(ab));
            const uint32_t b1 = __ldg(reinterpret_cast<const uint32_t *>(ab + 16));
            int d[4];
            mma_s8_c(d, a0, a1, a2, a3, b0, b1, czero);
            const float ws0 = __half2float(__ushort_as_half(__ldg(sbase + (size_t)kt * 16u)));
            const float ws1 = __half2float(__ushort_as_half(__ldg(sbase + (size_t)kt * 16u + 8)));
            const float2 as2 = __ldg(reinterpret_cast<const float2 *>(asb + (size_t)kt * T));
            acc[0] = fmaf((float)d[0], __fmul_rn(ws0, as2.x), acc[0]);
            acc[1] = fmaf((float)d[1], __fmul_rn(ws0, as2.y), acc[1]);
            acc[2] = fmaf((float)d[2], __fmul_rn(ws1, as2.x), acc[2]);
            acc[3] = fmaf((float)d[3], __fmul_rn(ws1, as2.y), acc[3]);
        }
        const size_t row = (size_t)rg * 16 + r, tok = (size_t)tg * 8 + 2 * c;
        y[tok * M + row] = acc[0];
        y[(tok + 1) * M + row] = acc[1];
        y[tok * M + row + 8] = acc[2];
        y[(tok + 1) * M + row + 8] = acc[3];
    }
}

int g_sms = 0;
int sms() {
    if (!g_sms) {
        int dev = 0;
        TQ_CHECK(cudaGetDevice(&dev));
        TQ_CHECK(cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev));
        if (g_sms <= 0) g_sms = 148;
    }
    return g_sms;
}

}  // namespace

void launch_gemv_w8a8(const uint8_t *codes, const uint16_t *scales, const int8_t *q,
                      const float *as, const float *residual, float *y, int M, int K, int splits) {
    const int groups = M / 16, Kt = K / 32;
    if (groups <= 0 || splits <= 0 || splits > kW || (kW % splits)) return;
    const int tpc = kW / splits;
    const int grid = std::min(8 * sms(), (groups + tpc - 1) / tpc);
    launch_pdl(gemv_w8a8_kernel, dim3(grid), dim3(kW * 32), 0, codes, scales, q, as, residual, y,
               groups, Kt, splits);
    TQ_LAUNCH_CHECK("gemv_w8a8_kernel");
}

void launch_gemm_w8a8(const uint8_t *codes, const uint16_t *scales, const int8_t *aq,
                      const float *as, float *y, int M, int K, int T) {
    const long tasks = (long)(M / 16) * (T / 8);
    if (tasks <= 0) return;
    const int grid = (int)std::min<long>((tasks + kGW - 1) / kGW, 16L * sms());
    launch_pdl(gemm_w8a8_kernel, dim3(grid), dim3(kGW * 32), 0, codes, scales, aq, as, y, M, K / 32, T);
    TQ_LAUNCH_CHECK("gemm_w8a8_kernel");
}

}  // namespace tq
