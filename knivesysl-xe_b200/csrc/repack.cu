// repack.cu — load-time conversion of a dense-E2M3 fragment payload into the packed
// int4 record (x_w4_repack_weight_mode, xpu/src/kernels_dpas.cpp:229-344, 403-424).
//
// One thread per (row, k-tile): decode the tile's 32 source weights
// (e2m3 code * block scale), fit scale + zero point over the group the mode asks for
// (K32, two K16 halves, or the K64 pair), store the FP16 scale with the zero point in
// its low nibble, then re-quantise the tile's codes against the STORED scale and pack
// them row-major inside the 256-byte tile. All arithmetic is IEEE fp32 without
// contraction so the CPU oracle reproduces every bit.
//
// K64 note: like the reference, the pair's fit is computed by both tiles' threads, each
// with the block scale of ITS OWN tile applied to all 64 values, and only the even tile
// stores the scale. With one block scale per 128 columns (the usual container) both
// threads see the same numbers.
#include "common.cuh"

namespace tq {

namespace {

__device__ __forceinline__ float e2m3f(uint32_t c) {
    const float m = (float)(c & 7u);
    const uint32_t e = (c >> 3) & 3u;
    const float v = (e == 0) ? __fmul_rn(m, 0.125f)
                             : __fmul_rn(__fadd_rn(1.0f, __fmul_rn(m, 0.125f)),
                                         (float)(1u << (e - 1)));
    return (c & 0x20u) ? -v : v;
}

// (row, col) -> 6-bit code of the fragment payload (kernels_dpas.cpp:59-69).
__device__ __forceinline__ uint32_t e2m3_code_at(const uint8_t *payload, int Kt, int row,
                                                 int col) {
    const int mt = row >> 4;
    const int kt = col >> 5;
    const int lane = (((row & 15) >> 1) << 2) | ((col & 31) >> 3);
    const int idx = (((col >> 2) & 1) << 3) | ((row & 1) << 2) | (col & 3);
    const int bit = 6 * idx;
    const uint8_t *p = payload + ((size_t)mt * Kt + kt) * 384u + (size_t)lane * 12u;
    uint32_t bits = p[bit >> 3];
    if ((bit & 7) > 2) bits |= (uint32_t)p[(bit >> 3) + 1] << 8;
    return (bits >> (bit & 7)) & 0x3fu;
}

// Asymmetric int4 group fit (kernels_dpas.cpp:229-256): returns the stored FP16 bits
// with the low nibble cleared; *out_z is the zero point.
__device__ uint16_t fit_int4_asym(const float *wf, int n, int *out_z) {
    float lo = 0.0f, hi = 0.0f;
    for (int j = 0; j < n; ++j) {
        lo = fminf(lo, wf[j]);
        hi = fmaxf(hi, wf[j]);
    }
    float s = __fdiv_rn(__fsub_rn(hi, lo), 15.0f);
    if (!(s > 0.0f)) s = 1.0f;
    for (int iter = 0; iter < 3; ++iter) {
        const int zi = (int)clampf(__fsub_rn(rintf(__fdiv_rn(-lo, s)), 8.0f), -8.0f, 7.0f);
        float num = 0.0f, den = 0.0f;
        for (int j = 0; j < n; ++j) {
            const float q =
                clampf(rintf(__fadd_rn(__fdiv_rn(wf[j], s), (float)zi)), -8.0f, 7.0f);
            const float centered = __fsub_rn(q, (float)zi);
            num = __fadd_rn(num, __fmul_rn(wf[j], centered));
            den = __fadd_rn(den, __fmul_rn(centered, centered));
        }
        if (den > 0.0f) s = __fdiv_rn(num, den);
    }
    *out_z = (int)clampf(__fsub_rn(rintf(__fdiv_rn(-lo, s)), 8.0f), -8.0f, 7.0f);
    uint16_t sh = __half_as_ushort(__float2half_rn(s));
    sh = (uint16_t)((sh + 8u) & 0xFFF0u);
    return sh;
}

__global__ void __launch_bounds__(128)
w4_repack_kernel(const uint8_t *__restrict__ payload, const float *__restrict__ bs, int scale_cols,
                 int M, int Kt, int mode, uint8_t *__restrict__ d_s4, uint16_t *__restrict__ d_sc) {
    const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= (size_t)M * Kt) return;
    const int row = (int)(gid / Kt);
    const int kt = (int)(gid % Kt);
    const int mt = row >> 4;
    const int sc = (scale_cols == Kt) ? kt : (kt >> 2);
    const float b = bs[(size_t)(mt >> 3) * scale_cols + sc];
    float wf[32];
    for (int j = 0; j < 32; ++j)
        wf[j] = __fmul_rn(e2m3f(e2m3_code_at(payload, Kt, row, kt * 32 + j)), b);
    const int rowgroup = row >> 4;
    const int n = row & 15;
    float gs[2];
    int gz[2];
    if (mode == 1) {
        for (int h = 0; h < 2; ++h) {
            int zh = 0;
            const uint16_t shh = fit_int4_asym(wf + h * 16, 16, &zh);
            d_sc[((size_t)rowgroup * (Kt * 2) + kt * 2 + h) * 16u + n] =
                (uint16_t)(shh | (zh & 0xF));
            gs[h] = __half2float(__ushort_as_half(shh));
            gz[h] = zh;
        }
    } else if (mode == 2) {
        const int kt0 = kt & ~1;
        float wf64[64];
        for (int j = 0; j < 64; ++j)
            wf64[j] = __fmul_rn(e2m3f(e2m3_code_at(payload, Kt, row, kt0 * 32 + j)), b);
        int zp = 0;
        const uint16_t sh = fit_int4_asym(wf64, 64, &zp);
        if ((kt & 1) == 0)
            d_sc[((size_t)rowgroup * (Kt / 2) + (kt >> 1)) * 16u + n] = (uint16_t)(sh | (zp & 0xF));
        gs[0] = gs[1] = __half2float(__ushort_as_half(sh));
        gz[0] = gz[1] = zp;
    } else {
        int zp = 0;
        const uint16_t sh = fit_int4_asym(wf, 32, &zp);
        d_sc[((size_t)rowgroup * Kt + kt) * 16u + n] = (uint16_t)(sh | (zp & 0xF));
        gs[0] = gs[1] = __half2float(__ushort_as_half(sh));
        gz[0] = gz[1] = zp;
    }
    // Row n owns bytes [n*16, n*16+16) of the tile; byte j/2 holds k = j (low) and j+1.
    uint8_t *dst = d_s4 + ((size_t)rowgroup * Kt + kt) * 256u + (size_t)n * 16u;
    for (int j = 0; j < 32; j += 2) {
        uint32_t qq[2];
        for (int u = 0; u < 2; ++u) {
            const int jj = j + u, h = jj >> 4;
            const float r = rintf(__fadd_rn(__fdiv_rn(wf[jj], gs[h]), (float)gz[h]));
            qq[u] = (uint32_t)(((int)clampf(r, -8.0f, 7.0f)) & 0xF);
        }
        dst[j >> 1] = (uint8_t)(qq[0] | (qq[1] << 4));
    }
}

// E2M3 -> symmetric int8 with one plain FP16 scale per (row, K32): w8_repack_kernel,
// xpu/src/kernels_dpas.cpp:348-395. codes[Mt][Kt][16 rows][32 B], scales[Mt][Kt][16].
__global__ void __launch_bounds__(128)
w8_repack_kernel(const uint8_t *__restrict__ payload, const float *__restrict__ bs, int scale_cols,
                 int M, int Kt, uint8_t *__restrict__ d_s8, uint16_t *__restrict__ d_sc) {
    const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= (size_t)M * Kt) return;
    const int row = (int)(gid / Kt);
    const int kt = (int)(gid % Kt);
    const int mt = row >> 4;
    const int sc = (scale_cols == Kt) ? kt : (kt >> 2);
    const float b = bs[(size_t)(mt >> 3) * scale_cols + sc];
    float wf[32];
    float hi = 0.0f, neg = 0.0f;
    for (int j = 0; j < 32; ++j) {
        wf[j] = __fmul_rn(e2m3f(e2m3_code_at(payload, Kt, row, kt * 32 + j)), b);
        hi = fmaxf(hi, wf[j]);
        neg = fmaxf(neg, -wf[j]);
    }
    float s = fmaxf(__fdiv_rn(hi, 127.0f), __fdiv_rn(neg, 128.0f));
    if (!(s > 0.0f)) s = 1.0f;
    for (int iter = 0; iter < 2; ++iter) {
        float num = 0.0f, den = 0.0f;
        for (int j = 0; j < 32; ++j) {
            const float q = clampf(rintf(__fdiv_rn(wf[j], s)), -128.0f, 127.0f);
            num = __fadd_rn(num, __fmul_rn(wf[j], q));
            den = __fadd_rn(den, __fmul_rn(q, q));
        }
        if (den > 0.0f) s = __fdiv_rn(num, den);
    }
    const uint16_t sh = __half_as_ushort(__float2half_rn(s));
    d_sc[((size_t)(row >> 4) * Kt + kt) * 16u + (row & 15)] = sh;
    const float stored = __half2float(__ushort_as_half(sh));
    uint8_t *dst = d_s8 + ((size_t)(row >> 4) * Kt + kt) * 512u + (size_t)(row & 15) * 32u;
    for (int j = 0; j < 32; ++j)
        dst[j] = (uint8_t)(int8_t)(int)clampf(rintf(__fdiv_rn(wf[j], stored)), -128.0f, 127.0f);
}

}  // namespace

void launch_w8_repack(const uint8_t *d_payload, const float *d_bs, int scale_cols, int M, int K,
                      uint8_t *d_codes, uint16_t *d_scales) {
    const int Kt = K / 32;
    const size_t items = (size_t)M * Kt;
    const unsigned grid = (unsigned)((items + 127) / 128);
    w8_repack_kernel<<<grid, 128, 0, stream()>>>(d_payload, d_bs, scale_cols, M, Kt, d_codes, d_scales);
    TQ_LAUNCH_CHECK("w8_repack_kernel");
}

void launch_w4_repack(const uint8_t *d_payload, const float *d_bs, int scale_cols, int M, int K,
                      int mode, uint8_t *d_codes, uint16_t *d_scales) {
    const int Kt = K / 32;
    const size_t items = (size_t)M * Kt;
    const unsigned grid = (unsigned)((items + 127) / 128);
    w4_repack_kernel<<<grid, 128, 0, stream()>>>(d_payload, d_bs, scale_cols, M, Kt, mode, d_codes,
                                                 d_scales);
    TQ_LAUNCH_CHECK("w4_repack_kernel");
}

}  // namespace tq
