// repack.cu — load-time conversion of a dense-E2M3 fragment payload into the packed
// int4 / int8 records (x_w4_repack_weight_mode, x_w8_repack_weight;
// xpu/src/kernels_dpas.cpp:229-399, 403-424).
//
// The arithmetic is the reference's, in its order, because the order is the contract: per
// (row, group) the source weights w = e2m3(code) * block_scale, the asymmetric fit of scale
// and zero point as sequential fp32 sums over the group, the FP16 scale stored with the zero
// point in its low nibble, and the codes re-quantised against the STORED scale. All IEEE fp32
// without contraction, so the CPU oracle reproduces every bit.
//
// The kernel around it is laid out for this GPU: one warp per (16-row group, pair of
// k-tiles), lane = (row, tile of the pair). The warp copies the pair's two 384-byte fragment
// tiles into shared memory with 16-byte loads, every lane decodes the 32 six-bit codes of
// its (row, tile) once from there and publishes them for the lane that fits the K64 pair,
// runs its group's fit, and stores its 16 packed bytes as one 16-byte word, so a tile's 256
// bytes leave as one coalesced run (the reference gave every (row, k-tile) its own work
// item, which decodes each K64 pair twice from scattered bytes and stores byte by byte).
//
// K64 note: like the reference, each tile of a pair fits all 64 values with the block scale
// of ITS OWN tile, and only the even tile stores the scale. With one block scale per 128
// columns (the usual container) both lanes of a row see the same numbers.
#include "e2m3.cuh"
#include "fit.cuh"

namespace tq {

namespace {

constexpr int kRepackWarps = 4;

// Copies the fragment tiles (g, 2p) and (g, 2p + 1) into this warp's shared buffer and decodes
// this lane's 32 codes (row n of tile u) to e2m3 values (not yet scaled).
__device__ __forceinline__ void load_and_decode(const uint8_t *__restrict__ payload, int Kt, int g, int p2,
                                                unsigned char *tiles, float (&v)[32], bool have) {
    const int lane = threadIdx.x & 31, n = lane & 15, u = lane >> 4;
    const int ntile = min(2, Kt - 2 * p2);
    const uint4 *src = reinterpret_cast<const uint4 *>(payload + ((size_t)g * Kt + 2 * p2) * 384u);
    for (int i = lane; i < ntile * 24; i += 32) reinterpret_cast<uint4 *>(tiles)[i] = __ldg(src + i);
    __syncwarp();
    if (!have) return;
    const unsigned char *t = tiles + u * 384;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        const int fl = ((n >> 1) << 2) | (j >> 3);
        const int idx = (((j >> 2) & 1) << 3) | ((n & 1) << 2) | (j & 3);
        const int bit = 6 * idx;
        const unsigned char *q = t + fl * 12 + (bit >> 3);
        uint32_t bits = q[0];
        if ((bit & 7) > 2) bits |= (uint32_t)q[1] << 8;
        v[j] = e2m3f((bits >> (bit & 7)) & 0x3fu);
    }
}

__global__ void __launch_bounds__(kRepackWarps * 32)
w4_repack_kernel(const uint8_t *__restrict__ payload, const float *__restrict__ bs, int scale_cols,
                 int M, int Kt, int mode, uint8_t *__restrict__ d_s4, uint16_t *__restrict__ d_sc) {
    __shared__ __align__(16) unsigned char s_tiles[kRepackWarps][768];
    __shared__ float s_val[kRepackWarps][2][16][33];          // decoded values, padded rows
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n = lane & 15, u = lane >> 4;
    const int pairs = (Kt + 1) >> 1;
    const size_t wid = (size_t)blockIdx.x * kRepackWarps + warp;
    if (wid >= (size_t)(M >> 4) * pairs) return;               // whole warps leave together
    const int g = (int)(wid / pairs), p2 = (int)(wid % pairs);
    const int kt = 2 * p2 + u;
    const bool have = kt < Kt;
    float v[32];
    load_and_decode(payload, Kt, g, p2, s_tiles[warp], v, have);
    if (mode == 2) {
#pragma unroll
        for (int j = 0; j < 32; ++j) s_val[warp][u][n][j] = have ? v[j] : 0.0f;
        __syncwarp();
    }
    if (!have) return;
    const int sc = (scale_cols == Kt) ? kt : (kt >> 2);
    const float b = bs[(size_t)(g >> 3) * scale_cols + sc];
    float wf[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) wf[j] = __fmul_rn(v[j], b);
    float gs[2];
    int gz[2];
    if (mode == 1) {
        for (int h = 0; h < 2; ++h) {
            int zh = 0;
            const uint16_t shh = fit_int4_asym(wf + h * 16, 16, &zh);
            d_sc[((size_t)g * (Kt * 2) + kt * 2 + h) * 16u + n] = (uint16_t)(shh | (zh & 0xF));
            gs[h] = __half2float(__ushort_as_half(shh));
            gz[h] = zh;
        }
    } else if (mode == 2) {
        float wf64[64];
        for (int j = 0; j < 32; ++j) {
            wf64[j] = __fmul_rn(s_val[warp][0][n][j], b);
            wf64[32 + j] = __fmul_rn(s_val[warp][1][n][j], b);
        }
        int zp = 0;
        const uint16_t sh = fit_int4_asym(wf64, 64, &zp);
        if (u == 0) d_sc[((size_t)g * (Kt / 2) + p2) * 16u + n] = (uint16_t)(sh | (zp & 0xF));
        gs[0] = gs[1] = __half2float(__ushort_as_half(sh));
        gz[0] = gz[1] = zp;
    } else {
        int zp = 0;
        const uint16_t sh = fit_int4_asym(wf, 32, &zp);
        d_sc[((size_t)g * Kt + kt) * 16u + n] = (uint16_t)(sh | (zp & 0xF));
        gs[0] = gs[1] = __half2float(__ushort_as_half(sh));
        gz[0] = gz[1] = zp;
    }
    // Row n owns bytes [n*16, n*16+16) of the tile; byte j/2 holds k = j (low nibble), j+1.
    uint32_t word[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        const int h = j >> 4;
        const float r = rintf(__fadd_rn(__fdiv_rn(wf[j], gs[h]), (float)gz[h]));
        const uint32_t q = (uint32_t)(((int)clampf(r, -8.0f, 7.0f)) & 0xF);
        word[j >> 3] |= q << (4 * (j & 7));
    }
    *reinterpret_cast<uint4 *>(d_s4 + ((size_t)g * Kt + kt) * 256u + (size_t)n * 16u) =
        make_uint4(word[0], word[1], word[2], word[3]);
}

// E2M3 -> symmetric int8 with one plain FP16 scale per (row, K32): w8_repack_kernel,
// xpu/src/kernels_dpas.cpp:348-395. codes[Mt][Kt][16 rows][32 B], scales[Mt][Kt][16].
__global__ void __launch_bounds__(kRepackWarps * 32)
w8_repack_kernel(const uint8_t *__restrict__ payload, const float *__restrict__ bs, int scale_cols,
                 int M, int Kt, uint8_t *__restrict__ d_s8, uint16_t *__restrict__ d_sc) {
    __shared__ __align__(16) unsigned char s_tiles[kRepackWarps][768];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n = lane & 15, u = lane >> 4;
    const int pairs = (Kt + 1) >> 1;
    const size_t wid = (size_t)blockIdx.x * kRepackWarps + warp;
    if (wid >= (size_t)(M >> 4) * pairs) return;
    const int g = (int)(wid / pairs), p2 = (int)(wid % pairs);
    const int kt = 2 * p2 + u;
    const bool have = kt < Kt;
    float v[32];
    load_and_decode(payload, Kt, g, p2, s_tiles[warp], v, have);
    if (!have) return;
    const int sc = (scale_cols == Kt) ? kt : (kt >> 2);
    const float b = bs[(size_t)(g >> 3) * scale_cols + sc];
    float wf[32];
    float hi = 0.0f, neg = 0.0f;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        wf[j] = __fmul_rn(v[j], b);
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
    d_sc[((size_t)g * Kt + kt) * 16u + n] = sh;
    const float stored = __half2float(__ushort_as_half(sh));
    uint32_t word[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        const uint32_t q = (uint32_t)(uint8_t)(int8_t)(int)clampf(rintf(__fdiv_rn(wf[j], stored)), -128.0f, 127.0f);
        word[j >> 2] |= q << (8 * (j & 3));
    }
    uint4 *dst = reinterpret_cast<uint4 *>(d_s8 + ((size_t)g * Kt + kt) * 512u + (size_t)n * 32u);
    dst[0] = make_uint4(word[0], word[1], word[2], word[3]);
    dst[1] = make_uint4(word[4], word[5], word[6], word[7]);
}

}  // namespace

void launch_w8_repack(const uint8_t *d_payload, const float *d_bs, int scale_cols, int M, int K,
                      uint8_t *d_codes, uint16_t *d_scales) {
    const int Kt = K / 32;
    const size_t warps = (size_t)(M / 16) * ((Kt + 1) / 2);
    const unsigned grid = (unsigned)((warps + kRepackWarps - 1) / kRepackWarps);
    w8_repack_kernel<<<grid, kRepackWarps * 32, 0, stream()>>>(d_payload, d_bs, scale_cols, M, Kt, d_codes,
                                                                d_scales);
    TQ_LAUNCH_CHECK("w8_repack_kernel");
}

void launch_w4_repack(const uint8_t *d_payload, const float *d_bs, int scale_cols, int M, int K,
                      int mode, uint8_t *d_codes, uint16_t *d_scales) {
    const int Kt = K / 32;
    const size_t warps = (size_t)(M / 16) * ((Kt + 1) / 2);
    const unsigned grid = (unsigned)((warps + kRepackWarps - 1) / kRepackWarps);
    w4_repack_kernel<<<grid, kRepackWarps * 32, 0, stream()>>>(d_payload, d_bs, scale_cols, M, Kt, mode,
                                                                d_codes, d_scales);
    TQ_LAUNCH_CHECK("w4_repack_kernel");
}

}  // namespace tq
