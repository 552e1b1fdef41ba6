// e2m3.cuh — the E2M3 source format of a weight record: six-bit codes (1 sign, 2 exponent
// bits with bias 1, 3 mantissa bits; exponent zero is the m/8 subnormal range) laid out as
// 384-byte fragment tiles of 16 rows x 32 columns (xpu/src/kernels_core.cpp:44-75,
// xpu/src/kernels_dpas.cpp:50-69).
#pragma once

#include "common.cuh"

namespace tq {

#ifdef __CUDACC__

__device__ __forceinline__ float e2m3f(uint32_t c) {
    const float m = (float)(c & 7u);
    const uint32_t e = (c >> 3) & 3u;
    const float v = (e == 0) ? __fmul_rn(m, 0.125f)
                             : __fmul_rn(__fadd_rn(1.0f, __fmul_rn(m, 0.125f)),
                                         (float)(1u << (e - 1)));
    return (c & 0x20u) ? -v : v;
}

// (row, col) -> 6-bit code of the fragment payload: tile (row / 16, col / 32) holds 32 lanes of
// 12 bytes; lane = (row % 16 / 2) * 4 + col % 32 / 8 carries sixteen codes as a little-endian
// 6-bit stream, code index ((col / 4) % 2) * 8 + (row % 2) * 4 + col % 4.
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

#endif  // __CUDACC__

}  // namespace tq
