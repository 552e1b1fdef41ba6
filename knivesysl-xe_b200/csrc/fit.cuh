// fit.cuh — the asymmetric int4 group fit shared by the repack kernel and the format probe.
#pragma once

#include "common.cuh"

namespace tq {

#ifdef __CUDACC__

// Asymmetric int4 group fit (kernels_dpas.cpp:229-256): returns the stored FP16 bits
// with the low nibble cleared; *out_z is the zero point.
__device__ inline uint16_t fit_int4_asym(const float *wf, int n, int *out_z) {
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

#endif  // __CUDACC__

}  // namespace tq
