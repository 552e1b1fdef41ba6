// grid_probe.cu — weight-format probe (qwn_w4_grid_probe, xpu/src/kernels_dpas.cpp:1726-2146):
// how well eleven candidate low-bit formats reconstruct one E2M3 source matrix, at their
// metadata budgets. Pure read; an offline qualification tool, not on the projection path.
//
// For every row the device accumulates |w|^2 and, per scheme, <w, w_hat> and |w_hat|^2 in
// fp32 (one thread per row, k ascending, as the reference does); the host adds the rows in
// double and reports cosine and relative L2 error per scheme. Schemes, per K32 group of a row
// unless noted:
//   0 int4 symmetric, fp16 scale            1 int4 asymmetric, fp16 scale + zero point (the
//   2 the same per K16                        shipped tier: the repack's own fit)
//   3 NVFP4: E2M1 codes, E4M3 scale per K16, fp32 global per 128 rows
//   4 int8 symmetric, fp16 scale            5 int4 asymmetric, E4M3 scale per K16 + global
//   6 int4 symmetric, E4M3 scale per K16 + global
//   7 int3 symmetric, fp16 scale            8 int3 asymmetric, fp16 scale + zero point
//   9 per group: int3 (8) unless its squared error exceeds 1.8x the int4 fit's (1)
//  10 int4 asymmetric, fp16 scale per K64
#include "e2m3.cuh"
#include "fit.cuh"

#include <cmath>
#include <cstdio>
#include <vector>

namespace tq {
namespace {

constexpr int kSchemes = 11;
constexpr int kStride = 1 + 2 * kSchemes + 1;      // |w|^2, (dot, |w_hat|^2) per scheme, int3 group count

__device__ __forceinline__ float half_round_trip(float s) { return __half2float(__float2half_rn(s)); }

// Nearest non-negative OCP FP8 E4M3 value (largest 448, subnormal step 2^-9).
__device__ float round_e4m3(float v) {
    if (!(v > 0.0f)) return 0.0f;
    if (v >= 448.0f) return 448.0f;
    if (v < 0.015625f) return __fmul_rn(fminf(rintf(__fmul_rn(v, 512.0f)), 7.0f), 0.001953125f);
    int e = ilogbf(v);                                    // floor(log2 v), exact
    float p = ldexpf(1.0f, e);
    int q = (int)rintf(__fmul_rn(__fsub_rn(__fdiv_rn(v, p), 1.0f), 8.0f));
    if (q >= 8) {
        q = 0;
        ++e;
        p = __fmul_rn(p, 2.0f);
    }
    if (e >= 8) {                                         // 2^8 * 1.75 = 448
        p = 256.0f;
        if (q > 6) q = 6;
    }
    return __fmul_rn(p, __fadd_rn(1.0f, __fmul_rn((float)q, 0.125f)));
}

// Nearest E2M1 magnitude {0, .5, 1, 1.5, 2, 3, 4, 6}; a tie keeps the smaller one.
__device__ float round_e2m1(float v) {
    const float grid[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    float best = 0.0f, bd = fabsf(v);
    for (int i = 1; i < 8; ++i) {
        const float d = fabsf(__fsub_rn(v, grid[i]));
        if (d < bd) {
            bd = d;
            best = grid[i];
        }
    }
    return best;
}

// Symmetric fit with codes in [lo_q, hi_q]: scale from the extremes, two least-squares
// refinements, stored as fp16.
__device__ float fit_sym(const float *v, int n, float lo_q, float hi_q) {
    float hi = 0.0f, neg = 0.0f;
    for (int j = 0; j < n; ++j) {
        hi = fmaxf(hi, v[j]);
        neg = fmaxf(neg, -v[j]);
    }
    float s = fmaxf(__fdiv_rn(hi, hi_q), __fdiv_rn(neg, -lo_q));
    if (!(s > 0.0f)) s = 1.0f;
    for (int iter = 0; iter < 2; ++iter) {
        float num = 0.0f, den = 0.0f;
        for (int j = 0; j < n; ++j) {
            const float q = clampf(rintf(__fdiv_rn(v[j], s)), lo_q, hi_q);
            num = __fadd_rn(num, __fmul_rn(v[j], q));
            den = __fadd_rn(den, __fmul_rn(q, q));
        }
        if (den > 0.0f) s = __fdiv_rn(num, den);
    }
    return half_round_trip(s);
}

struct Tally {
    float dot[kSchemes], nb[kSchemes];
    __device__ void add(int s, float ref, float hat) {
        dot[s] = __fadd_rn(dot[s], __fmul_rn(ref, hat));
        nb[s] = __fadd_rn(nb[s], __fmul_rn(hat, hat));
    }
};

__device__ __forceinline__ float asym_hat(float v, float s, int zp, float lo_q, float hi_q) {
    const float q = clampf(rintf(__fadd_rn(__fdiv_rn(v, s), (float)zp)), lo_q, hi_q);
    return __fmul_rn(s, __fsub_rn(q, (float)zp));
}

struct Src {
    const uint8_t *payload;
    const float *bs;
    int M, K, Kt, scale_cols;
};
__device__ __forceinline__ float src_value(const Src &w, int row, int k) {
    const int kt = k >> 5;
    const int sc = (w.scale_cols == w.Kt) ? kt : (kt >> 2);
    const float b = w.bs[(size_t)((row >> 4) >> 3) * w.scale_cols + sc];
    return __fmul_rn(e2m3f(e2m3_code_at(w.payload, w.Kt, row, k)), b);
}

// absmax of every 128-row block: the "global" of the two-level schemes
__global__ void __launch_bounds__(256) probe_block_absmax_kernel(const Src w, float *__restrict__ g) {
    __shared__ float red[8];
    const int row0 = blockIdx.x * 128, rows = min(128, w.M - row0);
    float mx = 0.0f;
    for (long i = threadIdx.x; i < (long)rows * w.K; i += 256)
        mx = fmaxf(mx, fabsf(src_value(w, row0 + (int)(i / w.K), (int)(i % w.K))));
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int i = 1; i < 8; ++i) mx = fmaxf(mx, red[i]);
        g[blockIdx.x] = mx > 0.0f ? mx : 0.0f;
    }
}

__global__ void __launch_bounds__(64) probe_grid_kernel(const Src w, const float *__restrict__ g,
                                                        float *__restrict__ acc) {
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= w.M) return;
    Tally t{};
    float na = 0.0f, count3 = 0.0f;
    float v64[64];
    const float global = g[row >> 7];
    for (int kt = 0; kt < w.Kt; ++kt) {
        float *v = v64 + (kt & 1) * 32;                   // the K64 scheme sees the pair
        for (int j = 0; j < 32; ++j) {
            v[j] = src_value(w, row, kt * 32 + j);
            na = __fadd_rn(na, __fmul_rn(v[j], v[j]));
        }
        {   // 0
            const float s = fit_sym(v, 32, -8.0f, 7.0f);
            for (int j = 0; j < 32; ++j)
                t.add(0, v[j], __fmul_rn(s, clampf(rintf(__fdiv_rn(v[j], s)), -8.0f, 7.0f)));
        }
        int zp4 = 0;
        const float s4 = __half2float(__ushort_as_half(fit_int4_asym(v, 32, &zp4)));
        float err4 = 0.0f;
        for (int j = 0; j < 32; ++j) {   // 1
            const float hat = asym_hat(v[j], s4, zp4, -8.0f, 7.0f);
            t.add(1, v[j], hat);
            const float d = __fsub_rn(v[j], hat);
            err4 = __fadd_rn(err4, __fmul_rn(d, d));
        }
        for (int h = 0; h < 2; ++h) {    // 2, 3, 5, 6: per K16
            const float *u = v + 16 * h;
            int zp = 0;
            const float s2 = __half2float(__ushort_as_half(fit_int4_asym(u, 16, &zp)));
            float mx = 0.0f, lo = 0.0f, hi = 0.0f;
            for (int j = 0; j < 16; ++j) {
                t.add(2, u[j], asym_hat(u[j], s2, zp, -8.0f, 7.0f));
                mx = fmaxf(mx, fabsf(u[j]));
                lo = fminf(lo, u[j]);
                hi = fmaxf(hi, u[j]);
            }
            const float g3 = global > 0.0f ? __fdiv_rn(global, 6.0f * 448.0f) : 1.0f;
            const float s3 = __fmul_rn(round_e4m3(__fdiv_rn(mx, __fmul_rn(6.0f, g3))), g3);
            const float g5 = global > 0.0f ? __fdiv_rn(__fmul_rn(2.0f, global), 15.0f * 448.0f) : 1.0f;
            float s5 = __fmul_rn(round_e4m3(__fdiv_rn(__fdiv_rn(__fsub_rn(hi, lo), 15.0f), g5)), g5);
            if (!(s5 > 0.0f)) s5 = g5;
            const int zp5 = (int)clampf(__fsub_rn(rintf(__fdiv_rn(-lo, s5)), 8.0f), -8.0f, 7.0f);
            const float g6 = global > 0.0f ? __fdiv_rn(global, 8.0f * 448.0f) : 1.0f;
            float s6 = __fmul_rn(round_e4m3(__fdiv_rn(__fdiv_rn(mx, 8.0f), g6)), g6);
            if (!(s6 > 0.0f)) s6 = g6;
            for (int j = 0; j < 16; ++j) {
                const float x = u[j];
                t.add(3, x, s3 > 0.0f ? __fmul_rn(copysignf(round_e2m1(fabsf(__fdiv_rn(x, s3))), x), s3) : 0.0f);
                t.add(5, x, asym_hat(x, s5, zp5, -8.0f, 7.0f));
                t.add(6, x, __fmul_rn(s6, clampf(rintf(__fdiv_rn(x, s6)), -8.0f, 7.0f)));
            }
        }
        {   // 4
            float mx = 0.0f;
            for (int j = 0; j < 32; ++j) mx = fmaxf(mx, fabsf(v[j]));
            const float s = half_round_trip(mx > 0.0f ? __fdiv_rn(mx, 127.0f) : 1.0f);
            for (int j = 0; j < 32; ++j)
                t.add(4, v[j], __fmul_rn(s, clampf(rintf(__fdiv_rn(v[j], s)), -128.0f, 127.0f)));
        }
        {   // 7
            const float s = fit_sym(v, 32, -4.0f, 3.0f);
            for (int j = 0; j < 32; ++j)
                t.add(7, v[j], __fmul_rn(s, clampf(rintf(__fdiv_rn(v[j], s)), -4.0f, 3.0f)));
        }
        {   // 8 and 9
            float lo = 0.0f, hi = 0.0f;
            for (int j = 0; j < 32; ++j) {
                lo = fminf(lo, v[j]);
                hi = fmaxf(hi, v[j]);
            }
            float s = __fdiv_rn(__fsub_rn(hi, lo), 7.0f);
            if (!(s > 0.0f)) s = 1.0f;
            for (int iter = 0; iter < 3; ++iter) {
                const int zi = (int)clampf(__fsub_rn(rintf(__fdiv_rn(-lo, s)), 4.0f), -4.0f, 3.0f);
                float num = 0.0f, den = 0.0f;
                for (int j = 0; j < 32; ++j) {
                    const float c = __fsub_rn(clampf(rintf(__fadd_rn(__fdiv_rn(v[j], s), (float)zi)), -4.0f, 3.0f),
                                              (float)zi);
                    num = __fadd_rn(num, __fmul_rn(v[j], c));
                    den = __fadd_rn(den, __fmul_rn(c, c));
                }
                if (den > 0.0f) s = __fdiv_rn(num, den);
            }
            s = __half2float(__ushort_as_half((uint16_t)((__half_as_ushort(__float2half_rn(s)) + 8u) & 0xFFF0u)));
            const int zi = (int)clampf(__fsub_rn(rintf(__fdiv_rn(-lo, s)), 4.0f), -4.0f, 3.0f);
            float err3 = 0.0f;
            for (int j = 0; j < 32; ++j) {
                const float hat = asym_hat(v[j], s, zi, -4.0f, 3.0f);
                t.add(8, v[j], hat);
                const float d = __fsub_rn(v[j], hat);
                err3 = __fadd_rn(err3, __fmul_rn(d, d));
            }
            const bool use3 = err3 <= __fmul_rn(1.8f, err4);
            if (use3) count3 = __fadd_rn(count3, 1.0f);
            for (int j = 0; j < 32; ++j)
                t.add(9, v[j], use3 ? asym_hat(v[j], s, zi, -4.0f, 3.0f) : asym_hat(v[j], s4, zp4, -8.0f, 7.0f));
        }
        if (kt & 1) {   // 10
            int zp = 0;
            const float s = __half2float(__ushort_as_half(fit_int4_asym(v64, 64, &zp)));
            for (int j = 0; j < 64; ++j) t.add(10, v64[j], asym_hat(v64[j], s, zp, -8.0f, 7.0f));
        }
    }
    float *out = acc + (size_t)row * kStride;
    out[0] = na;
    for (int s = 0; s < kSchemes; ++s) {
        out[1 + 2 * s] = t.dot[s];
        out[2 + 2 * s] = t.nb[s];
    }
    out[1 + 2 * kSchemes] = count3;
}

}  // namespace
}  // namespace tq

// Probes the E2M3 source of `w` (a record that has not been repacked). cos_out / rel_out /
// bits_out, when not NULL, receive eleven values each. Returns 0 when the shipped tier
// (scheme 1) has the best cosine among the schemes at or below its bits per weight, 1 when
// another scheme beats it, -1 / -2 / -3 for a bad, an already repacked or a non-E2M3 record.
extern "C" int qwn_w4_grid_probe(const tq_qmma_weight_t *w, double *cos_out, double *rel_out, double *bits_out) {
    using namespace tq;
    if (!w || w->M <= 0 || w->K <= 0 || (w->M % 16) || (w->K % 64)) return -1;
    if (w->s4_ready || w->s8_ready || !w->d_A || !w->d_block_scale_inv) return -2;
    if (!w->block_scaled || !w->e2m3 || w->row_major || w->word_major) return -3;
    const int M = w->M, K = w->K;
    const Src src{w->d_A, w->d_block_scale_inv, M, K, K / 32, w->scale_cols};
    const int nrb = (M + 127) / 128;
    float *d_g = static_cast<float *>(tq_dev_alloc((size_t)nrb * 4, "probe.global"));
    float *d_acc = static_cast<float *>(tq_dev_alloc((size_t)M * kStride * 4, "probe.acc"));
    probe_block_absmax_kernel<<<nrb, 256, 0, stream()>>>(src, d_g);
    TQ_LAUNCH_CHECK("probe_block_absmax_kernel");
    probe_grid_kernel<<<(M + 63) / 64, 64, 0, stream()>>>(src, d_g, d_acc);
    TQ_LAUNCH_CHECK("probe_grid_kernel");
    std::vector<float> acc((size_t)M * kStride);
    tq_d2h(acc.data(), d_acc, acc.size() * sizeof(float));
    tq_dev_free(d_g);
    tq_dev_free(d_acc);

    double na = 0.0, dot[kSchemes] = {}, nb[kSchemes] = {}, count3 = 0.0;
    for (int row = 0; row < M; ++row) {
        const float *r = acc.data() + (size_t)row * kStride;
        na += r[0];
        for (int s = 0; s < kSchemes; ++s) {
            dot[s] += r[1 + 2 * s];
            nb[s] += r[2 + 2 * s];
        }
        count3 += r[1 + 2 * kSchemes];
    }
    static const char *names[kSchemes] = {
        "int4 sym    fp16/k32", "int4 asym   fp16/k32", "int4 asym   fp16/k16", "NVFP4 e2m1  e4m3/k16",
        "int8 sym    fp16/k32", "int4 asym   e4m3/k16", "int4 sym    e4m3/k16", "int3 sym    fp16/k32",
        "int3 asym   fp16/k32", "mix3/4 asym fp16/k32", "int4 asym   fp16/k64"};
    double bits[kSchemes] = {4.50, 4.50, 5.00, 4.50, 8.50, 4.75, 4.50, 3.50, 3.50, 0.0, 4.25};
    const double groups = (double)M * (K / 32);
    bits[9] = 0.5 + (3.0 * count3 + 4.0 * (groups - count3)) / (groups > 0.0 ? groups : 1.0);   // measured
    printf("grid probe [%dx%d]\n  %-22s %7s %10s %10s\n", M, K, "scheme", "bits/w", "cos", "rel_L2");
    auto cosine = [&](int s) { return (na > 0.0 && nb[s] > 0.0) ? dot[s] / (std::sqrt(na) * std::sqrt(nb[s])) : 0.0; };
    int best = 1;
    for (int s = 0; s < kSchemes; ++s) {
        const double c = cosine(s);
        const double err = na > 0.0 ? std::sqrt(std::max(0.0, na - 2.0 * dot[s] + nb[s]) / na) : 0.0;
        printf("  %-22s %7.2f %10.6f %10.6f\n", names[s], bits[s], c, err);
        if (cos_out) cos_out[s] = c;
        if (rel_out) rel_out[s] = err;
        if (bits_out) bits_out[s] = bits[s];
        if (s != 1 && bits[s] <= bits[1] + 1e-9 && c > cosine(best)) best = s;
    }
    printf("  best tier at <=%.2f bits/w: %s\n", bits[1], names[best]);
    return best == 1 ? 0 : 1;
}
