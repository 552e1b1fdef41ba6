// checks.cu — model-free forms of the reference's self-checks and micro-benches
// (xpu/src/kernels_dpas.cpp:2146-2333, 2613-2693). They take a packed weight record
// instead of a layer of a loaded model and reproduce the reference's closed-form
// inputs, so the same gates can be run on synthetic weights.
#include "common.cuh"

#include <chrono>
#include <cmath>
#include <cstring>
#include <vector>

namespace {

// Input family of qwn_gemm_check / qwn_specwave_check (kernels_dpas.cpp:2225-2234,
// 2280-2286): magnitudes 2^-6..2^6, hashed signs, exact zeros every 97th column.
void fill_check_rows(std::vector<float> &x, int T, int K, int prefix, uint32_t salt) {
    for (int t = 0; t < T; ++t)
        for (int k = 0; k < K; ++k) {
            const uint32_t s = (t >= prefix) ? salt : 0u;
            const float mag = std::exp2((float)((k * 7 + t * 3 + (int)(s & 7)) % 13) - 6.0f);
            const float sgn = ((((uint32_t)k * 2654435761u + (uint32_t)t) ^ s) >> 31) ? -1.0f : 1.0f;
            x[(size_t)t * K + k] = ((k % 97) == 0) ? 0.0f : sgn * mag;
        }
}

struct DevBuf {
    void *p = nullptr;
    explicit DevBuf(size_t bytes, const char *what) { p = tq_dev_alloc(bytes, what); }
    ~DevBuf() { tq_dev_free(p); }
    template <class T> T *as() { return static_cast<T *>(p); }
};

}  // namespace

extern "C" {

double qwn_gemv_bench(const tq_qmma_weight_t *w, int iters) {
    if (!w || !w->s4_ready) return -2.0;
    const int M = w->M, K = w->K;
    const int n = (iters <= 0) ? 50 : iters;
    DevBuf x((size_t)K * 4, "gvb.x"), y((size_t)M * 4, "gvb.y");
    tq_dev_zero(x.p, (size_t)K * 4);
    x_prepare_gemv_act_s8(x.as<float>(), K);
    if (x_gemv_w4a8_prepared(w, y.as<float>()) != 0) return -3.0;
    tq_sync();
    const auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < n; ++i) x_gemv_w4a8_prepared(w, y.as<float>());
    tq_sync();
    const auto t1 = std::chrono::steady_clock::now();
    return std::chrono::duration<double, std::micro>(t1 - t0).count() / n;
}

double qwn_gemm_bench(const tq_qmma_weight_t *w, int tokens, int iters) {
    if (!w || !w->s4_ready || w->s4_k16) return -2.0;
    const int T = (tokens <= 0) ? 8 : ((tokens + 7) / 8) * 8;
    const int M = w->M, K = w->K, Kt = K / 32;
    const int n = (iters <= 0) ? 10 : iters;
    DevBuf x((size_t)T * K * 4, "gb.x"), y((size_t)T * M * 4, "gb.y");
    DevBuf aq((size_t)Kt * T * 32, "gb.aq"), as((size_t)Kt * T * 4, "gb.as"),
        asum((size_t)Kt * T * 4, "gb.asum");
    tq_dev_zero(x.p, (size_t)T * K * 4);
    x_quantize_act_chunk(x.as<float>(), K, T, aq.as<int8_t>(), as.as<float>(), asum.as<int32_t>());
    if (x_gemm_w4a8(w, aq.as<int8_t>(), as.as<float>(), asum.as<int32_t>(), y.as<float>(), T) != 0)
        return -3.0;
    tq_sync();
    const auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < n; ++i)
        x_gemm_w4a8(w, aq.as<int8_t>(), as.as<float>(), asum.as<int32_t>(), y.as<float>(), T);
    tq_sync();
    const auto t1 = std::chrono::steady_clock::now();
    return std::chrono::duration<double, std::micro>(t1 - t0).count() / n;
}

// Batched GEMM against the single-row GEMV, row by row; passes at cos >= 0.9999.
int qwn_gemm_check(const tq_qmma_weight_t *w, int tokens, double *worst_cos_out,
                   double *worst_rel_out) {
    if (!w || !w->s4_ready || w->s4_k16) return -2;
    const int T = (tokens <= 0) ? 8 : ((tokens + 7) / 8) * 8;
    const int M = w->M, K = w->K, Kt = K / 32;
    std::vector<float> hx((size_t)T * K);
    fill_check_rows(hx, T, K, T, 0u);
    DevBuf x((size_t)T * K * 4, "gc.x"), ref((size_t)T * M * 4, "gc.ref"),
        got((size_t)T * M * 4, "gc.got");
    DevBuf aq((size_t)Kt * T * 32, "gc.aq"), as((size_t)Kt * T * 4, "gc.as"),
        asum((size_t)Kt * T * 4, "gc.asum");
    tq_h2d(x.p, hx.data(), hx.size() * 4);
    for (int t = 0; t < T; ++t)
        if (x_gemv_w4a8(w, x.as<float>() + (size_t)t * K, ref.as<float>() + (size_t)t * M) != 0)
            return -3;
    x_quantize_act_chunk(x.as<float>(), K, T, aq.as<int8_t>(), as.as<float>(), asum.as<int32_t>());
    if (x_gemm_w4a8(w, aq.as<int8_t>(), as.as<float>(), asum.as<int32_t>(), got.as<float>(), T) != 0)
        return -4;
    std::vector<float> a((size_t)T * M), b((size_t)T * M);
    tq_d2h(a.data(), ref.p, a.size() * 4);
    tq_d2h(b.data(), got.p, b.size() * 4);
    double worst_cos = 1.0, worst_rel = 0.0;
    for (int t = 0; t < T; ++t) {
        double dot = 0, na = 0, nb = 0, rel = 0;
        for (int i = 0; i < M; ++i) {
            const double u = a[(size_t)t * M + i], v = b[(size_t)t * M + i];
            dot += u * v; na += u * u; nb += v * v;
            rel = std::max(rel, std::fabs(v - u) / (std::fabs(u) + 1e-3));
        }
        const double c = (na > 0 && nb > 0) ? dot / (std::sqrt(na) * std::sqrt(nb)) : 0.0;
        worst_cos = std::min(worst_cos, c);
        worst_rel = std::max(worst_rel, rel);
    }
    if (worst_cos_out) *worst_cos_out = worst_cos;
    if (worst_rel_out) *worst_rel_out = worst_rel;
    return worst_cos >= 0.9999 ? 0 : -5;
}

// Rows 0-3 of a T=8 GEMM must be byte-identical whatever rides in rows 4-7.
int qwn_specwave_check(const tq_qmma_weight_t *w) {
    if (!w || !w->s4_ready || w->s4_k16) return -2;
    const int T = 8, kPrefix = 4;
    const int M = w->M, K = w->K, Kt = K / 32;
    DevBuf x((size_t)T * K * 4, "sw.x"), y0((size_t)T * M * 4, "sw.y0"),
        y1((size_t)T * M * 4, "sw.y1");
    DevBuf aq((size_t)Kt * T * 32, "sw.aq"), as((size_t)Kt * T * 4, "sw.as"),
        asum((size_t)Kt * T * 4, "sw.asum");
    float *outs[2] = {y0.as<float>(), y1.as<float>()};
    std::vector<float> hx((size_t)T * K);
    for (int run = 0; run < 2; ++run) {
        fill_check_rows(hx, T, K, kPrefix, run ? 0x9E3779B9u : 0u);
        tq_h2d(x.p, hx.data(), hx.size() * 4);
        x_quantize_act_chunk(x.as<float>(), K, T, aq.as<int8_t>(), as.as<float>(),
                             asum.as<int32_t>());
        if (x_gemm_w4a8(w, aq.as<int8_t>(), as.as<float>(), asum.as<int32_t>(), outs[run], T) != 0)
            return -3;
        tq_sync();
    }
    std::vector<float> h0((size_t)kPrefix * M), h1((size_t)kPrefix * M);
    tq_d2h(h0.data(), y0.p, h0.size() * 4);
    tq_d2h(h1.data(), y1.p, h1.size() * 4);
    return std::memcmp(h0.data(), h1.data(), h0.size() * 4) == 0 ? 0 : 1;
}

// Column shards computed separately and concatenated must be bit-identical to the
// full GEMV (kernels_dpas.cpp:2652-2668), for any tp that divides the row-groups.
int qwn_shard_check(const tq_qmma_weight_t *w, int tp) {
    if (!w || !w->s4_ready || w->s4_k16) return -2;
    if (tp < 1) return -2;
    const int M = w->M, K = w->K;
    std::vector<float> hx(K);
    for (int i = 0; i < K; ++i)
        hx[i] = 0.05f * (float)(((uint32_t)i * 1103515245u + 12345u) % 97) - 2.0f;
    DevBuf x((size_t)K * 4, "sh.x"), ref((size_t)M * 4, "sh.ref"), got((size_t)M * 4, "sh.got");
    tq_h2d(x.p, hx.data(), (size_t)K * 4);
    x_prepare_gemv_act_s8(x.as<float>(), K);
    if (x_gemv_w4a8_prepared(w, ref.as<float>()) != 0) return -3;
    for (int r = 0; r < tp; ++r) {
        tq_qmma_weight_t s{};
        const int rc = x_w4_shard(&s, w, r, tp, 0, nullptr, 0);
        if (rc != 0) return rc;
        const int rc2 = x_gemv_w4a8_prepared(&s, got.as<float>() + (size_t)r * (M / tp));
        tq_sync();
        x_w4_shard_free(&s);
        if (rc2 != 0) return -3;
    }
    std::vector<float> a(M), b(M);
    tq_d2h(a.data(), ref.p, (size_t)M * 4);
    tq_d2h(b.data(), got.p, (size_t)M * 4);
    return std::memcmp(a.data(), b.data(), (size_t)M * 4) == 0 ? 0 : -4;
}

}  // extern "C"
