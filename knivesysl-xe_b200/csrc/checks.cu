// checks.cu — model-free forms of the reference's self-checks and micro-benches
// (xpu/src/kernels_dpas.cpp:2146-2333, 2462-2737). They take a packed weight record
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

}  // extern "C"

namespace {

// Input of the shard gates (kernels_dpas.cpp:2517-2518).
void fill_shard_row(std::vector<float> &x) {
    for (size_t i = 0; i < x.size(); ++i)
        x[i] = 0.05f * (float)(((uint32_t)i * 1103515245u + 12345u) % 97) - 2.0f;
}

struct Cmp {
    double cos, max_rel;
    bool exact;
};
Cmp compare_rows(const std::vector<float> &a, const std::vector<float> &b, double floor) {
    double dot = 0, na = 0, nb = 0, mrel = 0;
    bool exact = true;
    for (size_t i = 0; i < a.size(); ++i) {
        const double u = a[i], v = b[i];
        dot += u * v; na += u * u; nb += v * v;
        if (memcmp(&a[i], &b[i], 4) != 0) exact = false;
        mrel = std::max(mrel, std::fabs(u - v) / (std::fabs(u) + floor));
    }
    return Cmp{(na > 0 && nb > 0) ? dot / (std::sqrt(na) * std::sqrt(nb)) : 0.0, mrel, exact};
}

// One projection through x_w4_shard in the given mode, on one GPU: shards computed one after
// the other and reassembled (kernels_dpas.cpp:2544-2599). 0 column: bit-identical required;
// 1 row (K split, partial outputs added): cos >= 0.9999; 2 replicate: bit-identical.
// Returns 0 pass, 1 fail, < 0 error.
int shard_item(const tq_qmma_weight_t *w, int tp, int mode, const int *groups, int ngroups, Cmp *out) {
    if (!w || !w->s4_ready || w->s4_k16) return -2;
    if (tp < 1) return -2;
    const int M = w->M, K = w->K;
    std::vector<float> hx(K);
    fill_shard_row(hx);
    DevBuf x((size_t)K * 4, "sh.x"), ref((size_t)M * 4, "sh.ref"), got((size_t)M * 4, "sh.got"),
        tmp((size_t)M * 4, "sh.tmp");
    tq_h2d(x.p, hx.data(), (size_t)K * 4);
    x_prepare_gemv_act_s8(x.as<float>(), K);
    if (x_gemv_w4a8_prepared(w, ref.as<float>()) != 0) return -3;
    std::vector<float> a(M), b(M);
    if (mode == 0) {
        std::vector<float> part(M);
        for (int r = 0; r < tp; ++r) {
            tq_qmma_weight_t s{};
            const int rc = x_w4_shard(&s, w, r, tp, 0, groups, ngroups);
            if (rc != 0) return rc;
            const int rc2 = x_gemv_w4a8_prepared(&s, tmp.as<float>() + (size_t)r * (M / tp));
            tq_sync();
            x_w4_shard_free(&s);
            if (rc2 != 0) return -3;
        }
        tq_d2h(part.data(), tmp.p, (size_t)M * 4);
        // rank r owns run r of every block, so the per-rank outputs interleave by block
        const int nb = (groups && ngroups > 0) ? ngroups : 1;
        size_t base = 0, cur = 0;
        for (int g = 0; g < nb; ++g) {
            const size_t rows = (groups && ngroups > 0) ? (size_t)groups[g] : (size_t)M;
            const size_t per = rows / tp;
            for (int r = 0; r < tp; ++r)
                memcpy(&b[base + r * per], &part[(size_t)r * (M / tp) + cur], per * 4);
            base += rows;
            cur += per;
        }
    } else if (mode == 2) {
        tq_qmma_weight_t s{};
        const int rc = x_w4_shard(&s, w, 0, tp, 2, nullptr, 0);
        if (rc != 0) return rc;
        const int rc2 = x_gemv_w4a8_prepared(&s, got.as<float>());
        tq_sync();
        x_w4_shard_free(&s);
        if (rc2 != 0) return -3;
        tq_d2h(b.data(), got.p, (size_t)M * 4);
    } else {
        tq_dev_zero(got.p, (size_t)M * 4);
        for (int r = 0; r < tp; ++r) {
            tq_qmma_weight_t s{};
            const int rc = x_w4_shard(&s, w, r, tp, 1, nullptr, 0);
            if (rc != 0) return rc;
            x_prepare_gemv_act_s8(x.as<float>() + (size_t)r * (K / tp), K / tp);
            const int rc2 = x_gemv_w4a8_prepared(&s, tmp.as<float>());
            if (rc2 == 0) x_add_inplace(got.as<float>(), tmp.as<float>(), M);
            tq_sync();
            x_w4_shard_free(&s);
            if (rc2 != 0) return -3;
        }
        tq_d2h(b.data(), got.p, (size_t)M * 4);
    }
    tq_d2h(a.data(), ref.p, (size_t)M * 4);
    const Cmp c = compare_rows(a, b, 1e-6);
    if (out) *out = c;
    return (mode == 1 ? c.cos >= 0.9999 : c.exact) ? 0 : 1;
}

}  // namespace

extern "C" {

// The reference's qwn_shard_check on one weight (kernels_dpas.cpp:2613-2693): the column
// shards' outputs concatenated must be bit-identical to the full GEMV, and the row (K) shards'
// partial outputs added must agree with it at cos >= 0.9999. The column leg needs a shard to
// keep the full weight's split count (choose_gemv_splits: 8 between 5 and 4095 row-groups), as
// in the reference; the row leg is skipped (not failed) where x_w4_shard refuses the split
// (-7: tp does not divide the k-tiles, -8: a K64 pair would be cut). Returns 0 on pass, -4 when
// a leg fails its gate, another negative code on an error.
int qwn_shard_check(const tq_qmma_weight_t *w, int tp) {
    Cmp c{};
    const int col = shard_item(w, tp, 0, nullptr, 0, &c);
    if (col < 0) return col;
    const int row = shard_item(w, tp, 1, nullptr, 0, &c);
    if (row < 0 && row != -7 && row != -8) return row;
    return (col == 0 && row <= 0) ? 0 : -4;
}

// Model-free qwn_shard_check_all (kernels_dpas.cpp:2462-2611): every projection of a family,
// each in its intended mode (modes[i]: 0 column, 1 row, 2 replicate) and with its row blocks
// (groups + 3 * i, ngroups[i] of them; 0 = one block), sharded two ways. Prints one line per
// projection and returns the number that failed.
int qwn_shard_check_all(const tq_qmma_weight_t *const *ws, const int *modes, const int *groups,
                        const int *ngroups, int count) {
    if (!ws || !modes || count < 0) return -1;
    int fails = 0;
    for (int i = 0; i < count; ++i) {
        const tq_qmma_weight_t *w = ws[i];
        if (!w || !w->s4_ready || w->s4_k16) {
            printf("  item %-3d SKIP (not a K32/K64 int4 weight)\n", i);
            continue;
        }
        const int ng = ngroups ? ngroups[i] : 0;
        Cmp c{};
        const int rc = shard_item(w, 2, modes[i], (ng && groups) ? groups + 3 * i : nullptr, ng, &c);
        const char *mode = modes[i] == 0 ? "col" : modes[i] == 1 ? "row" : "rep";
        if (rc < 0) {
            printf("  item %-3d M=%-6d K=%-6d mode=%s FAIL rc=%d\n", i, w->M, w->K, mode, rc);
            ++fails;
            continue;
        }
        printf("  item %-3d M=%-6d K=%-6d mode=%s cos=%.8f max_rel=%-9.3g exact=%-3s %s\n", i, w->M, w->K,
               mode, c.cos, c.max_rel, c.exact ? "yes" : "no", rc == 0 ? "PASS" : "FAIL");
        fails += rc != 0;
    }
    return fails;
}

// Model-free qwn_w4_check (kernels_dpas.cpp:2696-2737): the weight must still hold its E2M3
// payload. The scalar E2M3 GEMV of the closed-form input is the reference; the weight is then
// repacked (mode 0 / 1 / 2; -1: mode 2 when TQ_XPU_K64=1, else 0 - the reference's switch)
// and the W4A8 GEMV of the same input must agree at cos >= 0.99. The weight stays repacked.
// Returns 0 pass, -2 already repacked, -3 / -4 / -5 a call failed, -6 below the gate.
int qwn_w4_check(tq_qmma_weight_t *w, int mode, double *cos_out, double *max_rel_out) {
    if (!w) return -1;
    if (w->s4_ready || w->s8_ready) return -2;
    const int M = w->M, K = w->K;
    if (M <= 0 || K <= 0) return -1;
    std::vector<float> hx((size_t)K);
    fill_check_rows(hx, 1, K, 1, 0u);
    DevBuf x((size_t)K * 4, "w4chk.x"), ref((size_t)M * 4, "w4chk.ref"), got((size_t)M * 4, "w4chk.got");
    tq_h2d(x.p, hx.data(), (size_t)K * 4);
    if (x_gemv_qmma(w, x.as<float>(), ref.as<float>()) != 0) return -3;
    if (mode < 0) {
        const char *e = getenv("TQ_XPU_K64");
        mode = (e && e[0] == '1') ? 2 : 0;
    }
    if (x_w4_repack_weight_mode(w, mode) != 0) return -4;
    if (x_gemv_w4a8(w, x.as<float>(), got.as<float>()) != 0) return -5;
    std::vector<float> a(M), b(M);
    tq_d2h(a.data(), ref.p, (size_t)M * 4);
    tq_d2h(b.data(), got.p, (size_t)M * 4);
    const Cmp c = compare_rows(a, b, 1e-3);
    if (cos_out) *cos_out = c.cos;
    if (max_rel_out) *max_rel_out = c.max_rel;
    printf("qwn_w4_check [%dx%d] mode %d: cos=%.6f max_rel=%.4f %s\n", M, K, mode, c.cos, c.max_rel,
           c.cos >= 0.99 ? "PASS" : "FAIL");
    return c.cos >= 0.99 ? 0 : -6;
}

}  // extern "C"
