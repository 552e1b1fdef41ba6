// dispatch.cu — the projection API of the library: argument checks, split heuristics,
// tier routing and launches. Same names, argument meaning and return codes as
// xpu/src/kernels_dpas.cpp (x_* functions) and xpu/src/kernels_core.cpp:164-252.
#include "common.cuh"

#include <algorithm>
#include <string.h>

namespace tq {

// xpu/src/kernels_dpas.cpp:170-173
int choose_gemv_splits(int groups) {
    if (groups <= 4) return 16;
    return groups >= 4096 ? 1 : 8;
}

// Split count of a batched GEMM (the rule of xpu/src/kernels_dpas.cpp:1226-1250, which fixes
// the order an output's partial sums are added in): the smallest power of two that brings
// row-groups x token-groups x splits to 2048 tasks, never more than 16 nor than the number
// of k-tiles. TQ_XPU_GEMM_SPLITS = 1, 2, 4, 8 or 16 overrides the count (same cap).
namespace {
int forced_gemm_splits() {
    static int cached = -1;
    if (cached < 0) {
        const char *e = getenv("TQ_XPU_GEMM_SPLITS");
        const int v = (e && *e) ? atoi(e) : 0;
        cached = (v > 0 && v <= 16 && (v & (v - 1)) == 0) ? v : 0;
    }
    return cached;
}
}  // namespace

int choose_gemm_splits(int rgroups, int tgroups, int ktiles) {
    const long tasks = (long)rgroups * tgroups;
    if (tasks <= 0) return 1;
    int cap = 1;                                   // largest power of two <= min(16, ktiles)
    while (cap < 16 && cap * 2 <= ktiles) cap *= 2;
    if (const int f = forced_gemm_splits()) return std::min(f, cap);
    const long kEnough = 2048;                     // 128 work-groups of 16 sub-groups
    int s = 1;
    while (s < cap && tasks * s < kEnough) s *= 2;
    return s;
}

// Split count of the per-token decode GEMMs (own rule; the reference has no per-token mode).
// A warp of the decode kernel carries all tokens of a call, so the task count does not grow
// with the tokens: as many splits as an 8-token call of the same weight, doubled while the
// staged activations of one split (320 bytes per k-tile and 8 tokens) exceed 88 KB, so that
// they fit beside the weight rings in shared memory. Splits cut whole weight-scale groups.
int choose_pertoken_splits(int rgroups, int tgroups, int ktiles, int ksh) {
    const int kgroups = ktiles >> ksh;
    int s = choose_gemm_splits(rgroups, 1, kgroups);
    if (forced_gemm_splits()) return s;
    int cap = 1;
    while (cap < 16 && cap * 2 <= kgroups) cap *= 2;
    const long budget = 88 * 1024;
    while (s < cap && (long)(((kgroups + s - 1) / s) << ksh) * tgroups * 320 > budget) s *= 2;
    return s;
}

bool decode_prefers_mma() {
    static const int v = [] {
        const char *e = getenv("TQ_XPU_DECODE_MMA");
        return (e && *e && *e != '0') ? 1 : 0;
    }();
    return v != 0;
}

int decode_dtc_min_tokens() {
    static const int v = [] {
        const char *e = getenv("TQ_XPU_DTC_MIN_TOKENS");
        const int n = (e && *e) ? atoi(e) : 1 << 20;     // default: never by itself
        return n < 8 ? 8 : n;
    }();
    return v;
}

namespace {

bool w4_usable(const tq_qmma_weight_t *w) {
    return w && w->s4_ready && w->d_s4 && w->d_s4_scale;
}

int gemv_prepared_impl(const tq_qmma_weight_t *w, float *d_y, const float *d_residual,
                       int32_t *dump, const float *d_x_fused = nullptr) {
    if (!w4_usable(w) || (!d_y && !dump)) return -1;
    ActScratch &s = act_scratch();
    if (s.cap < w->K || !s.q || !s.scale || s.prepared_K < w->K) return -2;
    if (w->M % 16 || w->K % 32) return -1;
    if (w->s4_k16 && (dump || d_x_fused)) return -1;   // K16: prepared activations, no dump
    ProfScope prof(w->M, w->K, 1, weight_tier(w));
    GemvArgs a{};
    a.codes[0] = w->d_s4;
    a.scales[0] = w->d_s4_scale;
    a.y[0] = d_y;
    a.goff[0] = 0;
    a.goff[1] = w->M / 16;
    a.count = 1;
    a.qp = s.qp;
    a.as = s.scale;
    a.sum32 = s.sum32;
    a.sum16 = s.sum16;
    a.k16 = w->s4_k16 ? 1 : 0;
    a.residual = d_residual;
    a.K = w->K;
    a.ksh = w->s4_k64 ? 1 : 0;
    a.splits = choose_gemv_splits(w->M / 16);
    a.serial = 0;
    a.dump = dump;
    if (d_x_fused) {
        a.x = d_x_fused;
        a.sq = s.q; a.sqp = s.qp; a.sscale = s.scale; a.ssum16 = s.sum16; a.ssum32 = s.sum32;
    }
    launch_gemv(a);
    return 0;
}

// One launch for a GEMV from the fp32 row (x_gemv_w4a8_fused): the GEMV quantises the row in
// its own prologue and keeps the prepared scratch current. x_gemv_w4a8 / _add themselves take
// the reference's two launches, which are the faster form on B200 (17408x5120: 11.8 us
// against 13.7 us; 5120x17408: 12.3 us against 28.7 us): with the quantiser inside, every CTA
// quantises the whole row from the same L2 lines at the same moment and the kernel cannot
// use its one-row-group launch shape. Rows too long for the kernel's shared memory, and the
// K16 tier, take the two launches here too.
int gemv_fused_impl(const tq_qmma_weight_t *w, const float *d_x, const float *d_residual,
                    float *d_y) {
    if (!w4_usable(w) || w->K <= 0 || (w->K % 32) || w->s4_k16) {
        x_prepare_gemv_act_s8(d_x, w ? w->K : 0);
        return gemv_prepared_impl(w, d_y, d_residual, nullptr);
    }
    ensure_act_scratch(w->K);
    ActScratch &s = act_scratch();
    if ((size_t)w->K + (size_t)(w->K / 32) * 8 > 40 * 1024) {
        x_prepare_gemv_act_s8(d_x, w->K);
        return gemv_prepared_impl(w, d_y, d_residual, nullptr);
    }
    const int before = s.prepared_K;
    s.prepared_K = w->K;      // the launch below (re)writes the scratch for this K
    const int rc = gemv_prepared_impl(w, d_y, d_residual, nullptr, d_x);
    if (rc != 0) s.prepared_K = before;
    return rc;
}

// Segment table + per-weight split counts (kernels_dpas.cpp:1343-1367).
int build_segments(int rgroups, int Kt, int T, const int *offsets, int segments,
                   GemmSegments &out, int &max_splits) {
    const int tgroups = T / 8;
    max_splits = 1;
    if (offsets) {
        if (segments < 1 || segments > 8 || offsets[0] != 0 || offsets[segments] != T) return -2;
        out.count = segments;
        for (int i = 0; i < segments; ++i) {
            if (offsets[i] < 0 || offsets[i + 1] <= offsets[i] || offsets[i + 1] > T ||
                offsets[i] % 8 || offsets[i + 1] % 8)
                return -2;
            out.end[i] = offsets[i + 1] / 8;
            out.split[i] = choose_gemm_splits(rgroups, (offsets[i + 1] - offsets[i]) / 8, Kt);
            max_splits = std::max(max_splits, out.split[i]);
        }
    } else {
        if (segments != 0) return -2;
        out.count = 1;
        out.end[0] = tgroups;
        out.split[0] = max_splits = choose_gemm_splits(rgroups, tgroups, Kt);
    }
    return 0;
}

}  // namespace
}  // namespace tq

using namespace tq;

// ---- repack -------------------------------------------------------------------------
int x_w4_repack_weight_mode(tq_qmma_weight_t *w, int mode) {
    if (!w || !w->d_A || !w->d_block_scale_inv || !w->block_scaled || !w->e2m3) return -1;
    if (w->M % 16 || w->K % 128) return -2;
    if (mode == 2 && (w->Kt & 1)) return -3;
    const size_t code_bytes = (size_t)w->Mt * w->Kt * 256u;
    const size_t scale_groups = (mode == 1) ? (size_t)w->Kt * 2u
                              : (mode == 2) ? (size_t)w->Kt / 2u : (size_t)w->Kt;
    const size_t scale_bytes = (size_t)w->M * scale_groups * sizeof(uint16_t);
    w->d_s4 = static_cast<uint8_t *>(tq_dev_alloc(code_bytes, "w4.codes"));
    w->d_s4_scale = static_cast<uint16_t *>(tq_dev_alloc(scale_bytes, "w4.scales"));
    launch_w4_repack(w->d_A, w->d_block_scale_inv, w->scale_cols, w->M, w->K, mode, w->d_s4,
                     w->d_s4_scale);
    tq_sync();
    tq_dev_free(w->d_A);
    tq_dev_free(w->d_block_scale_inv);
    w->d_A = nullptr;
    w->d_block_scale_inv = nullptr;
    w->s4_k16 = (mode == 1) ? 1 : 0;
    w->s4_k64 = (mode == 2) ? 1 : 0;
    w->s4_ready = 1;
    return 0;
}

int x_w4_repack_weight(tq_qmma_weight_t *w) { return x_w4_repack_weight_mode(w, 0); }

// ---- decode staging -------------------------------------------------------------------
void x_quantize_act_s8(const float *d_x, int K, int8_t *d_q, float *d_scale, int32_t *d_sum) {
    if (!d_x || !d_q || !d_scale || K <= 0) return;
    launch_quant_s8(d_x, nullptr, nullptr, K, d_q, nullptr, d_scale, d_sum, nullptr, false);
}

void x_prepare_gemv_act_s8(const float *d_x, int K) {
    if (!d_x || K <= 0 || (K % 32) != 0) return;
    ensure_act_scratch(K);
    ActScratch &s = act_scratch();
    launch_quant_s8(d_x, nullptr, nullptr, K, s.q, s.qp, s.scale, s.sum16, s.sum32, false);
    s.prepared_K = K;
}

void x_silu_mul_quant(float *d_out, const float *d_gate, const float *d_up, int K) {
    if (!d_out || !d_gate || !d_up || K <= 0 || (K % 32) != 0) return;
    ensure_act_scratch(K);
    ActScratch &s = act_scratch();
    launch_quant_s8(d_gate, d_up, d_out, K, s.q, s.qp, s.scale, s.sum16, s.sum32, true);
    s.prepared_K = K;
}

// Per-token forms of the two decode stagings: one scale (absmax / 127) for the whole row.
void x_prepare_gemv_act_s8_pertoken(const float *d_x, int K) {
    if (!d_x || K <= 0 || (K % 32) != 0) return;
    ensure_act_scratch(K);
    ActScratch &s = act_scratch();
    launch_quant_s8_pertoken(d_x, nullptr, nullptr, K, s.q, s.qp, s.scale, s.sum16, s.sum32, s.norm_partial,
                             false);
    s.prepared_K = K;
}

void x_silu_mul_quant_pertoken(float *d_out, const float *d_gate, const float *d_up, int K) {
    if (!d_out || !d_gate || !d_up || K <= 0 || (K % 32) != 0) return;
    ensure_act_scratch(K);
    ActScratch &s = act_scratch();
    launch_quant_s8_pertoken(d_gate, d_up, d_out, K, s.q, s.qp, s.scale, s.sum16, s.sum32, s.norm_partial,
                             true);
    s.prepared_K = K;
}

void x_rmsnorm_quant(float *d_out, const float *d_in, const uint16_t *d_w, int H, float eps) {
    if (!d_out || !d_in || !d_w || H <= 0 || (H % 32) != 0) return;
    ensure_act_scratch(H);
    ActScratch &s = act_scratch();
    launch_rmsnorm_quant(d_out, d_in, d_w, H, eps, s.norm_partial, s.q, s.qp, s.scale, s.sum16,
                         s.sum32);
    s.prepared_K = H;
}

void x_silu_mul(float *d_out, const float *d_gate, const float *d_up, int N) {
    if (!d_out || !d_gate || !d_up || N <= 0) return;
    launch_silu_mul(d_out, d_gate, d_up, N);
}

void x_add_inplace(float *d_x, const float *d_y, int N) {
    if (!d_x || !d_y || N <= 0) return;
    launch_add_inplace(d_x, d_y, N);
}

// ---- GEMV ---------------------------------------------------------------------------
int x_gemv_w4a8_prepared(const tq_qmma_weight_t *w, float *d_y, const float *d_residual) {
    return gemv_prepared_impl(w, d_y, d_residual, nullptr);
}

int x_gemv_w4a8(const tq_qmma_weight_t *w, const float *d_x, float *d_y) {
    if (!w || !d_x) return -1;
    x_prepare_gemv_act_s8(d_x, w->K);
    return gemv_prepared_impl(w, d_y, nullptr, nullptr);
}

int x_gemv_w4a8_add(const tq_qmma_weight_t *w, const float *d_x, const float *d_residual,
                    float *d_y) {
    if (!w || !d_x || !d_residual) return -1;
    x_prepare_gemv_act_s8(d_x, w->K);
    return gemv_prepared_impl(w, d_y, d_residual, nullptr);
}

int x_gemv_w4a8_fused(const tq_qmma_weight_t *w, const float *d_x, const float *d_residual,
                      float *d_y) {
    if (!w || !d_x) return -1;
    return gemv_fused_impl(w, d_x, d_residual, d_y);
}

int x_gemv_w4a8_fanout(const tq_qmma_weight_t *const *ws, float *const *ys, int count) {
    if (!ws || !ys || count <= 0 || count > 4) return -1;
    if (!ws[0]) return -2;
    int prof_rows = 0;
    for (int i = 0; i < count; ++i) prof_rows += ws[i] ? ws[i]->M : 0;
    ProfScope prof(prof_rows, ws[0]->K, 1, weight_tier(ws[0]));
    GemvArgs a{};
    const int K = ws[0]->K;
    const int ksh = ws[0]->s4_k64 ? 1 : 0;
    a.goff[0] = 0;
    for (int i = 0; i < count; ++i) {
        const tq_qmma_weight_t *w = ws[i];
        if (!w || !w->s4_ready || w->s4_k16 || !w->d_s4 || !w->d_s4_scale || !ys[i] ||
            w->K != K || (w->M % 16) || (w->s4_k64 ? 1 : 0) != ksh)
            return -2;
        a.codes[i] = w->d_s4;
        a.scales[i] = w->d_s4_scale;
        a.y[i] = ys[i];
        a.goff[i + 1] = a.goff[i] + w->M / 16;
    }
    ActScratch &s = act_scratch();
    if (s.cap < K || !s.q || !s.scale || s.prepared_K < K) return -3;
    a.count = count;
    a.qp = s.qp;
    a.as = s.scale;
    a.sum32 = s.sum32;
    a.residual = nullptr;
    a.K = K;
    a.ksh = ksh;
    a.splits = choose_gemv_splits(a.goff[count]);
    a.serial = 1;
    a.dump = nullptr;
    launch_gemv(a);
    return 0;
}

// ---- W8A8 tier (xpu/src/kernels_dpas.cpp:558-573, 768-843, 1578-1629, 1682-1726) --------
int x_w8_repack_weight(tq_qmma_weight_t *w) {
    if (!w || !w->d_A || !w->d_block_scale_inv || !w->block_scaled || !w->e2m3) return -1;
    if (w->M % 16 || w->K % 128) return -2;
    w->d_s8 = static_cast<uint8_t *>(tq_dev_alloc((size_t)w->Mt * w->Kt * 512u, "w8.codes"));
    w->d_s8_scale =
        static_cast<uint16_t *>(tq_dev_alloc((size_t)w->M * w->Kt * sizeof(uint16_t), "w8.scales"));
    launch_w8_repack(w->d_A, w->d_block_scale_inv, w->scale_cols, w->M, w->K, w->d_s8, w->d_s8_scale);
    tq_sync();
    tq_dev_free(w->d_A);
    tq_dev_free(w->d_block_scale_inv);
    w->d_A = nullptr;
    w->d_block_scale_inv = nullptr;
    w->s8_ready = 1;
    return 0;
}

int x_gemv_w8a8_prepared(const tq_qmma_weight_t *w, float *d_y, const float *d_residual) {
    if (!w || !w->s8_ready || !w->d_s8 || !w->d_s8_scale || !d_y) return -1;
    ProfScope prof(w->M, w->K, 1, 8);
    ActScratch &s = act_scratch();
    if (s.cap < w->K || !s.q || !s.scale || s.prepared_K < w->K) return -2;
    if (w->M % 16 || w->K % 32) return -1;
    launch_gemv_w8a8(w->d_s8, w->d_s8_scale, s.q, s.scale, d_residual, d_y, w->M, w->K,
                     choose_gemv_splits(w->M / 16));
    return 0;
}

int x_gemv_w8a8(const tq_qmma_weight_t *w, const float *d_x, float *d_y) {
    if (!w || !d_x) return -1;
    x_prepare_gemv_act_s8(d_x, w->K);
    return x_gemv_w8a8_prepared(w, d_y, nullptr);
}

int x_gemv_w8a8_add(const tq_qmma_weight_t *w, const float *d_x, const float *d_residual,
                    float *d_y) {
    if (!w || !d_x || !d_residual) return -1;
    x_prepare_gemv_act_s8(d_x, w->K);
    return x_gemv_w8a8_prepared(w, d_y, d_residual);
}

int x_gemm_w8a8(const tq_qmma_weight_t *w, const int8_t *d_aq, const float *d_as, float *d_y,
                int T) {
    if (!w || !w->s8_ready || !w->d_s8 || !w->d_s8_scale) return -1;
    if (!d_aq || !d_as || !d_y || T <= 0 || (T % 8) != 0) return -2;
    ProfScope prof(w->M, w->K, T, 8);
    launch_gemm_w8a8(w->d_s8, w->d_s8_scale, d_aq, d_as, d_y, w->M, w->K, T);
    return 0;
}

// ---- tier dispatchers (xpu/src/kernels_core.cpp:164-252) -------------------------------
int x_gemv_qmma(const tq_qmma_weight_t *w, const float *d_x, float *d_y) {
    if (!w || !d_x || !d_y) return -1;
    if (w->M <= 0 || w->K <= 0 || w->Mt <= 0 || w->Kt <= 0) return -2;
    if (w->s8_ready) return x_gemv_w8a8(w, d_x, d_y);
    if (w->s4_ready) return x_gemv_w4a8(w, d_x, d_y);
    return launch_gemv_e2m3(w, d_x, nullptr, d_y);   // not repacked yet: the scalar E2M3 tier
}

int x_gemv_qmma_add(const tq_qmma_weight_t *w, const float *d_x, const float *d_residual,
                    float *d_y) {
    if (!w || !d_x || !d_residual || !d_y) return -1;
    if (w->s8_ready) return x_gemv_w8a8_add(w, d_x, d_residual, d_y);
    if (w->s4_ready) return x_gemv_w4a8_add(w, d_x, d_residual, d_y);
    // the reference adds the residual with a separate x_add_inplace: the same single fp32 add
    if (w->M <= 0 || w->K <= 0 || w->Mt <= 0 || w->Kt <= 0) return -2;
    return launch_gemv_e2m3(w, d_x, d_residual, d_y);
}

int x_gemv_qmma_prepared(const tq_qmma_weight_t *w, const float *d_x, float *d_y,
                         const float *d_residual) {
    if (!w || !d_x || !d_y) return -1;
    if (w->s8_ready) return x_gemv_w8a8_prepared(w, d_y, d_residual);
    if (w->s4_ready) return x_gemv_w4a8_prepared(w, d_y, d_residual);
    return d_residual ? x_gemv_qmma_add(w, d_x, d_residual, d_y) : x_gemv_qmma(w, d_x, d_y);
}

// ---- chunk staging + GEMM ------------------------------------------------------------------
void x_quantize_act_chunk(const float *d_x, int K, int T, int8_t *d_aq, float *d_as,
                          int32_t *d_asum) {
    if (!d_x || !d_aq || !d_as || !d_asum || K <= 0 || T <= 0 || (K % 32) != 0) return;
    launch_quant_chunk(d_x, K, T, d_aq, d_as, d_asum);
}

void x_quantize_act_chunk_pertoken(const float *d_x, int K, int T, int8_t *d_aq, float *d_as,
                                   int32_t *d_asum, float *d_as_tok) {
    if (!d_x || !d_aq || !d_as || !d_asum || !d_as_tok || K <= 0 || T <= 0 || (K % 32) != 0)
        return;
    launch_quant_chunk_pertoken(d_x, K, T, d_aq, d_as, d_asum, d_as_tok);
}

namespace {

// Library-owned chunk staging for the fused-quantiser entry points when the shape is not
// the ring kernel's (grown on demand, like the decode scratch).
struct ChunkScratch {
    int8_t *aq = nullptr;
    float *as = nullptr;
    int32_t *asum = nullptr;
    float *as_tok = nullptr;
    size_t blocks = 0;
    int tokens = 0;
} g_chunk;

void ensure_chunk_scratch(size_t blocks, int T) {
    if (blocks > g_chunk.blocks) {
        if (g_chunk.aq) { tq_dev_free(g_chunk.aq); tq_dev_free(g_chunk.as); tq_dev_free(g_chunk.asum); }
        g_chunk.aq = static_cast<int8_t *>(tq_dev_alloc(blocks * 32, "chunk.aq"));
        g_chunk.as = static_cast<float *>(tq_dev_alloc(blocks * 4, "chunk.as"));
        g_chunk.asum = static_cast<int32_t *>(tq_dev_alloc(blocks * 4, "chunk.asum"));
        g_chunk.blocks = blocks;
    }
    if (T > g_chunk.tokens) {
        if (g_chunk.as_tok) tq_dev_free(g_chunk.as_tok);
        g_chunk.as_tok = static_cast<float *>(tq_dev_alloc((size_t)T * 4, "chunk.as_tok"));
        g_chunk.tokens = T;
    }
}

// Common part of the fan-out GEMM entry points. d_x != nullptr: quantise x[T][K] first
// (x_mode 1 per (token, K32) block, 2 per token) - inside the GEMM kernel when the ring kernel
// takes the call, else into the library's chunk scratch.
int fanout_args(GemmArgs &a, const tq_qmma_weight_t *const *ws, int count, int T, const int *offsets,
                int segments, const int *full_rows = nullptr) {
    if (!ws || count <= 0 || count > 4 || !ws[0]) return -1;
    const int K = ws[0]->K;
    const int ksh = ws[0]->s4_k64 ? 1 : 0;
    for (int i = 0; i < count; ++i) {
        const tq_qmma_weight_t *w = ws[i];
        if (!w || !w->s4_ready || w->s4_k16 || !w->d_s4 || !w->d_s4_scale) return -1;
        if (w->K != K || (w->s4_k64 ? 1 : 0) != ksh || (w->M % 16) || (K % 32)) return -1;
    }
    if (T <= 0 || (T % 8) != 0) return -2;
    a.goff[0] = 0;
    a.max_splits = 1;
    for (int i = 0; i < count; ++i) {
        const tq_qmma_weight_t *w = ws[i];
        a.codes[i] = w->d_s4;
        a.scales[i] = w->d_s4_scale;
        a.M[i] = w->M;
        a.goff[i + 1] = a.goff[i] + w->M / 16;
        int ms = 1;
        // a column shard keeps the split count (hence the summation order) of the whole weight
        const int rows = (full_rows && full_rows[i] > 0) ? full_rows[i] : w->M;
        const int rc = build_segments(rows / 16, K / 32, T, offsets, segments, a.seg[i], ms);
        if (rc) return rc;
        a.max_splits = std::max(a.max_splits, ms);
    }
    a.count = count;
    a.K = K;
    a.ksh = ksh;
    a.T = T;
    a.dump = nullptr;
    return 0;
}

// Per-token calls use their own split rule (one segment, the same count for every weight).
// full_rows: row counts of the whole projections when the weights are column shards.
void apply_pertoken_splits(GemmArgs &a, const int *full_rows = nullptr) {
    int s = 1;
    for (int i = 0; i < a.count; ++i) {
        const int rows = (full_rows && full_rows[i] > 0) ? full_rows[i] : a.M[i];
        s = std::max(s, choose_pertoken_splits(rows / 16, a.T / 8, a.K / 32, a.ksh));
    }
    a.max_splits = s;
    for (int i = 0; i < a.count; ++i) a.seg[i].split[0] = s;
}

// Sets the activation source of a prepared GemmArgs: the caller's staging, or x fused / staged.
void set_fused_input(GemmArgs &a, const float *d_x, int per_token) {
    a.x = d_x;
    a.x_mode = per_token ? 2 : 1;
    if (gemm_ring_covers(a)) return;
    const size_t blocks = (size_t)(a.K / 32) * a.T;
    ensure_chunk_scratch(blocks, a.T);
    if (per_token)
        launch_quant_chunk_pertoken(d_x, a.K, a.T, g_chunk.aq, g_chunk.as, g_chunk.asum, g_chunk.as_tok);
    else
        launch_quant_chunk(d_x, a.K, a.T, g_chunk.aq, g_chunk.as, g_chunk.asum);
    a.x = nullptr;
    a.x_mode = 0;
    a.aq = g_chunk.aq;
    a.as = g_chunk.as;
    a.asum = g_chunk.asum;
}

}  // namespace

int x_gemm_w4a8_fanout(const tq_qmma_weight_t *const *ws, float *const *ys, int count,
                       const int8_t *d_aq, const float *d_as, const int32_t *d_asum, int T,
                       const int *offsets, int segments) {
    if (!ys) return -1;
    GemmArgs a{};
    const int rc = fanout_args(a, ws, count, T, offsets, segments);
    if (rc) return rc;
    ProfScope prof(a.goff[a.count] * 16, a.K, T, a.ksh ? 64 : 4);
    if (!d_aq || !d_as || !d_asum) return -2;
    for (int i = 0; i < count; ++i) {
        if (!ys[i]) return -2;
        a.y[i] = ys[i];
    }
    a.aq = d_aq;
    a.as = d_as;
    a.asum = d_asum;
    launch_gemm(a);
    return 0;
}

// The same projection from fp32 rows: x[T][K] is quantised like x_quantize_act_chunk
// (per_token == 0) or x_quantize_act_chunk_pertoken (per_token != 0) and multiplied in one
// call; for T = 8 the quantiser runs in the GEMM kernel's prologue (one launch). Results are
// bit-identical to staging first and calling x_gemm_w4a8_fanout.
int x_gemm_w4a8_fanout_fused(const tq_qmma_weight_t *const *ws, float *const *ys, int count,
                             const float *d_x, int T, int per_token) {
    if (!ys) return -1;
    GemmArgs a{};
    const int rc = fanout_args(a, ws, count, T, nullptr, 0);
    if (rc) return rc;
    if (!d_x) return -2;
    ProfScope prof(a.goff[a.count] * 16, a.K, T, a.ksh ? 64 : 4);
    for (int i = 0; i < count; ++i) {
        if (!ys[i]) return -2;
        a.y[i] = ys[i];
    }
    set_fused_input(a, d_x, per_token);
    launch_gemm(a);
    return 0;
}

// Fused projection + all-gather of a column shard: this rank's outputs [count][T][M_i] go
// to block `rank` of the gathered buffer [2 halves][world][count][T][M_i] of EVERY rank (peer stores
// from the kernel's epilogue), followed by a flag store; tq_comm_gather_wait() orders later
// work after the arrival of all ranks' blocks. Decode shapes only (the streaming kernel).
namespace {
// d_x != nullptr: the fused-quantiser form (d_aq / d_as / d_asum unused).
int gathered_impl(const tq_qmma_weight_t *const *ws, int count, const int8_t *d_aq, const float *d_as,
                  const int32_t *d_asum, const float *d_x, int per_token, int T,
                  size_t *half_offset_floats) {
    GatherState &g = gather_state();
    if (g.world < 1) return -3;
    GemmArgs a{};
    const int rc = fanout_args(a, ws, count, T, nullptr, 0);
    if (rc) return rc;
    if (d_x ? false : (!d_aq || !d_as || !d_asum)) return -2;
    ProfScope prof(a.goff[a.count] * 16, a.K, T, a.ksh ? 64 : 4);
    size_t block = 0;
    for (int i = 0; i < count; ++i) block += (size_t)T * ws[i]->M;
    // two halves, used alternately: a rank that is one step ahead never overwrites a block
    // its peers may still be reading
    const size_t half = (size_t)((g.step + 1) & 1) * g.world * block;
    size_t off = 0;
    for (int i = 0; i < count; ++i) {
        for (int p = 0; p < g.world; ++p) a.ypeer[p][i] = g.buf[p] + half + (size_t)g.rank * block + off;
        off += (size_t)T * ws[i]->M;
    }
    a.aq = d_aq; a.as = d_as; a.asum = d_asum;
    a.npeer = g.world;
    if (!gemm_stream_covers(a)) return -21;
    if (d_x) set_fused_input(a, d_x, per_token);
    g.step += 1;
    if (half_offset_floats) *half_offset_floats = (size_t)(g.step & 1) * g.world * block;
    launch_gemm_stream(a);
    launch_gather_publish(g.step);
    return 0;
}
}  // namespace

int x_gemm_w4a8_fanout_gathered(const tq_qmma_weight_t *const *ws, int count, const int8_t *d_aq,
                                const float *d_as, const int32_t *d_asum, int T,
                                size_t *half_offset_floats) {
    return gathered_impl(ws, count, d_aq, d_as, d_asum, nullptr, 0, T, half_offset_floats);
}

int x_gemm_w4a8_fanout_gathered_fused(const tq_qmma_weight_t *const *ws, int count, const float *d_x,
                                      int T, int per_token, size_t *half_offset_floats) {
    if (!d_x) return -2;
    return gathered_impl(ws, count, nullptr, nullptr, nullptr, d_x, per_token, T, half_offset_floats);
}

// Per-token activation scales for decode batches (T < 128): several weights that share the
// staged codes, one launch on the tcgen05 decode kernel. Each weight is split like
// x_gemm_w4a8 splits it (choose_gemm_splits), the splits cutting whole weight-scale groups.
int x_gemm_w4a8_fanout_pertoken(const tq_qmma_weight_t *const *ws, float *const *ys, int count,
                                const int8_t *d_aq, const float *d_as_tok, const int32_t *d_asum,
                                int T) {
    if (!ys) return -1;
    GemmArgs a{};
    const int rc = fanout_args(a, ws, count, T, nullptr, 0);
    if (rc) return rc;
    if (!d_aq || !d_as_tok || !d_asum) return -2;
    ProfScope prof(a.goff[a.count] * 16, a.K, T, a.ksh ? 64 : 4);
    for (int i = 0; i < count; ++i) {
        if (!ys[i]) return -2;
        a.y[i] = ys[i];
    }
    a.aq = d_aq;
    a.asum = d_asum;
    a.as_tok = d_as_tok;
    a.mode = 1;
    if (a.T > 64) return -3;
    apply_pertoken_splits(a);
    return launch_gemm(a) ? 0 : -3;
}

// Tensor-parallel form of the fan-out GEMM for decode batches. The weights are column shards
// (x_w4_shard mode 0) of projections with full_rows[i] rows, and each is split like the whole
// projection would be, so a shard's outputs are bit-identical to the same rows of the
// unsharded call. slot < 0: outputs go to ys[i] ([T][M_i], local). slot >= 0: outputs go into
// columns [col_off[i], col_off[i] + M_i) of the registered symmetric [T][ld] matrix `slot` of
// EVERY rank (peer stores from the GEMM's epilogue); the kernel that consumes the matrix
// carries the exchange point (x_quantize_act_chunk*_sync, x_rmsnorm_chunk_sync,
// tq_comm_exchange_sync). d_as_tok != NULL selects per-token activation scales.
int x_gemm_w4a8_fanout_tp(const tq_qmma_weight_t *const *ws, int count, const int8_t *d_aq,
                          const float *d_as, const float *d_as_tok, const int32_t *d_asum, int T,
                          const int *full_rows, float *const *ys, int slot, const size_t *col_off,
                          size_t ld) {
    GemmArgs a{};
    const int rc = fanout_args(a, ws, count, T, nullptr, 0, full_rows);
    if (rc) return rc;
    if (!d_aq || !d_asum || (!d_as && !d_as_tok)) return -2;
    ProfScope prof(a.goff[a.count] * 16, a.K, T, a.ksh ? 64 : 4);
    a.aq = d_aq;
    a.asum = d_asum;
    a.as = d_as;
    if (d_as_tok) {
        a.as_tok = d_as_tok;
        a.mode = 1;
        apply_pertoken_splits(a, full_rows);
    }
    if (slot < 0) {
        if (!ys) return -2;
        for (int i = 0; i < count; ++i) {
            if (!ys[i]) return -2;
            a.y[i] = ys[i];
        }
    } else {
        GatherState &g = gather_state();
        if (g.world < 1 || slot >= 16 || !col_off || !g.sym[slot][g.rank]) return -3;
        a.npeer = g.world;
        for (int i = 0; i < count; ++i) {
            if (col_off[i] + (size_t)ws[i]->M > ld) return -2;
            a.ld[i] = (int)ld;
            for (int p = 0; p < g.world; ++p) a.ypeer[p][i] = g.sym[slot][p] + col_off[i];
        }
    }
    if (a.T == 8 && gemm_ring_covers(a)) {
        launch_gemm_stream(a);
    } else if (gemm_dtc_covers(a)) {
        launch_gemm_dtc(a);
    } else {
        return -21;
    }
    return 0;
}

// The staging and norm kernels behind a scattering projection: the same results as the calls
// without _sync, after this rank's step flag has been published to all ranks and all ranks'
// flags have arrived (bounded wait, status 10032). One exchange point per call.
void x_quantize_act_chunk_sync(const float *d_x, int K, int T, int8_t *d_aq, float *d_as, int32_t *d_asum) {
    if (!d_x || !d_aq || !d_as || !d_asum || K <= 0 || T <= 0 || (K % 32) != 0) return;
    const SyncArgs sa = exchange_point();
    launch_quant_chunk(d_x, K, T, d_aq, d_as, d_asum, &sa);
}

void x_quantize_act_chunk_pertoken_sync(const float *d_x, int K, int T, int8_t *d_aq, float *d_as,
                                        int32_t *d_asum, float *d_as_tok) {
    if (!d_x || !d_aq || !d_as || !d_asum || !d_as_tok || K <= 0 || T <= 0 || (K % 32) != 0) return;
    const SyncArgs sa = exchange_point();
    launch_quant_chunk_pertoken(d_x, K, T, d_aq, d_as, d_asum, d_as_tok, &sa);
}

void x_rmsnorm_chunk_sync(float *d_out, const float *d_in, const uint16_t *d_w, int H, int T, float eps) {
    if (!d_out || !d_in || !d_w || H <= 0 || T <= 0) return;
    const SyncArgs sa = exchange_point();
    launch_rmsnorm_chunk(d_out, d_in, d_w, H, T, eps, &sa);
}

// x_rmsnorm_chunk followed by x_quantize_act_chunk_pertoken of its output, and x_silu_mul
// followed by the same quantiser: one launch for decode batches, the same bits as the two
// calls (own additions: the reference runs the two kernels, xpu/src/kernels_dpas.cpp:
// 1124-1144 and 185-206). sync != 0: the kernel carries the next exchange point.
void x_rmsnorm_quant_chunk_pertoken(float *d_out, const float *d_in, const uint16_t *d_w, int H, int T,
                                    float eps, int8_t *d_aq, float *d_as, int32_t *d_asum, float *d_as_tok,
                                    int sync) {
    if (!d_out || !d_in || !d_w || !d_aq || !d_as || !d_asum || !d_as_tok || H <= 0 || T <= 0 || (H % 32) != 0)
        return;
    if (sync) {
        const SyncArgs sa = exchange_point();
        launch_rmsnorm_quant_chunk_pertoken(d_out, d_in, d_w, H, T, eps, d_aq, d_as, d_asum, d_as_tok, &sa);
    } else {
        launch_rmsnorm_quant_chunk_pertoken(d_out, d_in, d_w, H, T, eps, d_aq, d_as, d_asum, d_as_tok, nullptr);
    }
}

void x_silu_mul_quant_chunk_pertoken(float *d_out, const float *d_gate, const float *d_up, int K, int T,
                                     int8_t *d_aq, float *d_as, int32_t *d_asum, float *d_as_tok) {
    if (!d_out || !d_gate || !d_up || !d_aq || !d_as || !d_asum || !d_as_tok || K <= 0 || T <= 0 || (K % 32) != 0)
        return;
    launch_silu_mul_quant_chunk_pertoken(d_out, d_gate, d_up, K, T, d_aq, d_as, d_asum, d_as_tok);
}

// silu(gate) * up of this rank's column slice [T][n] into columns [col_off, col_off + n) of the
// symmetric [T][ld] matrix `slot` of every rank.
int x_silu_mul_scatter(const float *d_gate, const float *d_up, int T, int n, int slot, size_t col_off,
                       size_t ld) {
    GatherState &g = gather_state();
    if (!d_gate || !d_up || T <= 0 || n <= 0) return -1;
    if (g.world < 1 || slot < 0 || slot >= 16 || !g.sym[slot][g.rank] || col_off + (size_t)n > ld) return -3;
    float *dst[8];
    for (int p = 0; p < g.world; ++p) dst[p] = g.sym[slot][p] + col_off;
    launch_silu_mul_scatter(dst, g.world, d_gate, d_up, T, n, ld);
    return 0;
}

int x_gemm_w4a8(const tq_qmma_weight_t *w, const int8_t *d_aq, const float *d_as,
                const int32_t *d_asum, float *d_y, int T, const int *offsets, int segments) {
    if (!w || !w->s4_ready || w->s4_k16 || !w->d_s4 || !w->d_s4_scale) return -1;
    if (!d_aq || !d_as || !d_asum || !d_y || T <= 0 || (T % 8) != 0) return -2;
    // Unsplit large-T calls go to the tcgen05 kernel when it covers the shape.
    if (offsets == nullptr || segments >= 1) {
        GemmSegments seg{};
        int ms = 1;
        const int rc = build_segments(w->M / 16, w->K / 32, T, offsets, segments, seg, ms);
        if (rc) return rc;
        if (ms == 1) {
            GemmTcArgs t{};
            t.codes = w->d_s4; t.scales = w->d_s4_scale; t.aq = d_aq; t.as = d_as;
            t.as_tok = nullptr; t.asum = d_asum; t.y = d_y; t.M = w->M; t.K = w->K;
            t.ksh = w->s4_k64 ? 1 : 0; t.T = T; t.out_bf16 = 0;
            if (launch_gemm_tc(t) == 0) return 0;
        }
    }
    const tq_qmma_weight_t *ws[1] = {w};
    float *ys[1] = {d_y};
    return x_gemm_w4a8_fanout(ws, ys, 1, d_aq, d_as, d_asum, T, offsets, segments);
}

int x_gemm_w4a8_pertoken(const tq_qmma_weight_t *w, const int8_t *d_aq, const float *d_as_tok,
                         const int32_t *d_asum, void *d_y, int T, int out_bf16) {
    if (!w || !w->s4_ready || w->s4_k16 || !w->d_s4 || !w->d_s4_scale) return -1;
    if (!d_aq || !d_as_tok || !d_asum || !d_y || T <= 0 || (T % 8) != 0) return -2;
    GemmTcArgs t{};
    t.codes = w->d_s4; t.scales = w->d_s4_scale; t.aq = d_aq; t.as = nullptr;
    t.as_tok = d_as_tok; t.asum = d_asum; t.y = d_y; t.M = w->M; t.K = w->K;
    t.ksh = w->s4_k64 ? 1 : 0; t.T = T; t.out_bf16 = out_bf16;
    if (launch_gemm_tc(t) == 0) return 0;
    if (out_bf16) return -3;   // decode batches store fp32
    const tq_qmma_weight_t *ws[1] = {w};
    float *ys[1] = {static_cast<float *>(d_y)};
    return x_gemm_w4a8_fanout_pertoken(ws, ys, 1, d_aq, d_as_tok, d_asum, T);
}

// xpu/src/kernels_dpas.cpp:1124-1144: (1+w) RMSNorm of a chunk of token rows.
void x_rmsnorm_chunk(float *d_out, const float *d_in, const uint16_t *d_w, int H, int T, float eps) {
    if (!d_out || !d_in || !d_w || H <= 0 || T <= 0) return;
    launch_rmsnorm_chunk(d_out, d_in, d_w, H, T, eps);
}

// ---- W4A4 (xpu/src/kernels_dpas.cpp:1495-1571): the tier K64 weights run at prefill -------
void x_quantize_act_chunk_s4(const float *d_x, int K, int T, uint8_t *d_aq4, float *d_as4,
                             int32_t *d_asum4) {
    if (!d_x || !d_aq4 || !d_as4 || !d_asum4 || K <= 0 || T <= 0 || (K % 64) != 0) return;
    launch_quant_chunk_s4(d_x, K, T, d_aq4, d_as4, d_asum4);
}

// One exact int32 dot per (row, token, K64 group) on the tcgen05 kernel: both k-tiles of the
// group accumulate in TMEM before the single fp32 promote. Covers prefill shapes (T >= 128,
// rows a multiple of 128); -3 otherwise.
int x_gemm_w4a4(const tq_qmma_weight_t *w, const uint8_t *d_aq4, const float *d_as4,
                const int32_t *d_asum4, float *d_y, int T) {
    if (!w || !w->s4_ready || !w->s4_k64 || !w->d_s4 || !w->d_s4_scale) return -1;
    if (!d_aq4 || !d_as4 || !d_asum4 || !d_y || T <= 0 || (T % 8) != 0) return -2;
    GemmTcArgs t{};
    t.codes = w->d_s4; t.scales = w->d_s4_scale; t.aq4 = d_aq4; t.as = d_as4;
    t.asum = d_asum4; t.y = d_y; t.M = w->M; t.K = w->K; t.ksh = 1; t.T = T;
    const int rc = launch_gemm_tc(t);
    return rc == 0 ? 0 : -3;
}

// ---- tensor-parallel column shard (xpu/src/kernels_dpas.cpp:450-499, 549-556) ------------
int x_w4_shard(tq_qmma_weight_t *dst, const tq_qmma_weight_t *src, int rank, int tp, int mode,
               const int *groups, int ngroups) {
    if (!dst || !src || !src->s4_ready || !src->d_s4 || !src->d_s4_scale) return -1;
    if (tp < 1 || rank < 0 || rank >= tp) return -2;
    const int ksh = src->s4_k64 ? 1 : 0;
    if (src->s4_k16) return -3;
    const int Kt = src->Kt;
    const int sg = Kt >> ksh;
    if (mode == 1) {
        // Row-parallel (K) shard, kernels_dpas.cpp:501-526: rank takes k-tiles
        // [rank*Kt/tp, (rank+1)*Kt/tp) of every row-group; the ranks' outputs are partial sums
        // (tq_comm_allreduce_sum adds them).
        if (Kt % tp) return -7;
        if (ksh && (Kt / tp) % 2) return -8;       // K64 needs paired tiles
        const int Ktnew = Kt / tp, sgnew = Ktnew >> ksh;
        *dst = *src;
        dst->d_A = nullptr;
        dst->d_block_scale_inv = nullptr;
        dst->K = src->K / tp;
        dst->Kt = Ktnew;
        dst->scale_cols = sgnew;
        dst->d_s4 = static_cast<uint8_t *>(tq_dev_alloc((size_t)src->Mt * Ktnew * 256u, "shard.codes"));
        dst->d_s4_scale =
            static_cast<uint16_t *>(tq_dev_alloc((size_t)src->M * sgnew * 2u, "shard.scales"));
        const size_t kt0 = (size_t)Ktnew * (size_t)rank;
        TQ_CHECK(cudaMemcpy2DAsync(dst->d_s4, (size_t)Ktnew * 256u, src->d_s4 + kt0 * 256u,
                                   (size_t)Kt * 256u, (size_t)Ktnew * 256u, (size_t)src->Mt,
                                   cudaMemcpyDeviceToDevice, stream()));
        TQ_CHECK(cudaMemcpy2DAsync(dst->d_s4_scale, (size_t)sgnew * 32u,
                                   src->d_s4_scale + (kt0 >> ksh) * 16u, (size_t)sg * 32u,
                                   (size_t)sgnew * 32u, (size_t)src->Mt, cudaMemcpyDeviceToDevice,
                                   stream()));
        tq_sync();
        return 0;
    }
    if (mode == 2) {
        // Replicate, kernels_dpas.cpp:527-546: a full copy for this rank.
        *dst = *src;
        dst->d_A = nullptr;
        dst->d_block_scale_inv = nullptr;
        const size_t code_bytes = (size_t)src->Mt * Kt * 256u, scale_bytes = (size_t)src->M * sg * 2u;
        dst->d_s4 = static_cast<uint8_t *>(tq_dev_alloc(code_bytes, "rep.codes"));
        dst->d_s4_scale = static_cast<uint16_t *>(tq_dev_alloc(scale_bytes, "rep.scales"));
        tq_d2d_async(dst->d_s4, src->d_s4, code_bytes);
        tq_d2d_async(dst->d_s4_scale, src->d_s4_scale, scale_bytes);
        tq_sync();
        return 0;
    }
    if (mode != 0) return -9;
    // Column shard (the slicing rule of kernels_dpas.cpp:463-499): the rows are `ngroups`
    // consecutive blocks (one when no list is given, e.g. [gate | up]); each block is cut
    // into tp equal runs of whole 16-row groups and rank r keeps its run of every block, in
    // block order. A row-group's codes and scale lines are contiguous, so a run is one copy
    // of each array.
    const int nblocks = (groups && ngroups > 0) ? ngroups : 1;
    if (nblocks > 8) return -4;
    struct Run { size_t first_group, n_groups; } runs[8];
    {
        long covered = 0;
        for (int b = 0; b < nblocks; ++b) covered += groups && ngroups > 0 ? groups[b] : src->M;
        if (covered != src->M) return -5;
        size_t first = 0;
        for (int b = 0; b < nblocks; ++b) {
            const int rows = groups && ngroups > 0 ? groups[b] : src->M;
            if (rows % (16 * tp)) return -6;
            const size_t per_rank = (size_t)(rows / 16) / (size_t)tp;
            runs[b] = Run{first + per_rank * (size_t)rank, per_rank};
            first += (size_t)(rows / 16);
        }
    }
    *dst = *src;
    dst->d_A = nullptr;
    dst->d_block_scale_inv = nullptr;
    dst->M = src->M / tp;
    dst->Mt = dst->M / 16;
    const size_t code_row = (size_t)Kt * 256u;                    // bytes of codes per row-group
    const size_t scale_row = (size_t)sg * 16u * sizeof(uint16_t); // bytes of scale lines
    uint8_t *codes = static_cast<uint8_t *>(tq_dev_alloc((size_t)dst->Mt * code_row, "shard.codes"));
    uint8_t *scl = static_cast<uint8_t *>(tq_dev_alloc((size_t)dst->Mt * scale_row, "shard.scales"));
    size_t at = 0;                                                // row-groups placed so far
    for (int b = 0; b < nblocks; ++b) {
        const Run &r = runs[b];
        tq_d2d_async(codes + at * code_row, src->d_s4 + r.first_group * code_row, r.n_groups * code_row);
        tq_d2d_async(scl + at * scale_row,
                     reinterpret_cast<const uint8_t *>(src->d_s4_scale) + r.first_group * scale_row,
                     r.n_groups * scale_row);
        at += r.n_groups;
    }
    dst->d_s4 = codes;
    dst->d_s4_scale = reinterpret_cast<uint16_t *>(scl);
    tq_sync();
    return 0;
}

void x_w4_shard_free(tq_qmma_weight_t *w) {
    if (!w) return;
    tq_dev_free(w->d_s4);
    tq_dev_free(w->d_s4_scale);
    w->d_s4 = nullptr;
    w->d_s4_scale = nullptr;
    w->s4_ready = 0;
}

// ---- flat C entry points ---------------------------------------------------------------
extern "C" {

int qwn_x_w4_repack_weight(tq_qmma_weight_t *w) { return x_w4_repack_weight(w); }
int qwn_x_w4_repack_weight_mode(tq_qmma_weight_t *w, int mode) {
    return x_w4_repack_weight_mode(w, mode);
}
void qwn_x_quantize_act_s8(const float *d_x, int K, int8_t *d_q, float *d_scale, int32_t *d_sum) {
    x_quantize_act_s8(d_x, K, d_q, d_scale, d_sum);
}
void qwn_x_prepare_gemv_act_s8(const float *d_x, int K) { x_prepare_gemv_act_s8(d_x, K); }
void qwn_x_silu_mul_quant(float *d_out, const float *d_gate, const float *d_up, int K) {
    x_silu_mul_quant(d_out, d_gate, d_up, K);
}
void qwn_x_prepare_gemv_act_s8_pertoken(const float *d_x, int K) {
    x_prepare_gemv_act_s8_pertoken(d_x, K);
}
void qwn_x_silu_mul_quant_pertoken(float *d_out, const float *d_gate, const float *d_up, int K) {
    x_silu_mul_quant_pertoken(d_out, d_gate, d_up, K);
}
void qwn_x_rmsnorm_quant(float *d_out, const float *d_in, const uint16_t *d_w, int H, float eps) {
    x_rmsnorm_quant(d_out, d_in, d_w, H, eps);
}
int qwn_x_gemv_w4a8(const tq_qmma_weight_t *w, const float *d_x, float *d_y) {
    return x_gemv_w4a8(w, d_x, d_y);
}
int qwn_x_gemv_w4a8_add(const tq_qmma_weight_t *w, const float *d_x, const float *d_residual,
                        float *d_y) {
    return x_gemv_w4a8_add(w, d_x, d_residual, d_y);
}
int qwn_x_gemv_w4a8_prepared(const tq_qmma_weight_t *w, float *d_y, const float *d_residual) {
    return x_gemv_w4a8_prepared(w, d_y, d_residual);
}
int qwn_x_gemv_w4a8_fanout(const tq_qmma_weight_t *const *ws, float *const *ys, int count) {
    return x_gemv_w4a8_fanout(ws, ys, count);
}
int qwn_x_w8_repack_weight(tq_qmma_weight_t *w) { return x_w8_repack_weight(w); }
int qwn_x_gemv_w8a8(const tq_qmma_weight_t *w, const float *d_x, float *d_y) {
    return x_gemv_w8a8(w, d_x, d_y);
}
int qwn_x_gemv_w8a8_add(const tq_qmma_weight_t *w, const float *d_x, const float *d_residual,
                        float *d_y) {
    return x_gemv_w8a8_add(w, d_x, d_residual, d_y);
}
int qwn_x_gemv_w8a8_prepared(const tq_qmma_weight_t *w, float *d_y, const float *d_residual) {
    return x_gemv_w8a8_prepared(w, d_y, d_residual);
}
int qwn_x_gemm_w8a8(const tq_qmma_weight_t *w, const int8_t *d_aq, const float *d_as, float *d_y,
                    int T) {
    return x_gemm_w8a8(w, d_aq, d_as, d_y, T);
}
int qwn_x_gemv_w4a8_fused(const tq_qmma_weight_t *w, const float *d_x, const float *d_residual,
                          float *d_y) {
    return x_gemv_w4a8_fused(w, d_x, d_residual, d_y);
}
int qwn_x_gemv_qmma(const tq_qmma_weight_t *w, const float *d_x, float *d_y) {
    return x_gemv_qmma(w, d_x, d_y);
}
int qwn_x_gemv_qmma_add(const tq_qmma_weight_t *w, const float *d_x, const float *d_residual,
                        float *d_y) {
    return x_gemv_qmma_add(w, d_x, d_residual, d_y);
}
int qwn_x_gemv_qmma_prepared(const tq_qmma_weight_t *w, const float *d_x, float *d_y,
                             const float *d_residual) {
    return x_gemv_qmma_prepared(w, d_x, d_y, d_residual);
}
void qwn_x_silu_mul(float *d_out, const float *d_gate, const float *d_up, int N) {
    x_silu_mul(d_out, d_gate, d_up, N);
}
void qwn_x_add_inplace(float *d_x, const float *d_y, int N) { x_add_inplace(d_x, d_y, N); }
void qwn_x_quantize_act_chunk(const float *d_x, int K, int T, int8_t *d_aq, float *d_as,
                              int32_t *d_asum) {
    x_quantize_act_chunk(d_x, K, T, d_aq, d_as, d_asum);
}
int qwn_x_gemm_w4a8(const tq_qmma_weight_t *w, const int8_t *d_aq, const float *d_as,
                    const int32_t *d_asum, float *d_y, int T, const int *offsets, int segments) {
    return x_gemm_w4a8(w, d_aq, d_as, d_asum, d_y, T, offsets, segments);
}
int qwn_x_w4_shard(tq_qmma_weight_t *dst, const tq_qmma_weight_t *src, int rank, int tp, int mode,
                   const int *groups, int ngroups) {
    return x_w4_shard(dst, src, rank, tp, mode, groups, ngroups);
}
void qwn_x_w4_shard_free(tq_qmma_weight_t *w) { x_w4_shard_free(w); }
int qwn_choose_gemv_splits(int groups) { return tq::choose_gemv_splits(groups); }
int qwn_choose_pertoken_splits(int rgroups, int tgroups, int ktiles, int ksh) {
    return tq::choose_pertoken_splits(rgroups, tgroups, ktiles, ksh);
}
int qwn_choose_gemm_splits(int rgroups, int tgroups, int ktiles) {
    return tq::choose_gemm_splits(rgroups, tgroups, ktiles);
}
int qwn_x_gemm_w4a8_fanout(const tq_qmma_weight_t *const *ws, float *const *ys, int count,
                           const int8_t *d_aq, const float *d_as, const int32_t *d_asum, int T,
                           const int *offsets, int segments) {
    return x_gemm_w4a8_fanout(ws, ys, count, d_aq, d_as, d_asum, T, offsets, segments);
}
void qwn_x_quantize_act_chunk_pertoken(const float *d_x, int K, int T, int8_t *d_aq, float *d_as,
                                       int32_t *d_asum, float *d_as_tok) {
    x_quantize_act_chunk_pertoken(d_x, K, T, d_aq, d_as, d_asum, d_as_tok);
}
int qwn_x_gemm_w4a8_pertoken(const tq_qmma_weight_t *w, const int8_t *d_aq, const float *d_as_tok,
                             const int32_t *d_asum, void *d_y, int T, int out_bf16) {
    return x_gemm_w4a8_pertoken(w, d_aq, d_as_tok, d_asum, d_y, T, out_bf16);
}
int qwn_x_gemm_w4a8_fanout_pertoken(const tq_qmma_weight_t *const *ws, float *const *ys, int count,
                                    const int8_t *d_aq, const float *d_as_tok, const int32_t *d_asum,
                                    int T) {
    return x_gemm_w4a8_fanout_pertoken(ws, ys, count, d_aq, d_as_tok, d_asum, T);
}

void qwn_x_rmsnorm_chunk(float *d_out, const float *d_in, const uint16_t *d_w, int H, int T,
                         float eps) {
    x_rmsnorm_chunk(d_out, d_in, d_w, H, T, eps);
}
void qwn_x_quantize_act_chunk_s4(const float *d_x, int K, int T, uint8_t *d_aq4, float *d_as4,
                                 int32_t *d_asum4) {
    x_quantize_act_chunk_s4(d_x, K, T, d_aq4, d_as4, d_asum4);
}
int qwn_x_gemm_w4a4(const tq_qmma_weight_t *w, const uint8_t *d_aq4, const float *d_as4,
                    const int32_t *d_asum4, float *d_y, int T) {
    return x_gemm_w4a4(w, d_aq4, d_as4, d_asum4, d_y, T);
}

int qwn_x_gemm_w4a8_fanout_fused(const tq_qmma_weight_t *const *ws, float *const *ys, int count,
                                 const float *d_x, int T, int per_token) {
    return x_gemm_w4a8_fanout_fused(ws, ys, count, d_x, T, per_token);
}
int qwn_x_gemm_w4a8_fanout_gathered_fused(const tq_qmma_weight_t *const *ws, int count,
                                          const float *d_x, int T, int per_token,
                                          size_t *half_offset_floats) {
    return x_gemm_w4a8_fanout_gathered_fused(ws, count, d_x, T, per_token, half_offset_floats);
}
int qwn_x_gemm_w4a8_fanout_gathered(const tq_qmma_weight_t *const *ws, int count,
                                    const int8_t *d_aq, const float *d_as, const int32_t *d_asum,
                                    int T, size_t *half_offset_floats) {
    return x_gemm_w4a8_fanout_gathered(ws, count, d_aq, d_as, d_asum, T, half_offset_floats);
}

int qwn_x_gemm_w4a8_fanout_tp(const tq_qmma_weight_t *const *ws, int count, const int8_t *d_aq,
                              const float *d_as, const float *d_as_tok, const int32_t *d_asum, int T,
                              const int *full_rows, float *const *ys, int slot, const size_t *col_off,
                              size_t ld) {
    return x_gemm_w4a8_fanout_tp(ws, count, d_aq, d_as, d_as_tok, d_asum, T, full_rows, ys, slot, col_off, ld);
}
void qwn_x_quantize_act_chunk_sync(const float *d_x, int K, int T, int8_t *d_aq, float *d_as,
                                   int32_t *d_asum) {
    x_quantize_act_chunk_sync(d_x, K, T, d_aq, d_as, d_asum);
}
void qwn_x_quantize_act_chunk_pertoken_sync(const float *d_x, int K, int T, int8_t *d_aq, float *d_as,
                                            int32_t *d_asum, float *d_as_tok) {
    x_quantize_act_chunk_pertoken_sync(d_x, K, T, d_aq, d_as, d_asum, d_as_tok);
}
void qwn_x_rmsnorm_chunk_sync(float *d_out, const float *d_in, const uint16_t *d_w, int H, int T, float eps) {
    x_rmsnorm_chunk_sync(d_out, d_in, d_w, H, T, eps);
}
void qwn_x_rmsnorm_quant_chunk_pertoken(float *d_out, const float *d_in, const uint16_t *d_w, int H, int T,
                                        float eps, int8_t *d_aq, float *d_as, int32_t *d_asum,
                                        float *d_as_tok, int sync) {
    x_rmsnorm_quant_chunk_pertoken(d_out, d_in, d_w, H, T, eps, d_aq, d_as, d_asum, d_as_tok, sync);
}
void qwn_x_silu_mul_quant_chunk_pertoken(float *d_out, const float *d_gate, const float *d_up, int K, int T,
                                         int8_t *d_aq, float *d_as, int32_t *d_asum, float *d_as_tok) {
    x_silu_mul_quant_chunk_pertoken(d_out, d_gate, d_up, K, T, d_aq, d_as, d_asum, d_as_tok);
}
int qwn_x_silu_mul_scatter(const float *d_gate, const float *d_up, int T, int n, int slot, size_t col_off,
                           size_t ld) {
    return x_silu_mul_scatter(d_gate, d_up, T, n, slot, col_off, ld);
}

int qwn_dbg_tile_dots_gemv(const tq_qmma_weight_t *w, int32_t *d_out) {
    if (!d_out) return -1;
    return tq::gemv_prepared_impl(w, nullptr, nullptr, d_out);
}

int qwn_dbg_tile_dots_gemm(const tq_qmma_weight_t *w, const int8_t *d_aq, int T, int32_t *d_out) {
    if (!w || !w->s4_ready || w->s4_k16 || !w->d_s4 || !w->d_s4_scale) return -1;
    if (!d_aq || !d_out || T <= 0 || (T % 8) != 0) return -2;
    tq::GemmArgs a{};
    a.codes[0] = w->d_s4;
    a.scales[0] = w->d_s4_scale;
    a.M[0] = w->M;
    a.goff[0] = 0;
    a.goff[1] = w->M / 16;
    a.count = 1;
    a.aq = d_aq;
    // The dot does not depend on scales or sums; the -8*asum correction does, so the
    // debug launch needs true K32 sums: they are recomputed from the codes below.
    a.K = w->K;
    a.ksh = w->s4_k64 ? 1 : 0;
    a.T = T;
    a.seg[0].count = 1;
    a.seg[0].end[0] = T / 8;
    a.seg[0].split[0] = 1;
    a.max_splits = 1;
    a.dump = d_out;
    const size_t nblk = (size_t)(w->K / 32) * T;
    float *d_as = static_cast<float *>(tq_dev_alloc(nblk * 4, "dbg.as"));
    int32_t *d_asum = static_cast<int32_t *>(tq_dev_alloc(nblk * 4, "dbg.asum"));
    tq_dev_zero(d_as, nblk * 4);
    tq::launch_code_sums(d_aq, nblk, d_asum);
    a.as = d_as;
    a.asum = d_asum;
    tq::launch_gemm(a);
    tq_sync();
    tq_dev_free(d_as);
    tq_dev_free(d_asum);
    return 0;
}

int qwn_dbg_prepared_act(int K, int8_t *d_q, float *d_scale, int32_t *d_sum) {
    tq::ActScratch &s = tq::act_scratch();
    if (K <= 0 || s.prepared_K < K) return -2;
    if (d_q) tq_d2d_async(d_q, s.q, (size_t)K);
    if (d_scale) tq_d2d_async(d_scale, s.scale, (size_t)(K / 32) * 4);
    if (d_sum) tq_d2d_async(d_sum, s.sum16, (size_t)(K / 16) * 4);
    return 0;
}

}  // extern "C"
