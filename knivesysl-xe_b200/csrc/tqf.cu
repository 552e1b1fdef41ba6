// tqf.cu — the two load-time pieces of the weight path that do not need a whole model file:
// reading one quantised-matrix record of a TQF1 container into a weight record on the device
// (read_qmma, xpu/src/tqf_loader.cpp:186-255), and the repack policy that picks a tier per
// matrix from the environment selectors (xpu/src/tqf_loader.cpp:40-57, 997-1058). The
// container's header, tensor order and non-quantised tensors belong to the model loader and
// are not built.
#include "common.cuh"

#include <string.h>

namespace {

// TQF1 header flags that describe the quantised matrices (xpu/src/tq_common.hpp:35-44).
constexpr uint32_t kFlagBlockScaled = 1u << 5, kFlagRowMajor = 1u << 6, kFlagWordMajor = 1u << 7,
                   kFlagE2M3 = 1u << 8;

bool is_blank(char c) { return c == ' ' || c == '\t'; }

}  // namespace

extern "C" {

// Selector grammar of TQ_XPU_W8 / TQ_XPU_W4_K16 / TQ_XPU_K64: a comma-separated list of
// matrix labels, blanks around an entry ignored, the entry "all" matching every label.
int tq_selector_has(const char *selector, const char *key) {
    if (!selector || !key || !*selector || !*key) return 0;
    const size_t klen = strlen(key);
    for (const char *p = selector; *p;) {
        const char *end = strchr(p, ',');
        if (!end) end = p + strlen(p);
        const char *a = p, *b = end;
        while (a < b && is_blank(*a)) ++a;
        while (b > a && is_blank(b[-1])) --b;
        const size_t n = (size_t)(b - a);
        if ((n == 3 && !memcmp(a, "all", 3)) || (n == klen && !memcmp(a, key, klen))) return 1;
        p = *end ? end + 1 : end;
    }
    return 0;
}

// Tier the policy gives a matrix label ("gate", "up", "down", "q", "k", "v", "o", "in_qkv",
// "in_z", "in_a", "in_b", "out", "lm_head"): -1 keep the E2M3 payload (TQ_XPU_W4A8=0), 8 int8
// (TQ_XPU_W8, default "lm_head"), 1 int4 with K16 scales (TQ_XPU_W4_K16), 2 int4 with K64
// scales (TQ_XPU_K64; "1" means "all"), 0 int4 with K32 scales. W8 wins over K16 wins over K64.
int tq_repack_tier_for(const char *kind) {
    const char *integer = getenv("TQ_XPU_W4A8");
    if (integer && integer[0] == '0') return -1;
    const char *w8 = getenv("TQ_XPU_W8");
    if (tq_selector_has(w8 ? w8 : "lm_head", kind)) return 8;
    if (tq_selector_has(getenv("TQ_XPU_W4_K16"), kind)) return 1;
    const char *k64 = getenv("TQ_XPU_K64");
    if (k64 && k64[0] == '1' && k64[1] == '\0') k64 = "all";
    if (tq_selector_has(k64, kind)) return 2;
    return 0;
}

// Applies the policy to a matrix that still holds its E2M3 payload. Returns the tier that was
// applied (see tq_repack_tier_for), or -100 + rc when the repack call failed with rc < 0.
int qwn_repack_by_policy(tq_qmma_weight_t *w, const char *kind) {
    if (!w || !kind) return -101;
    if (!w->d_A) return -102;                 // nothing to repack
    const int tier = tq_repack_tier_for(kind);
    if (tier < 0) return tier;
    const int rc = (tier == 8) ? x_w8_repack_weight(w) : x_w4_repack_weight_mode(w, tier);
    return rc == 0 ? tier : -100 + rc;
}

// One quantised-matrix record: uint32 scale_rows, uint32 scale_cols, scale_rows * scale_cols
// fp32 block scales (dequantisation multipliers), then (M/16) * (K/32) fragment tiles of 384
// bytes. `flags` are the container's header flags. Fills the record's shape and format fields,
// uploads both arrays (tq_dev_alloc) and reports the bytes consumed. Returns 0, or -1 with a
// message for a shape, format or size the reader does not accept (as the reference does).
int qwn_tqf_read_qmma(const void *bytes, size_t nbytes, int M, int K, uint32_t flags, tq_qmma_weight_t *w,
                      size_t *consumed) {
    if (!bytes || !w) return -1;
    if (M <= 0 || K <= 0 || (M % 16) || (K % 32)) {
        fprintf(stderr, "tqf: unaligned QMMA shape %dx%d\n", M, K);
        return -1;
    }
    memset(w, 0, sizeof *w);
    w->M = M;
    w->K = K;
    w->Mt = M / 16;
    w->Kt = K / 32;
    w->block_scaled = (flags & kFlagBlockScaled) != 0;
    w->row_major = (flags & kFlagRowMajor) != 0;
    w->word_major = (flags & kFlagWordMajor) != 0;
    w->e2m3 = (flags & kFlagE2M3) != 0;
    if (!w->block_scaled || !w->e2m3) {
        fprintf(stderr, "tqf: only block-scaled dense E2M3 matrices are supported\n");
        return -1;
    }
    const unsigned char *p = static_cast<const unsigned char *>(bytes);
    if (nbytes < 8) {
        fprintf(stderr, "tqf: record truncated in its scale header\n");
        return -1;
    }
    uint32_t rows = 0, cols = 0;
    memcpy(&rows, p, 4);
    memcpy(&cols, p + 4, 4);
    const uint32_t want_rows = (uint32_t)((M + 127) / 128);
    const uint32_t cols128 = (uint32_t)((K + 127) / 128), cols32 = (uint32_t)(K / 32);
    if (rows != want_rows || (cols != cols128 && cols != cols32)) {
        fprintf(stderr, "tqf: invalid block scale shape %ux%u, expected %ux%u (or %u columns)\n", rows, cols,
                want_rows, cols128, cols32);
        return -1;
    }
    const size_t scale_bytes = (size_t)rows * cols * sizeof(float);
    const size_t payload_bytes = (size_t)w->Mt * (size_t)w->Kt * 384u;
    if (nbytes - 8 < scale_bytes || nbytes - 8 - scale_bytes < payload_bytes) {
        fprintf(stderr, "tqf: record truncated: %zu bytes, needs %zu\n", nbytes, 8 + scale_bytes + payload_bytes);
        return -1;
    }
    w->scale_rows = (int)rows;
    w->scale_cols = (int)cols;
    w->inv_scale = 1.0f;
    w->d_block_scale_inv = static_cast<float *>(tq_dev_alloc(scale_bytes, "tqf.block_scale"));
    w->d_A = static_cast<uint8_t *>(tq_dev_alloc(payload_bytes, "tqf.payload"));
    tq_h2d(w->d_block_scale_inv, p + 8, scale_bytes);
    tq_h2d(w->d_A, p + 8 + scale_bytes, payload_bytes);
    if (consumed) *consumed = 8 + scale_bytes + payload_bytes;
    return 0;
}

// Releases whatever tier the record holds (payload, int4 or int8 arrays).
void qwn_tqf_free_qmma(tq_qmma_weight_t *w) {
    if (!w) return;
    tq_dev_free(w->d_A);
    tq_dev_free(w->d_block_scale_inv);
    tq_dev_free(w->d_s4);
    tq_dev_free(w->d_s4_scale);
    tq_dev_free(w->d_s8);
    tq_dev_free(w->d_s8_scale);
    w->d_A = nullptr;
    w->d_block_scale_inv = nullptr;
    w->d_s4 = nullptr;
    w->d_s4_scale = nullptr;
    w->d_s8 = nullptr;
    w->d_s8_scale = nullptr;
    w->s4_ready = w->s8_ready = 0;
}

}  // extern "C"
