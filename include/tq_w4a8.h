/*
 * tq_w4a8.h — boundary of the B200 W4A8 projection library (libforward_qwen_xpu.so).
 *
 * The library is a drop-in for the projection path of knivesysl-xe: the packed
 * weight record, the C++ projection functions and the flat C entry points below
 * keep the reference's names, argument meaning and return codes. Every pointer
 * named d_* is CUDA device memory on the current device; all calls are
 * asynchronous on ONE in-order stream per device (tq_stream()) and are not
 * thread-safe, exactly like the reference's single in-order queue
 * (xpu/src/decode.cpp:74-75, xpu/src/tq_common.hpp:407-409).
 *
 * Each declaration cites the reference interface it replaces.
 */
#ifndef TQ_W4A8_H
#define TQ_W4A8_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Packed weight record. Field order, names and meaning follow
 * xpu/src/tq_common.hpp:49-76 so that a caller's struct can be passed as is.
 * Only the W4 members are read by this library:
 *   M, K, Mt = M/16, Kt = K/32
 *   d_s4        [Mt][Kt][16 rows][16 B]; byte b of a row holds k = 2b (low
 *               nibble) and k = 2b+1 (high nibble), two's-complement int4
 *   d_s4_scale  uint16 [Mt][Kt >> s4_k64][16] (k16 tier: [Mt][2*Kt][16]);
 *               FP16 scale with its low 4 mantissa bits replaced by a signed
 *               4-bit zero point z: weight ~= scale * (q - z)
 *   s4_ready / s4_k16 / s4_k64 select the tier
 * The E2M3 source members (d_A, d_block_scale_inv, block_scaled, e2m3,
 * scale_rows, scale_cols) are read only by the repack entry points. */
typedef struct {
    int M, K, Mt, Kt;
    float inv_scale;
    uint8_t *d_A;
    float *d_block_scale_inv;
    int block_scaled;
    int row_major;
    int word_major;
    int e2m3;
    int e2m1;
    int e2m3_byte;
    int scale_rows;
    int scale_cols;
    uint8_t *d_s4;
    uint16_t *d_s4_scale;
    int s4_ready;
    int s4_k16;
    int s4_k64;
    uint8_t *d_s8;
    uint16_t *d_s8_scale;
    int s8_ready;
} tq_qmma_weight_t;

/* ---- device runtime: replaces tq_q()/tq_dev_* of xpu/src/decode.cpp:86-130 and
 * xpu/src/tq_common.hpp:200-216. Allocation failure aborts with a message, like
 * the reference. tq_stream() returns the cudaStream_t every call is ordered on.
 * tq_dev_alloc, tq_dev_free, tq_h2d, tq_d2h and tq_dev_zero have C++ linkage in the
 * reference (tq_common.hpp:212-216); the library exports them under those mangled names
 * too (csrc/cxx_linkage.cpp), so objects compiled against the reference header link. */
int tq_set_device(int device);            /* one process per GPU: pick it once */
int tq_device(void);
void *tq_stream(void);
void *tq_dev_alloc(size_t bytes, const char *what);
void tq_dev_free(void *p);
void tq_h2d(void *dst, const void *src, size_t bytes);   /* blocking */
void tq_d2h(void *dst, const void *src, size_t bytes);   /* blocking */
void tq_dev_zero(void *dst, size_t bytes);
void tq_dev_fill(void *dst, int byte, size_t bytes);
void tq_sync(void);                        /* wait for the stream; returns after errors are read */
int tq_last_error(void);                   /* sticky: cudaError of the last failed call, or a
                                              device-side wait status (>= 10000); 0 = clean */
/* Every wait inside a kernel (the mbarrier waits of the tcgen05 GEMM, the flag wait of the
 * fused all-gather) gives up after a wall-clock limit, records a status word and lets the
 * kernel return normally; tq_sync() then turns the status into tq_last_error() = 10000 +
 * code (10021-10023: tcgen05 pipeline, 10031: a rank's gather flag never arrived). Data
 * produced by a call whose wait gave up is incomplete: check tq_last_error() after
 * tq_sync() before trusting gathered outputs. The limit is two seconds unless changed here
 * (a rank can legitimately be further behind during a long prefill). tq_clear_error waits
 * for the stream, then clears the sticky error and the device status word. No counterpart
 * in the reference, whose waits are host-side joins (xpu/src/decode.cpp:133-154). */
void tq_set_wait_limit_ms(int ms);
void tq_clear_error(void);
/* Number of tq_dev_alloc calls made so far in this process, by callers and by the library
 * itself (scratch growth): lets a caller verify that a steady-state loop allocates nothing. */
unsigned long long tq_dev_alloc_count(void);
void *tq_host_alloc_pinned(size_t bytes);
void tq_host_free_pinned(void *p);
void tq_h2d_async(void *dst, const void *src, size_t bytes);
void tq_d2h_async(void *dst, const void *src, size_t bytes);
void tq_d2d_async(void *dst, const void *src, size_t bytes);
/* Read-back that overlaps the calls that follow: the copy runs on a second stream once
 * everything queued so far has run, and returns a ticket (0..15, reused in turn; -1 on
 * failure). The library stream does not wait for it; before a later call may overwrite src,
 * pass the ticket to tq_stream_wait_copy(). tq_sync() also waits for these copies. */
int tq_d2h_overlapped(void *dst, const void *src, size_t bytes);
/* The same for an upload (on a third stream, so that both directions can run at once): the
 * copy starts once everything queued so far has run, hence may overwrite a buffer that
 * earlier calls read; pass the ticket to tq_stream_wait_copy() before the call that reads
 * dst. Issued before step i's calls, it brings step i+1's input in while step i runs. */
int tq_h2d_overlapped(void *dst, const void *src, size_t bytes);
void tq_stream_wait_copy(int ticket);
/* CUDA events on tq_stream() for device-side timing. */
void *tq_event_create(void);
void tq_event_destroy(void *ev);
void tq_event_record(void *ev);
float tq_event_elapsed_ms(void *start, void *stop);     /* synchronises on stop */
/* CUDA graph capture of the calls made on tq_stream() between begin and end (the B200
 * counterpart of replaying a recorded command list on the reference's in-order queue): no
 * allocating or blocking call in between, so call every entry point once before capturing.
 * tq_graph_capture_end returns a handle for tq_graph_launch, or NULL on failure. */
int tq_graph_capture_begin(void);
void *tq_graph_capture_end(void);
void tq_graph_launch(void *graph_exec);
void tq_graph_destroy(void *graph_exec);

/* ---- flat C entry points (for ctypes / cgo / JNI style bindings). Each forwards
 * to the C++ function of the same name without the qwn_ prefix. */

/* xpu/src/kernels_dpas.cpp:403-428 (x_w4_repack_weight_mode, x_w4_repack_weight):
 * E2M3 fragment payload -> packed int4 + FP16 scale/zero-point per group.
 * mode 0 = one scale per K32, 1 = per K16, 2 = per K64. Allocates d_s4/d_s4_scale,
 * frees d_A/d_block_scale_inv. Returns 0, -1 (bad record), -2 (M%16 or K%128),
 * -3 (mode 2 with odd Kt). */
int qwn_x_w4_repack_weight(tq_qmma_weight_t *w);
int qwn_x_w4_repack_weight_mode(tq_qmma_weight_t *w, int mode);

/* xpu/src/kernels_dpas.cpp:188-223: fp32[K] -> s8[K], one fp32 scale per K32,
 * one int32 code sum per K16 (d_sum may be NULL). */
void qwn_x_quantize_act_s8(const float *d_x, int K, int8_t *d_q, float *d_scale, int32_t *d_sum);
/* xpu/src/kernels_dpas.cpp:846-849: quantise into the library's prepared scratch. */
void qwn_x_prepare_gemv_act_s8(const float *d_x, int K);
/* xpu/src/kernels_dpas.cpp:851-855: hidden = silu(gate)*up stored to d_out, then
 * staged like x_prepare_gemv_act_s8. Silently returns on bad arguments. */
void qwn_x_silu_mul_quant(float *d_out, const float *d_gate, const float *d_up, int K);
/* xpu/src/kernels_dpas.cpp:866-929: (1+w) RMSNorm stored to d_out plus staging. */
void qwn_x_rmsnorm_quant(float *d_out, const float *d_in, const uint16_t *d_w, int H, float eps);

/* xpu/src/kernels_dpas.cpp:1664-1680 and 586-675: single-row GEMV. The split
 * count follows choose_gemv_splits; y = sum over splits (+ residual).
 * Returns 0, -1 (bad record/pointers), -2 (scratch not prepared for this K). */
int qwn_x_gemv_w4a8(const tq_qmma_weight_t *w, const float *d_x, float *d_y);
int qwn_x_gemv_w4a8_add(const tq_qmma_weight_t *w, const float *d_x, const float *d_residual,
                        float *d_y);
int qwn_x_gemv_w4a8_prepared(const tq_qmma_weight_t *w, float *d_y, const float *d_residual);
/* x_gemv_w4a8 (d_residual == NULL) or x_gemv_w4a8_add in ONE launch: the GEMV quantises the
 * row in its prologue and leaves the prepared scratch as x_prepare_gemv_act_s8 would. Same
 * bits as the two-launch entry points above, which are the faster form on B200 for wide
 * weights; this one serves callers that count launches. No counterpart in the reference. */
int qwn_x_gemv_w4a8_fused(const tq_qmma_weight_t *w, const float *d_x, const float *d_residual,
                          float *d_y);
/* xpu/src/kernels_dpas.cpp:945-1102: up to 4 weights sharing K, tier and the prepared
 * activation in one launch. Returns 0, -1, -2 (tier/K mismatch), -3 (not prepared). */
int qwn_x_gemv_w4a8_fanout(const tq_qmma_weight_t *const *ws, float *const *ys, int count);

/* W8A8 tier (xpu/src/kernels_dpas.cpp:345-395, 558-573, 768-843, 1578-1629, 1682-1726): int8
 * weights d_s8[Mt][Kt][16 rows][32 B] with one plain FP16 scale per (row, K32)
 * d_s8_scale[Mt][Kt][16], no zero point; activations are the W4A8 staging. The repack takes
 * the E2M3 payload like x_w4_repack_weight and sets s8_ready. GEMV: the W4A8 GEMV's two
 * accumulators and split order with term ((float)d * ws) * as[kt]; GEMM: unsplit, one
 * accumulator, (float)d * (ws * as[kt][tok]). Error codes as the W4 entry points. */
int qwn_x_w8_repack_weight(tq_qmma_weight_t *w);
int qwn_x_gemv_w8a8(const tq_qmma_weight_t *w, const float *d_x, float *d_y);
int qwn_x_gemv_w8a8_add(const tq_qmma_weight_t *w, const float *d_x, const float *d_residual,
                        float *d_y);
int qwn_x_gemv_w8a8_prepared(const tq_qmma_weight_t *w, float *d_y, const float *d_residual);
int qwn_x_gemm_w8a8(const tq_qmma_weight_t *w, const int8_t *d_aq, const float *d_as, float *d_y,
                    int T);

/* xpu/src/kernels_core.cpp:164-252: tier dispatchers used by the layer bodies: s8_ready
 * weights go to the W8A8 GEMV, s4_ready ones (K16, K32 or K64 scales) to the W4A8 GEMV, and a
 * weight that still holds its E2M3 payload to the scalar GEMV (return codes -3..-6 as the
 * reference's validation). */
int qwn_x_gemv_qmma(const tq_qmma_weight_t *w, const float *d_x, float *d_y);
int qwn_x_gemv_qmma_add(const tq_qmma_weight_t *w, const float *d_x, const float *d_residual,
                        float *d_y);
int qwn_x_gemv_qmma_prepared(const tq_qmma_weight_t *w, const float *d_x, float *d_y,
                             const float *d_residual);
/* xpu/src/kernels_core.cpp:254-281: the fp32 glue either side of a projection. */
/* xpu/src/kernels_dpas.cpp:1124-1144: out[tok] = x[tok] * rsqrt(mean(x^2) + eps) * (1 + bf16 w)
 * for T rows of H values (the norm in front of a prefill chunk's projections). */
void qwn_x_rmsnorm_chunk(float *d_out, const float *d_in, const uint16_t *d_w, int H, int T,
                         float eps);
void qwn_x_silu_mul(float *d_out, const float *d_gate, const float *d_up, int N);
void qwn_x_add_inplace(float *d_x, const float *d_y, int N);

/* xpu/src/kernels_dpas.cpp:1149-1207: fp32 [T][K] -> aq[kt][tok][32], as[kt][tok],
 * asum[kt][tok]. */
void qwn_x_quantize_act_chunk(const float *d_x, int K, int T, int8_t *d_aq, float *d_as,
                              int32_t *d_asum);
/* xpu/src/kernels_dpas.cpp:1334-1490: Y[T][M] for T % 8 == 0; offsets is HOST memory
 * (segments+1 entries, <= 8 segments, 8-aligned) and keeps each segment's own split-K
 * count. Returns 0, -1 (bad record), -2 (bad arguments). */
int qwn_x_gemm_w4a8(const tq_qmma_weight_t *w, const int8_t *d_aq, const float *d_as,
                    const int32_t *d_asum, float *d_y, int T, const int *offsets, int segments);

/* xpu/src/kernels_dpas.cpp:450-499, 549-556: column (mode 0) shard of a packed weight.
 * Returns 0, -1..-6 as the reference. Mode 1 (kernels_dpas.cpp:501-526) is the row-parallel
 * shard: rank takes k-tiles [rank*Kt/tp, (rank+1)*Kt/tp) of every row-group (-7 if tp does not
 * divide Kt, -8 if a K64 shard would split a tile pair); its outputs are partial sums, added
 * across ranks with tq_comm_allreduce_sum. Mode 2 (527-546) replicates the weight. Other
 * modes: -9. */
int qwn_x_w4_shard(tq_qmma_weight_t *dst, const tq_qmma_weight_t *src, int rank, int tp, int mode,
                   const int *groups, int ngroups);
void qwn_x_w4_shard_free(tq_qmma_weight_t *w);

/* xpu/src/kernels_dpas.cpp:170-173 and 1226-1250: the split heuristics, exported so
 * callers and tests can see the order a result was summed in. */
/* Per-projection timers (the reference's profile_projection, xpu/src/decode.cpp:156-219, which
 * waits for the queue and reads the host clock around each call): with profiling on
 * (TQ_XPU_PROFILE_PROJ=1 in the environment, or tq_profile_enable(1); returns the previous
 * setting) every GEMV / GEMM entry point brackets its launches with a pair of CUDA events, and
 * nothing waits until tq_profile_report, which synchronises, prints one line per
 * (rows, K, tokens, tier) projection and clears the record. rows, when not NULL, receives up to
 * max_rows entries of six doubles {rows, K, tokens, tier, calls, total microseconds}; the
 * return value is the number of distinct projections. tier: 4 / 64 / 16 = W4A8 with K32 /
 * K64 / K16 scales, 8 = W8A8, 6 = scalar E2M3, 44 = W4A4. Calls made while the stream is
 * being captured into a CUDA graph are not timed. */
int tq_profile_enable(int on);
int tq_profile_report(double *rows, int max_rows);
int qwn_choose_gemv_splits(int groups);
int qwn_choose_gemm_splits(int rgroups, int tgroups, int ktiles);
/* Split count of the per-token decode GEMMs (x_gemm_w4a8_fanout_pertoken, x_gemm_w4a8_fanout_tp with
 * d_as_tok; own rule): as many splits as an 8-token call of the same weight, doubled while one
 * split's staged activations (320 bytes per k-tile and 8 tokens) exceed 88 KB; splits cut whole
 * weight-scale groups (ksh = 1: K64). */
int qwn_choose_pertoken_splits(int rgroups, int tgroups, int ktiles, int ksh);

/* ---- additions without a counterpart in the reference ----------------------- */

/* Several weights that share K, tier and one staged activation chunk, as ONE launch
 * (the reference issues one x_gemm_w4a8 per weight, xpu/src/decode.cpp:1859-1862).
 * Each weight keeps the split count it would get alone, so results are bit-identical
 * to per-weight calls. */
int qwn_x_gemm_w4a8_fanout(const tq_qmma_weight_t *const *ws, float *const *ys, int count,
                           const int8_t *d_aq, const float *d_as, const int32_t *d_asum, int T,
                           const int *offsets, int segments);
/* The fan-out GEMM from fp32 rows x[T][K]: quantised like x_quantize_act_chunk (per_token == 0)
 * or x_quantize_act_chunk_pertoken (per_token != 0) and multiplied in one call, results
 * bit-identical to staging first and calling x_gemm_w4a8_fanout. For T = 8 the quantiser
 * runs in the GEMM kernel's prologue (one launch, nothing staged in global memory); other
 * shapes stage into a library-owned scratch. No counterpart in the reference (its decode
 * GEMV fuses the quantiser the same way). On B200 the one-launch form is the slower one for
 * a wide projection (34.9 us against 29.7 us for the two calls on 2 x 17408 x 5120 with
 * per-token scales: 148 CTAs fetch the same 160 KB of fp32 rows from L2 at the same moment);
 * it is there for callers that must not keep a staging buffer. */
int qwn_x_gemm_w4a8_fanout_fused(const tq_qmma_weight_t *const *ws, float *const *ys, int count,
                                 const float *d_x, int T, int per_token);
/* Per-token activation scale (absmax/127 over the whole row): same staging layout as
 * x_quantize_act_chunk with the scale replicated into every as[kt][tok], plus the
 * per-token vector d_as_tok[T]. */
void qwn_x_quantize_act_chunk_pertoken(const float *d_x, int K, int T, int8_t *d_aq, float *d_as,
                                       int32_t *d_asum, float *d_as_tok);
/* The decode stagings with a per-token scale: x_prepare_gemv_act_s8 and x_silu_mul_quant with
 * scale = absmax(row) / 127 for every K32 block (the "int8 per token" activation of the
 * benchmark configurations; the reference quantises per (token, K32) block,
 * xpu/src/kernels_dpas.cpp:185-206). The prepared scratch then serves x_gemv_w4a8_prepared,
 * x_gemv_w4a8_fanout and x_gemv_qmma_prepared unchanged. */
void qwn_x_prepare_gemv_act_s8_pertoken(const float *d_x, int K);
void qwn_x_silu_mul_quant_pertoken(float *d_out, const float *d_gate, const float *d_up, int K);
/* GEMM for per-token scales: the int32 dot runs over a whole weight-scale group before
 * the fp32 promote; y = (sum_g (d_g - z*asum_g) * ws_g) * as_tok. out_bf16 != 0 stores
 * bfloat16 instead of fp32. Returns like x_gemm_w4a8. */
int qwn_x_gemm_w4a8_pertoken(const tq_qmma_weight_t *w, const int8_t *d_aq, const float *d_as_tok,
                             const int32_t *d_asum, void *d_y, int T, int out_bf16);
/* The same arithmetic for decode batches (T < 128, fp32 out), up to 4 weights that share the
 * staged codes in one launch (gate|up). Each weight is cut into the split count x_gemm_w4a8
 * gives it (choose_gemm_splits), a split covering whole weight-scale groups
 * [G*s/S, G*(s+1)/S) of the G = K/32 (K32) or K/64 (K64) groups; y = ((0 + p_0) + ... + p_S-1)
 * * as_tok with p_s the split's fma chain (an unsplit weight: y = acc * as_tok).
 * x_gemm_w4a8_pertoken routes here below 128 tokens. Returns -3 for shapes outside 8..64
 * tokens. */
int qwn_x_gemm_w4a8_fanout_pertoken(const tq_qmma_weight_t *const *ws, float *const *ys, int count,
                                    const int8_t *d_aq, const float *d_as_tok, const int32_t *d_asum,
                                    int T);

/* W4A4, the tier the reference runs K64 weights at in prefill (x_quantize_act_chunk_s4 and
 * x_gemm_w4a4, xpu/src/kernels_dpas.cpp:1495-1571). Staging: one block per (token, 64
 * values), codes in [-7, 7] with scale absmax/7, two per byte (byte b of a block's 32 =
 * k 2b low nibble, k 2b+1 high nibble): aq4[(kt64*T+tok)*32+b], as4[kt64*T+tok],
 * asum4[kt64*T+tok]. GEMM: K64 weights only (-1 otherwise); y[tok][n] accumulates
 * (float)(d - z*asum4) * (ws*as4) over the K64 groups in ascending order, d the exact int32
 * dot of the 64 int4 x int4 products. Built for prefill shapes: T >= 128 and rows a multiple
 * of 128, else -3. */
void qwn_x_quantize_act_chunk_s4(const float *d_x, int K, int T, uint8_t *d_aq4, float *d_as4,
                                 int32_t *d_asum4);
int qwn_x_gemm_w4a4(const tq_qmma_weight_t *w, const uint8_t *d_aq4, const float *d_as4,
                    const int32_t *d_asum4, float *d_y, int T);

/* int32 layer exposed for bit-exact checks: the dot of every (row, k-tile) with the
 * staged activation, produced by the same unpack/dot code as the kernels above.
 * gemv: d[(g*Kt+kt)*16+n] from the prepared scratch; gemm: d[(kt*T+tok)*M+row]. */
int qwn_dbg_tile_dots_gemv(const tq_qmma_weight_t *w, int32_t *d_out);
int qwn_dbg_tile_dots_gemm(const tq_qmma_weight_t *w, const int8_t *d_aq, int T, int32_t *d_out);
/* Copies of the prepared scratch (device->device), for tests: any pointer may be NULL. */
int qwn_dbg_prepared_act(int K, int8_t *d_q, float *d_scale, int32_t *d_sum);

/* Model-free forms of the reference's self-checks and micro-benches
 * (xpu/src/kernels_dpas.cpp:2146-2333, 2613-2693): they take a weight record instead of
 * a layer index of a loaded model. Checks return 0 on pass. */
double qwn_gemv_bench(const tq_qmma_weight_t *w, int iters);              /* us per call */
double qwn_gemm_bench(const tq_qmma_weight_t *w, int tokens, int iters);  /* us per call */
int qwn_gemm_check(const tq_qmma_weight_t *w, int tokens, double *worst_cos, double *worst_rel);
int qwn_specwave_check(const tq_qmma_weight_t *w);
/* xpu/src/kernels_dpas.cpp:2613-2693: column shards concatenated must be bit-identical to the
 * full GEMV (which needs every shard to keep the full weight's split count, as in the
 * reference), row (K) shards' partial outputs added must agree at cos >= 0.9999 (leg skipped
 * where x_w4_shard refuses the split). 0 pass, -4 a leg failed. */
int qwn_shard_check(const tq_qmma_weight_t *w, int tp);
/* xpu/src/kernels_dpas.cpp:2462-2611: a family of projections, each sharded two ways in its
 * intended mode (0 column, 1 row, 2 replicate) with its row blocks (groups + 3*i, ngroups[i]
 * entries; 0 = one block). Returns the number of failures. */
int qwn_shard_check_all(const tq_qmma_weight_t *const *ws, const int *modes, const int *groups,
                        const int *ngroups, int count);
/* xpu/src/kernels_dpas.cpp:2696-2737: scalar E2M3 GEMV (the weight must still hold its payload)
 * against the W4A8 GEMV after repacking in `mode` (0 / 1 / 2; -1 = 2 when TQ_XPU_K64=1 else 0);
 * passes at cos >= 0.99. The weight stays repacked. 0 pass, -2 already repacked, -6 below
 * the gate. */
int qwn_w4_check(tq_qmma_weight_t *w, int mode, double *cos_out, double *max_rel_out);

/* Load-time pieces that need no model file. qwn_tqf_read_qmma: one quantised-matrix record of a
 * TQF1 container (read_qmma, xpu/src/tqf_loader.cpp:186-255: uint32 scale_rows, uint32
 * scale_cols, fp32 block scales, then M/16 * K/32 fragment tiles of 384 bytes) from host memory
 * into a weight record on the device; `flags` are the container's header flags
 * (xpu/src/tq_common.hpp:35-44). 0, or -1 with a message. tq_selector_has / tq_repack_tier_for /
 * qwn_repack_by_policy: the selector grammar and tier policy of xpu/src/tqf_loader.cpp:40-57,
 * 997-1058 (TQ_XPU_W4A8, TQ_XPU_W8, TQ_XPU_W4_K16, TQ_XPU_K64): tier -1 keep E2M3, 8 int8, 1 / 2 /
 * 0 int4 with K16 / K64 / K32 scales; qwn_repack_by_policy returns the applied tier or
 * -100 + rc of the failed repack call. */
/* Weight-format probe (xpu/src/kernels_dpas.cpp:1726-2146, there bound to a model layer): how
 * well eleven candidate low-bit formats reconstruct the E2M3 source of `w` (a record that has
 * not been repacked; nothing is modified). Prints the reference's table; cos_out / rel_out /
 * bits_out, when not NULL, receive eleven values each (cosine, relative L2 error, bits per
 * weight incl. metadata; scheme 9's bits are measured). Returns 0 when the shipped tier
 * (scheme 1: int4 asymmetric, fp16 scale per K32) has the best cosine among the schemes at or
 * below its 4.5 bits, 1 when another one beats it, -1 / -2 / -3 for a bad, an already
 * repacked or a non-E2M3 record. An offline qualification tool. */
int qwn_w4_grid_probe(const tq_qmma_weight_t *w, double *cos_out, double *rel_out, double *bits_out);
int qwn_tqf_read_qmma(const void *bytes, size_t nbytes, int M, int K, uint32_t flags, tq_qmma_weight_t *w,
                      size_t *consumed);
void qwn_tqf_free_qmma(tq_qmma_weight_t *w);
int tq_selector_has(const char *selector, const char *key);
int tq_repack_tier_for(const char *kind);
int qwn_repack_by_policy(tq_qmma_weight_t *w, const char *kind);

/* Issue-rate measurement of tcgen05.mma kind::i8 (M128 x N x K32, int32 accumulators in TMEM,
 * no epilogue) on every SM: the measured dense int8 peak in TOP/s that the prefill GEMM's
 * fractions are quoted against. qwn_tc_int8_probe takes the MMA width n (16..256, multiple of
 * 16), the queue length and the number of accumulators used in turn, and can return SM 0's
 * {issue clocks, clocks to completion}. The reference measures its own roofs with standalone
 * probes (xpu/probe/dpas_probe.cpp); this is the B200 counterpart. */
double qwn_tc_int8_peak(int iters);
double qwn_tc_int8_probe(int n, int iters, int accs, long long *clocks_out);

/* No counterpart in the reference. Same result as qwn_x_gemv_w4a8, for callers that must
 * not trigger a device allocation (pre-allocated serving loops, callers whose memory pool
 * already owns the GPU): the quantised-activation staging lives in a fixed array inside the
 * library's device image (about 80 KiB per GPU, held from load to exit) instead of
 * cudaMalloc'ed scratch, and no allocating call is made. K is limited to
 * qwn_static_max_k() (32768); larger K returns -30 with a message. All calls share that one
 * array: calls ordered on the library's stream are fine, calls made to overlap on the GPU
 * race. The first call on a device resolves the array's address; make it before any stream
 * capture. Other return codes as qwn_x_gemv_w4a8 (-31: the address lookup failed). */
int qwn_x_gemv_w4a8_static(const tq_qmma_weight_t *w, const float *d_x, float *d_y);
int qwn_static_max_k(void);

/* ---- tensor-parallel exchange: one process per GPU, NCCL loaded at run time.
 * Replaces tq_allreduce's role as the only collective (xpu/src/decode.cpp:133-154) with
 * the all-gather a column shard needs. */
int tq_comm_unique_id(void *id128);                       /* rank 0 fills 128 bytes */
int tq_comm_init(const void *id128, int rank, int world);
int tq_comm_allgather(const void *d_send, void *d_recv, size_t bytes_per_rank);
/* Sum of fp32 partial outputs over the ranks: the exchange of a row-parallel (K) shard,
 * x_w4_shard mode 1. In place when d_send == d_recv. NCCL's summation order: equal to the
 * unsharded projection to fp32 rounding, not bit for bit. */
int tq_comm_allreduce_sum(const float *d_send, float *d_recv, size_t count);
/* Fused all-gather over peer memory (no counterpart in the reference). Every rank owns a
 * gathered buffer [2][world][block] (two halves used by alternate calls, so a rank that
 * runs one step ahead never overwrites what its peers still read; the half a call used is
 * returned in *half_offset_floats) and a zeroed flag array int[world] in plain device memory;
 * tq_comm_ipc_export / _open map them into the other ranks' processes (64-byte CUDA IPC
 * handles, exchanged by the host program), tq_comm_gather_setup registers the world's
 * pointers. qwn_x_gemm_w4a8_fanout_gathered then writes this rank's outputs
 * [count][T][M_i] into block `rank` of EVERY rank's buffer from the GEMM epilogue; a one-warp
 * kernel behind the GEMM publishes a step flag to every rank and waits (bounded; status 10031
 * from tq_last_error() if a rank never publishes) for all ranks' flags, so work queued after
 * the call finds the whole gathered block. tq_comm_gather_wait is kept for callers of the
 * earlier two-call form and enqueues nothing. All ranks must make the same sequence of
 * gathered calls. Returns -21 when the shape is not a decode batch. */
int tq_comm_ipc_export(void *d_ptr, void *handle64);
void *tq_comm_ipc_open(const void *handle64);
void tq_comm_ipc_close(void *p);
int tq_comm_gather_setup(void *const *bufs, void *const *flags, int world, int rank);
int tq_comm_gather_wait(void);
int qwn_x_gemm_w4a8_fanout_gathered(const tq_qmma_weight_t *const *ws, int count,
                                    const int8_t *d_aq, const float *d_as, const int32_t *d_asum,
                                    int T, size_t *half_offset_floats);
/* The gathered call from fp32 rows (see qwn_x_gemm_w4a8_fanout_fused). */
int qwn_x_gemm_w4a8_fanout_gathered_fused(const tq_qmma_weight_t *const *ws, int count,
                                          const float *d_x, int T, int per_token,
                                          size_t *half_offset_floats);
/* Tensor-parallel decode chain without a kernel of its own for the exchange (no counterpart in
 * the reference, whose TP forward is not built, xpu/docs/level-up-xpu.md:757-801). Every rank
 * keeps the activations between projections as full [T][ld] fp32 matrices ("symmetric
 * buffers": same size on every rank, mapped into the other ranks with tq_comm_ipc_*, named by
 * a slot with tq_comm_sym_register after tq_comm_gather_setup has set world, rank and flag
 * arrays; bufs[] of that call may repeat any registered buffer). A projection on a column shard
 * writes its output columns into the matrix of EVERY rank from its epilogue
 * (qwn_x_gemm_w4a8_fanout_tp with slot >= 0, qwn_x_silu_mul_scatter); the kernel that reads the
 * matrix next carries the exchange point in its prologue: its first CTA publishes this rank's
 * step flag to all ranks behind a system-scope fence, every CTA waits (bounded; status 10032)
 * for all ranks' flags, then the kernel does the work of its plain namesake. The step number
 * is read from device memory, base + index within the pass; tq_comm_exchange_advance closes a
 * pass, so a pass can be recorded in a CUDA graph and replayed (tq_comm_exchange_rewind
 * restarts the host-side index after recording). All ranks make the same sequence of calls.
 * full_rows[i] = rows of the unsharded projection: the shard is split like the whole weight, so
 * its outputs are bit-identical to those rows of the unsharded call. d_as_tok != NULL selects
 * per-token activation scales (d_as then unused). Returns -21 for shapes outside 8..64 tokens. */
int tq_comm_sym_register(int slot, void *const *ptrs);
int tq_comm_exchange_advance(void);
int tq_comm_exchange_rewind(void);
int tq_comm_exchange_sync(void);
int qwn_x_gemm_w4a8_fanout_tp(const tq_qmma_weight_t *const *ws, int count, const int8_t *d_aq,
                              const float *d_as, const float *d_as_tok, const int32_t *d_asum, int T,
                              const int *full_rows, float *const *ys, int slot, const size_t *col_off,
                              size_t ld);
void qwn_x_quantize_act_chunk_sync(const float *d_x, int K, int T, int8_t *d_aq, float *d_as,
                                   int32_t *d_asum);
void qwn_x_quantize_act_chunk_pertoken_sync(const float *d_x, int K, int T, int8_t *d_aq, float *d_as,
                                            int32_t *d_asum, float *d_as_tok);
void qwn_x_rmsnorm_chunk_sync(float *d_out, const float *d_in, const uint16_t *d_w, int H, int T, float eps);
/* Two decode-batch fusions, each the same bits as the two calls it replaces (own additions;
 * the reference runs the separate kernels, xpu/src/kernels_dpas.cpp:1124-1144, 185-206):
 * x_rmsnorm_chunk then x_quantize_act_chunk_pertoken of its output (sync != 0: the kernel
 * carries the next exchange point, like x_rmsnorm_chunk_sync), and x_silu_mul then the same
 * quantiser. d_out receives the intermediate rows [T][H] / [T][K]. For T <= 32 and rows
 * that divide into K32-aligned slices it is one launch of thread-block clusters (8, 4 or 2
 * CTAs per token, row maxima joined through distributed shared memory). */
void qwn_x_rmsnorm_quant_chunk_pertoken(float *d_out, const float *d_in, const uint16_t *d_w, int H, int T,
                                        float eps, int8_t *d_aq, float *d_as, int32_t *d_asum,
                                        float *d_as_tok, int sync);
void qwn_x_silu_mul_quant_chunk_pertoken(float *d_out, const float *d_gate, const float *d_up, int K, int T,
                                         int8_t *d_aq, float *d_as, int32_t *d_asum, float *d_as_tok);
int qwn_x_silu_mul_scatter(const float *d_gate, const float *d_up, int T, int n, int slot, size_t col_off,
                           size_t ld);
int tq_comm_rank(void);
int tq_comm_world(void);
void tq_comm_destroy(void);

#ifdef __cplusplus
}  /* extern "C" */

/* C++ projection contract, same signatures as xpu/src/tq_common.hpp:386-461. */
int x_w4_repack_weight(tq_qmma_weight_t *w);
int x_w4_repack_weight_mode(tq_qmma_weight_t *w, int mode);
void x_quantize_act_s8(const float *d_x, int K, int8_t *d_q, float *d_scale, int32_t *d_sum);
int x_gemv_w4a8(const tq_qmma_weight_t *w, const float *d_x, float *d_y);
int x_gemv_w4a8_add(const tq_qmma_weight_t *w, const float *d_x, const float *d_residual,
                    float *d_y);
int x_gemv_qmma(const tq_qmma_weight_t *w, const float *d_x, float *d_y);
int x_gemv_qmma_add(const tq_qmma_weight_t *w, const float *d_x, const float *d_residual,
                    float *d_y);
void x_prepare_gemv_act_s8(const float *d_x, int K);
void x_silu_mul_quant(float *d_out, const float *d_gate, const float *d_up, int K);
void x_silu_mul(float *d_out, const float *d_gate, const float *d_up, int N);
void x_rmsnorm_chunk(float *d_out, const float *d_in, const uint16_t *d_w, int H, int T, float eps);
void x_add_inplace(float *d_x, const float *d_y, int N);
void x_rmsnorm_quant(float *d_out, const float *d_in, const uint16_t *d_w, int H, float eps);
int x_gemv_w4a8_fanout(const tq_qmma_weight_t *const *ws, float *const *ys, int count);
void x_quantize_act_chunk(const float *d_x, int K, int T, int8_t *d_aq, float *d_as,
                          int32_t *d_asum);
int x_gemm_w4a8(const tq_qmma_weight_t *w, const int8_t *d_aq, const float *d_as,
                const int32_t *d_asum, float *d_y, int T, const int *offsets = nullptr,
                int segments = 0);
int x_gemv_w4a8_fused(const tq_qmma_weight_t *w, const float *d_x, const float *d_residual,
                      float *d_y);
int x_gemv_w4a8_prepared(const tq_qmma_weight_t *w, float *d_y,
                         const float *d_residual = nullptr);
int x_gemv_qmma_prepared(const tq_qmma_weight_t *w, const float *d_x, float *d_y,
                         const float *d_residual = nullptr);
int x_w4_shard(tq_qmma_weight_t *dst, const tq_qmma_weight_t *src, int rank, int tp, int mode,
               const int *groups, int ngroups);
void x_w4_shard_free(tq_qmma_weight_t *w);
/* additions (see the C section) */
int x_gemm_w4a8_fanout(const tq_qmma_weight_t *const *ws, float *const *ys, int count,
                       const int8_t *d_aq, const float *d_as, const int32_t *d_asum, int T,
                       const int *offsets = nullptr, int segments = 0);
int x_gemm_w4a8_fanout_gathered(const tq_qmma_weight_t *const *ws, int count, const int8_t *d_aq,
                                const float *d_as, const int32_t *d_asum, int T,
                                size_t *half_offset_floats = nullptr);
int x_gemm_w4a8_fanout_fused(const tq_qmma_weight_t *const *ws, float *const *ys, int count,
                             const float *d_x, int T, int per_token);
int x_gemm_w4a8_fanout_gathered_fused(const tq_qmma_weight_t *const *ws, int count, const float *d_x,
                                      int T, int per_token, size_t *half_offset_floats = nullptr);
void x_quantize_act_chunk_pertoken(const float *d_x, int K, int T, int8_t *d_aq, float *d_as,
                                   int32_t *d_asum, float *d_as_tok);
int x_gemm_w4a8_pertoken(const tq_qmma_weight_t *w, const int8_t *d_aq, const float *d_as_tok,
                         const int32_t *d_asum, void *d_y, int T, int out_bf16 = 0);
int x_gemm_w4a8_fanout_pertoken(const tq_qmma_weight_t *const *ws, float *const *ys, int count,
                                const int8_t *d_aq, const float *d_as_tok, const int32_t *d_asum,
                                int T);
int x_gemm_w4a8_fanout_tp(const tq_qmma_weight_t *const *ws, int count, const int8_t *d_aq,
                          const float *d_as, const float *d_as_tok, const int32_t *d_asum, int T,
                          const int *full_rows, float *const *ys, int slot, const size_t *col_off,
                          size_t ld);
void x_quantize_act_chunk_sync(const float *d_x, int K, int T, int8_t *d_aq, float *d_as, int32_t *d_asum);
void x_quantize_act_chunk_pertoken_sync(const float *d_x, int K, int T, int8_t *d_aq, float *d_as,
                                        int32_t *d_asum, float *d_as_tok);
void x_rmsnorm_chunk_sync(float *d_out, const float *d_in, const uint16_t *d_w, int H, int T, float eps);
void x_rmsnorm_quant_chunk_pertoken(float *d_out, const float *d_in, const uint16_t *d_w, int H, int T,
                                    float eps, int8_t *d_aq, float *d_as, int32_t *d_asum, float *d_as_tok,
                                    int sync);
void x_silu_mul_quant_chunk_pertoken(float *d_out, const float *d_gate, const float *d_up, int K, int T,
                                     int8_t *d_aq, float *d_as, int32_t *d_asum, float *d_as_tok);
int x_silu_mul_scatter(const float *d_gate, const float *d_up, int T, int n, int slot, size_t col_off,
                       size_t ld);
void x_prepare_gemv_act_s8_pertoken(const float *d_x, int K);
void x_silu_mul_quant_pertoken(float *d_out, const float *d_gate, const float *d_up, int K);
int x_w8_repack_weight(tq_qmma_weight_t *w);
int x_gemv_w8a8(const tq_qmma_weight_t *w, const float *d_x, float *d_y);
int x_gemv_w8a8_add(const tq_qmma_weight_t *w, const float *d_x, const float *d_residual, float *d_y);
int x_gemv_w8a8_prepared(const tq_qmma_weight_t *w, float *d_y, const float *d_residual = nullptr);
int x_gemm_w8a8(const tq_qmma_weight_t *w, const int8_t *d_aq, const float *d_as, float *d_y, int T);
void x_quantize_act_chunk_s4(const float *d_x, int K, int T, uint8_t *d_aq4, float *d_as4,
                             int32_t *d_asum4);
int x_gemm_w4a4(const tq_qmma_weight_t *w, const uint8_t *d_aq4, const float *d_as4,
                const int32_t *d_asum4, float *d_y, int T);
#endif /* __cplusplus */

#endif /* TQ_W4A8_H */
