// common.cuh — shared host/device helpers of the W4A8 projection library.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include "tq_w4a8.h"

namespace tq {

// ---- host runtime (runtime.cu) ------------------------------------------------
cudaStream_t stream();
void note_error(cudaError_t e, const char *where);
#define TQ_CHECK(expr)                                   \
    do {                                                 \
        cudaError_t e__ = (expr);                        \
        if (e__ != cudaSuccess) ::tq::note_error(e__, #expr); \
    } while (0)
#define TQ_LAUNCH_CHECK(name) ::tq::note_error(cudaGetLastError(), name)

// Prepared activation scratch consumed by the "*_prepared" GEMV and the fan-out
// (the reference's g_act_q / g_act_scale / g_act_sum, kernels_dpas.cpp:130-149).
// qp holds the same codes permuted for the dp4a unpack: inside each 32-byte tile
// the even-k codes come first (position (k>>3)*4 + ((k&7)>>1)), then the odd-k
// codes at +16. sum32 is the K32 sum (both K16 halves added).
struct ActScratch {
    int8_t *q = nullptr;
    int8_t *qp = nullptr;
    float *scale = nullptr;
    int32_t *sum16 = nullptr;
    int32_t *sum32 = nullptr;
    float *norm_partial = nullptr;
    int cap = 0;          // capacity in elements of K
    int prepared_K = 0;   // K of the last prepare (0 = nothing staged)
};
ActScratch &act_scratch();
void ensure_act_scratch(int K);

// Device status word for bounded waits inside kernels (0 = clean), and the wall-clock limit
// of those waits in nanoseconds (tq_set_wait_limit_ms).
int *device_status_word();
unsigned long long wait_limit_ns();

// State of the fused all-gather (comm.cu): buffers and flag words of every rank as mapped
// into this process, set up by tq_comm_gather_setup.
struct GatherState {
    int world = 0, rank = 0;
    float *buf[8] = {};       // rank p's gathered buffer
    int *flag[8] = {};        // rank p's flag array (one int per source rank)
    int step = 0;             // last published step
    float *sym[16][8] = {};   // registered symmetric buffers: [slot][rank]
    int *step_base = nullptr; // device word: steps completed before the current pass
    int pass_syncs = 0;       // exchange points queued since the last tq_comm_exchange_advance
};

// Exchange point carried by the kernel that consumes gathered data (the staging or norm
// kernel behind a scattering projection): its first CTA publishes this rank's step flag to
// every rank behind a system-scope fence - it runs after the projection kernel, peer stores
// included, has completed - and every CTA waits, bounded, for all ranks' flags before it
// reads. The step number is *base + k: base lives in device memory and advances once per
// pass (tq_comm_exchange_advance), so a pass recorded in a CUDA graph can be replayed.
// world == 0: no exchange.
struct SyncArgs {
    int *peer_flag[8];        // this rank's word in every rank's flag array
    const int *mine;          // this rank's flag array
    const int *base;
    int k, world;
    int *status;
    unsigned long long limit_ns;
};
SyncArgs exchange_point();    // the next exchange point of the current pass (comm.cu)
GatherState &gather_state();
// One-warp kernel behind the GEMM on the library stream: stores `step` into this rank's flag
// word on every rank once the GEMM has completed, then waits for every rank's flag.
void launch_gather_publish(int step);

// ---- per-projection timers (runtime.cu) -------------------------------------------
// Times the calls queued on the stream during its lifetime when profiling is on.
bool profile_on();
class ProfScope {
public:
    ProfScope(int M, int K, int T, int tier);
    ~ProfScope();
    ProfScope(const ProfScope &) = delete;
    ProfScope &operator=(const ProfScope &) = delete;

private:
    int index_ = -1;
};
inline int weight_tier(const tq_qmma_weight_t *w) {
    if (!w) return 0;
    if (w->s8_ready) return 8;
    if (!w->s4_ready) return 6;
    return w->s4_k16 ? 16 : (w->s4_k64 ? 64 : 4);
}

// ---- split heuristics (dispatch.cu) --------------------------------------------
int choose_gemv_splits(int groups);
int choose_gemm_splits(int rgroups, int tgroups, int ktiles);
int choose_pertoken_splits(int rgroups, int tgroups, int ktiles, int ksh);

// ---- kernel launchers -----------------------------------------------------------
// quant.cu
void launch_quant_s8(const float *d_x, const float *d_up, float *d_hidden, int K, int8_t *d_q,
                     int8_t *d_qp, float *d_scale, int32_t *d_sum16, int32_t *d_sum32, bool silu);
void launch_quant_s8_pertoken(const float *d_x, const float *d_up, float *d_hidden, int K,
                              int8_t *d_q, int8_t *d_qp, float *d_scale, int32_t *d_sum16,
                              int32_t *d_sum32, float *d_partial, bool silu);
void launch_rmsnorm_quant(float *d_out, const float *d_in, const uint16_t *d_w, int H, float eps,
                          float *d_partial, int8_t *d_q, int8_t *d_qp, float *d_scale,
                          int32_t *d_sum16, int32_t *d_sum32);
void launch_quant_chunk(const float *d_x, int K, int T, int8_t *d_aq, float *d_as, int32_t *d_asum,
                        const SyncArgs *sync = nullptr);
void launch_rmsnorm_chunk(float *d_out, const float *d_in, const uint16_t *d_w, int H, int T,
                          float eps, const SyncArgs *sync = nullptr);
void launch_quant_chunk_s4(const float *d_x, int K, int T, uint8_t *d_aq4, float *d_as4,
                           int32_t *d_asum4);
void launch_quant_chunk_pertoken(const float *d_x, int K, int T, int8_t *d_aq, float *d_as,
                                 int32_t *d_asum, float *d_as_tok, const SyncArgs *sync = nullptr);
// rmsnorm_chunk / silu_mul followed by quant_chunk_pertoken of the result, in one launch for
// decode batches (the intermediate rows are written to d_out as well)
void launch_rmsnorm_quant_chunk_pertoken(float *d_out, const float *d_in, const uint16_t *d_w, int H, int T,
                                         float eps, int8_t *d_aq, float *d_as, int32_t *d_asum,
                                         float *d_as_tok, const SyncArgs *sync = nullptr);
void launch_silu_mul_quant_chunk_pertoken(float *d_out, const float *d_gate, const float *d_up, int K, int T,
                                          int8_t *d_aq, float *d_as, int32_t *d_asum, float *d_as_tok);
// out[p][tok * ld + j] = silu(gate[tok][j]) * up[tok][j] for j < n, into ndst destinations
void launch_silu_mul_scatter(float *const *dst, int ndst, const float *d_gate, const float *d_up, int T,
                             int n, size_t ld);
void launch_code_sums(const int8_t *d_aq, size_t blocks, int32_t *d_asum);
void launch_silu_mul(float *d_out, const float *d_gate, const float *d_up, int N);
void launch_add_inplace(float *d_x, const float *d_y, int N);

// gemv.cu
struct GemvArgs {
    const uint8_t *codes[4];
    const uint16_t *scales[4];
    float *y[4];
    int goff[5];             // row-group prefix over the set
    int count;
    const int8_t *qp;        // permuted codes
    const float *as;
    const int32_t *sum32;
    const int32_t *sum16;    // K16 tier: the two half sums per tile
    int k16;                 // 1 = K16 scale tier (two scale lines per tile; single weight)
    const float *residual;   // single-weight only
    int K, ksh, splits;
    int serial;              // 1 = one serial accumulator (fan-out order), 0 = two accumulators
    int32_t *dump;           // non-null: write int32 tile dots instead of y
    // Fused activation quantisation (x_gemv_w4a8 / _add): when x is set every CTA quantises
    // the fp32 row itself into shared memory and CTA 0 also refreshes the prepared scratch
    // (sq, sqp, sscale, ssum16, ssum32), so the "prepared" state after the call is the same
    // as with a separate x_prepare_gemv_act_s8.
    const float *x;
    int8_t *sq, *sqp;
    float *sscale;
    int32_t *ssum16, *ssum32;
};
void launch_gemv(const GemvArgs &a);

// gemm_mma.cu
struct GemmSegments {
    int count;
    int end[8];     // in 8-token groups
    int split[8];
};
struct GemmArgs {
    const uint8_t *codes[4];
    const uint16_t *scales[4];
    float *y[4];
    int M[4];
    int goff[5];
    int count;
    const int8_t *aq;
    const float *as;
    const int32_t *asum;
    int K, ksh, T;
    // Fused activation quantisation (ring kernel, T = 8): when x is set the kernel quantises the
    // fp32 rows x[T][K] itself (aq / as / asum are not read): x_mode 1 = one scale per
    // (token, K32) block as x_quantize_act_chunk, 2 = one scale per token row as
    // x_quantize_act_chunk_pertoken.
    const float *x;
    int x_mode;
    GemmSegments seg[4];     // per weight (each keeps the splits it would get alone)
    int max_splits;
    int32_t *dump;           // non-null: write int32 tile dots (single weight)
    // Fused all-gather of a column shard (streaming kernels only): when npeer > 0 the
    // output of weight i goes to ypeer[p][i] for every rank p instead of y[i]; the step flag
    // is published by launch_gather_publish (comm.cu) after the GEMM.
    int npeer;
    float *ypeer[8][4];
    // Per-token activation scales (tcgen05 decode kernel only): mode 1 reads as_tok[T] and
    // asum, promotes once per weight-scale group and multiplies by as_tok at the end.
    int mode;
    const float *as_tok;
    // Row stride of y / ypeer in floats (0 = M): a column shard that writes its slice of a
    // wider [T][ld] matrix.
    int ld[4];
};
void launch_gemm_mma(const GemmArgs &a);
// gemm_stream.cu (decode batches: one segment, T <= 64, uniform split count <= 8)
bool gemm_stream_covers(const GemmArgs &a);
bool gemm_ring_covers(const GemmArgs &a);     // the T = 8 ring kernel takes the call
void launch_gemm_stream(const GemmArgs &a);
// gemm_dtc.cu (decode batches on tcgen05: one segment per weight, 8 <= T <= 64)
bool gemm_dtc_covers(const GemmArgs &a);
void launch_gemm_dtc(const GemmArgs &a);
bool decode_prefers_mma();   // TQ_XPU_DECODE_MMA=1: keep decode batches on the mma.sync kernels
int decode_dtc_min_tokens(); // fewest tokens the tcgen05 decode kernel takes by itself (TQ_XPU_DTC_MIN_TOKENS)
// Decode batches in the reference's arithmetic stay on the mma.sync kernels (ring kernel for
// windows of 8 tokens, streaming kernel otherwise): measured on B200 they are 3x faster than
// the tcgen05 decode kernel, whose steps are bound by the issue latency of its barrier and
// tcgen05 instructions, not by the tensor pipe (one tcgen05.mma of kind::i8 costs its issuing
// thread about 150 clocks whatever its N). The tcgen05 kernel takes the per-token calls the
// ring kernel does not (more than 8 tokens) and, with TQ_XPU_DTC_MIN_TOKENS=n, every decode
// batch of at least n tokens. Everything else goes to the general mma kernel. Returns false
// when no kernel takes a per-token call.
inline bool launch_gemm(const GemmArgs &a) {
    const bool dtc = gemm_dtc_covers(a) && !decode_prefers_mma();
    if (dtc && a.T >= decode_dtc_min_tokens()) {
        launch_gemm_dtc(a);
    } else if (a.mode ? gemm_ring_covers(a) : gemm_stream_covers(a)) {
        launch_gemm_stream(a);
    } else if (a.mode) {
        if (!gemm_dtc_covers(a)) return false;
        launch_gemm_dtc(a);
    } else {
        launch_gemm_mma(a);
    }
    return true;
}

// gemm_tc.cu (tcgen05 path, unsplit, per-token or per-block scales)
struct GemmTcArgs {
    const uint8_t *codes;
    const uint16_t *scales;
    const int8_t *aq;
    const uint8_t *aq4;      // W4A4: packed int4 activations per (K64 block, token) instead of aq;
                             // as and asum are then per (K64 block, token)
    const float *as;         // per (kt, tok) scales, or nullptr in per-token mode
    const float *as_tok;     // per-token scales, or nullptr
    const int32_t *asum;
    void *y;
    int M, K, ksh, T;
    int out_bf16;
};
int launch_gemm_tc(const GemmTcArgs &a);   // returns 0, or <0 when the shape is not covered

// gemv_e2m3.cu: the scalar tier of a weight that still holds its E2M3 payload
int launch_gemv_e2m3(const tq_qmma_weight_t *w, const float *d_x, const float *d_residual, float *d_y);

// repack.cu
void launch_w4_repack(const uint8_t *d_payload, const float *d_bs, int scale_cols, int M, int K,
                      int mode, uint8_t *d_codes, uint16_t *d_scales);

// w8a8.cu / repack.cu (W8A8 tier)
void launch_w8_repack(const uint8_t *d_payload, const float *d_bs, int scale_cols, int M, int K,
                      uint8_t *d_codes, uint16_t *d_scales);
void launch_gemv_w8a8(const uint8_t *codes, const uint16_t *scales, const int8_t *q,
                      const float *as, const float *residual, float *y, int M, int K, int splits);
void launch_gemm_w8a8(const uint8_t *codes, const uint16_t *scales, const int8_t *aq,
                      const float *as, float *y, int M, int K, int T);

// ---- device helpers ---------------------------------------------------------------
#ifdef __CUDACC__

// Programmatic dependent launch. A kernel started with launch_pdl may begin while the
// kernel before it on the stream is still running; it must call pdl_wait() before it reads
// anything an earlier kernel wrote and before its first global write (pdl_wait returns
// once every earlier kernel has completed and its writes are visible). What comes before
// pdl_wait may only read data no kernel writes, i.e. the packed weights. pdl_trigger() lets
// the next kernel's CTAs be scheduled as soon as there is room for them.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <class... KArgs, class... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                       Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    TQ_CHECK(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...));
}

// The same for a kernel whose CTAs form thread-block clusters of `cluster` CTAs along x.
template <class... KArgs, class... Args>
inline void launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, unsigned cluster,
                               Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream();
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = cluster;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    TQ_CHECK(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...));
}

// ---- thread-block cluster helpers (distributed shared memory) -----------------------
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Stores v at the address that `local` (a shared-memory address of this CTA) has in CTA
// `rank` of the cluster.
__device__ __forceinline__ void st_cluster_f32(uint32_t local, uint32_t rank, float v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

// The exchange point of a consuming kernel (see SyncArgs); call after pdl_wait().
__device__ __forceinline__ void exchange_sync(const SyncArgs &sa) {
    if (sa.world == 0) return;
    if ((int)threadIdx.x < sa.world) {
        const int step = *sa.base + sa.k;
        if (blockIdx.x == 0 && blockIdx.y == 0) {
            __threadfence_system();
            asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(sa.peer_flag[threadIdx.x]), "r"(step)
                         : "memory");
        }
        unsigned long long t0 = 0;
        for (unsigned polls = 0;; ++polls) {
            int v;
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(sa.mine + threadIdx.x) : "memory");
            if (v - step >= 0) break;
            if ((polls & 255u) == 255u) {
                unsigned long long now;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (t0 == 0) t0 = now;
                else if (now - t0 > sa.limit_ns) {
                    atomicCAS(sa.status, 0, 32);
                    break;
                }
            }
        }
    }
    __syncthreads();
}

// exp() built only from IEEE add/mul/fma so that host and device agree bit-for-bit
// (the reference's sycl::exp is implementation-defined within 3 ulp).
__device__ __forceinline__ float det_expf(float x) {
    if (x != x) return x;
    if (x > 88.72283935546875f) return __int_as_float(0x7F800000);
    if (x < -103.97208404541015625f) return 0.0f;
    const float n = rintf(__fmul_rn(x, 1.44269502162933349609375f));
    float r = fmaf(n, -0.693145751953125f, x);
    r = fmaf(n, -1.428606765330187045e-06f, r);
    float p = 1.9875691500e-4f;
    p = fmaf(p, r, 1.3981999507e-3f);
    p = fmaf(p, r, 8.3334519073e-3f);
    p = fmaf(p, r, 4.1665795894e-2f);
    p = fmaf(p, r, 1.6666665459e-1f);
    p = fmaf(p, r, 5.0000001201e-1f);
    p = fmaf(__fmul_rn(p, r), r, r);
    p = __fadd_rn(p, 1.0f);
    const int ni = (int)n;
    const int n1 = ni / 2, n2 = ni - n1;
    const float s1 = __int_as_float((n1 + 127) << 23);
    const float s2 = __int_as_float((n2 + 127) << 23);
    return __fmul_rn(__fmul_rn(p, s1), s2);
}

__device__ __forceinline__ float silu_mul_f(float g, float up) {
    return __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, det_expf(-g))), up);
}

__device__ __forceinline__ float clampf(float x, float lo, float hi) {
    return fminf(fmaxf(x, lo), hi);   // NaN clamps to lo, as sycl::clamp does on the device
}

// Packed scale word -> fp32 scale and signed 4-bit zero point
// (kernels_dpas.cpp:629-634).
__device__ __forceinline__ void unpack_scale(uint32_t packed, int &zp, float &ws) {
    zp = ((int)(packed << 28)) >> 28;
    ws = __half2float(__ushort_as_half((unsigned short)(packed & 0xFFF0u)));
}

// ---- pieces of the activation quantisers shared by quant.cu and the fused GEMV prologue ----
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
    return v;
}

// Sum inside each 16-lane half (the K16 sums).
__device__ __forceinline__ int half_sum16(int v) {
#pragma unroll
    for (int off = 8; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// Position of code k inside the permuted 32-byte tile (even-k codes, then odd-k).
__device__ __forceinline__ int permuted_pos(int k) {
    return ((k & 1) << 4) + ((k >> 3) << 2) + ((k & 7) >> 1);
}

__device__ __forceinline__ int quantise_one(float v, float s) {
    return (int)clampf(rintf(__fdiv_rn(v, s)), -127.0f, 127.0f);
}

__device__ __forceinline__ uint4 ldg_stream_v4(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_stream_u32(const void *p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

#endif  // __CUDACC__

}  // namespace tq
