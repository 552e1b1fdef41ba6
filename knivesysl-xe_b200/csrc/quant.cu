// quant.cu — activation quantisers of the W4A8 path and the fp32 glue beside them.
//
// All four follow the same per-block rule (xpu/src/kernels_dpas.cpp:203-206,
// 1173-1178): mx = max |v| over a 32-element K block, s = mx > 0 ? mx/127 : 1,
// q = clamp(rint(v / s), -127, 127) with a true division and round-half-even.
// One 32-lane warp owns one K32 block, so the block maximum and the code sums
// are warp shuffles. HBM traffic per block: 128 B in, 32 B codes + 8..16 B
// scale/sums out.
#include "common.cuh"

#include <algorithm>

namespace tq {

namespace {

constexpr int kWarpsPerBlock = 8;

// Decode staging (x_quantize_act_s8 / x_prepare_gemv_act_s8 / x_silu_mul_quant).
template <bool SILU>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
quant_s8_kernel(const float *__restrict__ x, const float *__restrict__ up,
                float *__restrict__ hidden, int blocks, int8_t *__restrict__ q,
                int8_t *__restrict__ qp, float *__restrict__ scale, int32_t *__restrict__ sum16,
                int32_t *__restrict__ sum32) {
    pdl_trigger();   // the next kernel may be scheduled (its weight prefetch, its launch latency)
    pdl_wait();      // ... while this one waits here for everything launched before it
    const int b = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (b >= blocks) return;
    float v = x[b * 32 + lane];
    if (SILU) {
        v = silu_mul_f(v, up[b * 32 + lane]);
        hidden[b * 32 + lane] = v;
    }
    const float mx = warp_max(fabsf(v));
    const float s = (mx > 0.0f) ? __fdiv_rn(mx, 127.0f) : 1.0f;
    const int qv = quantise_one(v, s);
    const int hs = half_sum16(qv);
    if (lane == 0) scale[b] = s;
    if (sum16 && (lane & 15) == 0) sum16[b * 2 + (lane >> 4)] = hs;
    if (sum32) {
        const int other = __shfl_xor_sync(0xffffffffu, hs, 16);
        if (lane == 0) sum32[b] = hs + other;
    }
    if (q) q[b * 32 + lane] = (int8_t)qv;
    if (qp) qp[b * 32 + permuted_pos(lane)] = (int8_t)qv;
}

// Decode staging with ONE scale for the whole row (absmax / 127), replicated into every K32
// slot of the prepared scratch so that the GEMV kernels read it like per-block scales. Two
// small launches spread over the machine (one CTA for the whole row took 14 us at K = 17408):
// the first stores hidden = silu(gate) * up (SILU) and the maximum of each 256 values, the
// second takes the maximum of those maxima (a maximum does not depend on the order) and
// quantises.
template <bool SILU>
__global__ void __launch_bounds__(256)
rowmax_partial_kernel(const float *__restrict__ x, const float *__restrict__ up, float *__restrict__ hidden,
                      int K, float *__restrict__ part) {
    pdl_trigger();
    pdl_wait();
    __shared__ float wmax[8];
    const int i = blockIdx.x * 256 + threadIdx.x;
    float m = -INFINITY;
    if (i < K) {
        float v = x[i];
        if (SILU) {
            v = silu_mul_f(v, up[i]);
            hidden[i] = v;
        }
        m = fabsf(v);
    }
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = wmax[0];
#pragma unroll
        for (int w = 1; w < 8; ++w) t = fmaxf(t, wmax[w]);
        part[blockIdx.x] = t;
    }
}

__global__ void __launch_bounds__(256)
quant_s8_rowscale_kernel(const float *__restrict__ v_in, int K, const float *__restrict__ part, int nblk,
                         int8_t *__restrict__ q, int8_t *__restrict__ qp, float *__restrict__ scale,
                         int32_t *__restrict__ sum16, int32_t *__restrict__ sum32) {
    pdl_trigger();
    pdl_wait();
    __shared__ float s_scale;
    if (threadIdx.x < 32) {
        float t = -INFINITY;
        for (int b = threadIdx.x; b < nblk; b += 32) t = fmaxf(t, part[b]);
        t = warp_max(t);
        if (threadIdx.x == 0) s_scale = (t > 0.0f) ? __fdiv_rn(t, 127.0f) : 1.0f;
    }
    __syncthreads();
    const float s = s_scale;
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= K) return;                      // K % 32 == 0: whole warps leave together
    const int lane = threadIdx.x & 31, b = i >> 5;
    const int qv = quantise_one(v_in[i], s);
    const int hs = half_sum16(qv);
    if (lane == 0) scale[b] = s;
    if ((lane & 15) == 0) sum16[b * 2 + (lane >> 4)] = hs;
    const int other = __shfl_xor_sync(0xffffffffu, hs, 16);
    if (lane == 0) sum32[b] = hs + other;
    q[i] = (int8_t)qv;
    qp[b * 32 + permuted_pos(lane)] = (int8_t)qv;
}

// Sum of squares per 256 elements: xor-butterfly in each warp, then the eight
// warp sums added 0..7 (the order the CPU oracle restates).
__global__ void __launch_bounds__(256)
sumsq_partial_kernel(const float *__restrict__ in, int H, float *__restrict__ part) {
    pdl_trigger();   // the next kernel may be scheduled (its weight prefetch, its launch latency)
    pdl_wait();      // ... while this one waits here for everything launched before it
    __shared__ float wsum[8];
    const int i = blockIdx.x * 256 + threadIdx.x;
    const float v = (i < H) ? in[i] : 0.0f;
    float s = __fmul_rn(v, v);
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, off));
    if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t = __fadd_rn(t, wsum[w]);
        part[blockIdx.x] = t;
    }
}

// Normalise + quantise in one pass (x_rmsnorm_quant, kernels_dpas.cpp:893-928).
__global__ void __launch_bounds__(256)
rmsnorm_quant_kernel(float *__restrict__ out, const float *__restrict__ in,
                     const uint16_t *__restrict__ w, int H, float eps,
                     const float *__restrict__ part, int nblk, int8_t *__restrict__ q,
                     int8_t *__restrict__ qp, float *__restrict__ scale,
                     int32_t *__restrict__ sum16, int32_t *__restrict__ sum32) {
    pdl_trigger();   // the next kernel may be scheduled (its weight prefetch, its launch latency)
    pdl_wait();      // ... while this one waits here for everything launched before it
    __shared__ float s_rms;
    if (threadIdx.x == 0) {
        float sum_sq = 0.0f;
        for (int b = 0; b < nblk; ++b) sum_sq = __fadd_rn(sum_sq, part[b]);
        s_rms = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum_sq, (float)H), eps)));
    }
    __syncthreads();
    const float rms_inv = s_rms;
    const int i = blockIdx.x * 256 + threadIdx.x;
    if (i >= H) return;   // H % 32 == 0, so whole warps leave together
    const int lane = threadIdx.x & 31;
    const float wf = __uint_as_float((uint32_t)w[i] << 16);
    const float v = __fmul_rn(__fmul_rn(in[i], rms_inv), __fadd_rn(1.0f, wf));
    out[i] = v;
    const float mx = warp_max(fabsf(v));
    const float s = (mx > 0.0f) ? __fdiv_rn(mx, 127.0f) : 1.0f;
    const int qv = quantise_one(v, s);
    const int hs = half_sum16(qv);
    const int b = i >> 5;
    if (lane == 0) scale[b] = s;
    if ((lane & 15) == 0) sum16[b * 2 + (lane >> 4)] = hs;
    const int other = __shfl_xor_sync(0xffffffffu, hs, 16);
    if (lane == 0) sum32[b] = hs + other;
    q[i] = (int8_t)qv;
    qp[b * 32 + permuted_pos(lane)] = (int8_t)qv;
}

// Chunk staging (x_quantize_act_chunk): block index blk = kt*T + tok.
// PER_TOKEN: the scale comes from as_tok[tok] instead of the block maximum.
template <bool PER_TOKEN>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
quant_chunk_kernel(const float *__restrict__ x, int K, int T, size_t blocks,
                   int8_t *__restrict__ aq, float *__restrict__ as, int32_t *__restrict__ asum,
                   const float *__restrict__ as_tok, const SyncArgs sync) {
    pdl_trigger();   // the next kernel may be scheduled (its weight prefetch, its launch latency)
    pdl_wait();      // ... while this one waits here for everything launched before it
    exchange_sync(sync);
    const size_t blk = (size_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (blk >= blocks) return;
    const size_t kt = blk / (size_t)T, tok = blk % (size_t)T;
    const float v = x[tok * (size_t)K + kt * 32 + lane];
    float s;
    if (PER_TOKEN) {
        s = as_tok[tok];
    } else {
        const float mx = warp_max(fmaxf(-INFINITY, fabsf(v)));
        s = (mx > 0.0f) ? __fdiv_rn(mx, 127.0f) : 1.0f;
    }
    const int qv = quantise_one(v, s);
    int sum = half_sum16(qv);
    sum += __shfl_xor_sync(0xffffffffu, sum, 16);
    aq[blk * 32 + lane] = (int8_t)qv;
    if (lane == 0) {
        as[blk] = s;
        asum[blk] = sum;
    }
}

// Prefill-sized chunk staging: the same blocks and results as quant_chunk_kernel, laid out for
// bandwidth. Eight lanes own a K32 block (a float4 each: block maximum and code sum are three
// shuffles), a warp takes 128 consecutive values of a token row per unit and four units per
// trip of a grid-stride loop, all four loads issued before the first division. One warp per
// block with a scalar load each, as above, ran 4096 x 5120 at 0.4 TB/s.
template <bool PER_TOKEN>
__global__ void __launch_bounds__(256)
quant_chunk_wide_kernel(const float *__restrict__ x, int K, int T, int8_t *__restrict__ aq,
                        float *__restrict__ as, int32_t *__restrict__ asum,
                        const float *__restrict__ as_tok) {
    pdl_trigger();
    pdl_wait();
    constexpr int kU = 4;
    const int lane = threadIdx.x & 31, sub = lane & 7;
    const int upr = K >> 7;                                  // units per token row (K % 128 == 0)
    const size_t units = (size_t)T * (size_t)upr;
    const size_t nwarps = (size_t)gridDim.x * 8;
    for (size_t u0 = ((size_t)blockIdx.x * 8 + (threadIdx.x >> 5)) * kU; u0 < units; u0 += nwarps * kU) {
        float4 v[kU];
#pragma unroll
        for (int i = 0; i < kU; ++i)
            if (u0 + i < units)
                v[i] = __ldcs(reinterpret_cast<const float4 *>(x + (u0 + i) * 128) + lane);
#pragma unroll
        for (int i = 0; i < kU; ++i) {
            if (u0 + i >= units) break;                      // uniform per warp
            const size_t tok = (u0 + i) / (size_t)upr;
            const size_t kt = ((u0 + i) % (size_t)upr) * 4 + (lane >> 3);
            float s;
            if (PER_TOKEN) {
                s = as_tok[tok];
            } else {
                float mx = fmaxf(fmaxf(-INFINITY, fabsf(v[i].x)), fabsf(v[i].y));
                mx = fmaxf(fmaxf(mx, fabsf(v[i].z)), fabsf(v[i].w));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                s = (mx > 0.0f) ? __fdiv_rn(mx, 127.0f) : 1.0f;
            }
            const int q0 = quantise_one(v[i].x, s), q1 = quantise_one(v[i].y, s);
            const int q2 = quantise_one(v[i].z, s), q3 = quantise_one(v[i].w, s);
            int sum = q0 + q1 + q2 + q3;
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            sum += __shfl_xor_sync(0xffffffffu, sum, 4);
            const size_t blk = kt * (size_t)T + tok;
            reinterpret_cast<uint32_t *>(aq + blk * 32)[sub] =
                (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) |
                ((uint32_t)(q3 & 0xFF) << 24);
            if (sub == 0) {
                as[blk] = s;
                asum[blk] = sum;
            }
        }
    }
}

// x_rmsnorm_chunk (xpu/src/kernels_dpas.cpp:1124-1144): one 256-thread block per token row.
// Thread t adds the squares of elements t, t+256, ... in order; the block sum is a fixed
// binary tree over the 256 partial sums (the reference leaves that order to the SYCL runtime).
__global__ void __launch_bounds__(256)
rmsnorm_chunk_kernel(float *__restrict__ out, const float *__restrict__ in,
                     const uint16_t *__restrict__ w, int H, float eps, const SyncArgs sync) {
    __shared__ float p[256];
    pdl_trigger();
    pdl_wait();
    exchange_sync(sync);
    const int tid = threadIdx.x;
    const float *row = in + (size_t)blockIdx.x * H;
    float ss = 0.0f;
    for (int i = tid; i < H; i += 256) ss = __fadd_rn(ss, __fmul_rn(row[i], row[i]));
    p[tid] = ss;
    __syncthreads();
    for (int stride = 128; stride >= 1; stride >>= 1) {
        if (tid < stride) p[tid] = __fadd_rn(p[tid], p[tid + stride]);
        __syncthreads();
    }
    const float rms_inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(p[0], (float)H), eps)));
    float *dst = out + (size_t)blockIdx.x * H;
    for (int i = tid; i < H; i += 256) {
        const float wf = __uint_as_float((uint32_t)w[i] << 16);
        dst[i] = __fmul_rn(__fmul_rn(row[i], rms_inv), __fadd_rn(1.0f, wf));
    }
}

// W4A4 staging (x_quantize_act_chunk_s4, xpu/src/kernels_dpas.cpp:1149-1193, 1495-1498): one
// warp per (token, 64 values) block blk = kt64*T + tok; lane l quantises k = 2l, 2l+1 to
// [-7, 7] with scale absmax/7 and stores them as one byte (low nibble = even k).
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
quant_chunk_s4_kernel(const float *__restrict__ x, int K, int T, size_t blocks,
                      uint8_t *__restrict__ aq4, float *__restrict__ as4,
                      int32_t *__restrict__ asum4) {
    pdl_trigger();
    pdl_wait();
    const size_t blk = (size_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (blk >= blocks) return;
    const size_t kt = blk / (size_t)T, tok = blk % (size_t)T;
    const float2 v = *reinterpret_cast<const float2 *>(x + tok * (size_t)K + kt * 64 + 2 * lane);
    const float mx = warp_max(fmaxf(fmaxf(-INFINITY, fabsf(v.x)), fabsf(v.y)));
    const float s = (mx > 0.0f) ? __fdiv_rn(mx, 7.0f) : 1.0f;
    const int q0 = (int)clampf(rintf(__fdiv_rn(v.x, s)), -7.0f, 7.0f);
    const int q1 = (int)clampf(rintf(__fdiv_rn(v.y, s)), -7.0f, 7.0f);
    int sum = q0 + q1;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    aq4[blk * 32 + lane] = (uint8_t)((q0 & 0xF) | ((q1 & 0xF) << 4));
    if (lane == 0) {
        as4[blk] = s;
        asum4[blk] = sum;
    }
}

// The same blocks for prefill-sized calls, laid out like quant_chunk_wide_kernel: sixteen lanes
// own a K64 block (a float4 each -> two packed bytes), a warp takes 128 consecutive values of
// a token row per unit and four units per trip.
__global__ void __launch_bounds__(256)
quant_chunk_s4_wide_kernel(const float *__restrict__ x, int K, int T, uint8_t *__restrict__ aq4,
                           float *__restrict__ as4, int32_t *__restrict__ asum4) {
    pdl_trigger();
    pdl_wait();
    constexpr int kU = 4;
    const int lane = threadIdx.x & 31, sub = lane & 15;
    const int upr = K >> 7;
    const size_t units = (size_t)T * (size_t)upr;
    const size_t nwarps = (size_t)gridDim.x * 8;
    for (size_t u0 = ((size_t)blockIdx.x * 8 + (threadIdx.x >> 5)) * kU; u0 < units; u0 += nwarps * kU) {
        float4 v[kU];
#pragma unroll
        for (int i = 0; i < kU; ++i)
            if (u0 + i < units)
                v[i] = __ldcs(reinterpret_cast<const float4 *>(x + (u0 + i) * 128) + lane);
#pragma unroll
        for (int i = 0; i < kU; ++i) {
            if (u0 + i >= units) break;                      // uniform per warp
            const size_t tok = (u0 + i) / (size_t)upr;
            const size_t kt = ((u0 + i) % (size_t)upr) * 2 + (lane >> 4);
            float mx = fmaxf(fmaxf(-INFINITY, fabsf(v[i].x)), fabsf(v[i].y));
            mx = fmaxf(fmaxf(mx, fabsf(v[i].z)), fabsf(v[i].w));
#pragma unroll
            for (int off = 1; off <= 8; off <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
            const float s = (mx > 0.0f) ? __fdiv_rn(mx, 7.0f) : 1.0f;
            const int q0 = (int)clampf(rintf(__fdiv_rn(v[i].x, s)), -7.0f, 7.0f);
            const int q1 = (int)clampf(rintf(__fdiv_rn(v[i].y, s)), -7.0f, 7.0f);
            const int q2 = (int)clampf(rintf(__fdiv_rn(v[i].z, s)), -7.0f, 7.0f);
            const int q3 = (int)clampf(rintf(__fdiv_rn(v[i].w, s)), -7.0f, 7.0f);
            int sum = q0 + q1 + q2 + q3;
#pragma unroll
            for (int off = 1; off <= 8; off <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
            const size_t blk = kt * (size_t)T + tok;
            reinterpret_cast<uint16_t *>(aq4 + blk * 32)[sub] =
                (uint16_t)((q0 & 0xF) | ((q1 & 0xF) << 4) | ((q2 & 0xF) << 8) | ((q3 & 0xF) << 12));
            if (sub == 0) {
                as4[blk] = s;
                asum4[blk] = sum;
            }
        }
    }
}

// Per-token absmax -> scale (one block per token row).
__global__ void __launch_bounds__(256)
token_scale_kernel(const float *__restrict__ x, int K, float *__restrict__ as_tok, const SyncArgs sync) {
    pdl_trigger();   // the next kernel may be scheduled (its weight prefetch, its launch latency)
    pdl_wait();      // ... while this one waits here for everything launched before it
    exchange_sync(sync);
    __shared__ float wmax[8];
    const float *row = x + (size_t)blockIdx.x * K;
    float m = -INFINITY;
    for (int i = threadIdx.x; i < K; i += 256) m = fmaxf(m, fabsf(row[i]));
    m = warp_max(m);
    if ((threadIdx.x & 31) == 0) wmax[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = wmax[0];
#pragma unroll
        for (int w = 1; w < 8; ++w) t = fmaxf(t, wmax[w]);
        as_tok[blockIdx.x] = (t > 0.0f) ? __fdiv_rn(t, 127.0f) : 1.0f;
    }
}

// Small token counts (decode batches): absmax and quantisation of a token row in ONE launch,
// one CTA per token; the row is read twice (the second time from L1/L2). Same arithmetic as
// token_scale_kernel followed by quant_chunk_kernel<true>.
__global__ void __launch_bounds__(1024)
quant_chunk_pertoken_fused_kernel(const float *__restrict__ x, int K, int T,
                                  int8_t *__restrict__ aq, float *__restrict__ as,
                                  int32_t *__restrict__ asum, float *__restrict__ as_tok,
                                  const SyncArgs sync) {
    pdl_trigger();
    pdl_wait();
    exchange_sync(sync);
    __shared__ float wmax[32];
    __shared__ float s_scale;
    const int tok = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float *row = x + (size_t)tok * K;
    float m = -INFINITY;
    const float4 *row4 = reinterpret_cast<const float4 *>(row);     // K % 32 == 0
    for (int i = threadIdx.x; i < (K >> 2); i += 1024) {
        const float4 v = row4[i];
        m = fmaxf(m, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
    m = warp_max(m);
    if (lane == 0) wmax[warp] = m;
    __syncthreads();
    if (warp == 0) {
        const float t = warp_max(wmax[lane]);
        if (lane == 0) {
            const float s = (t > 0.0f) ? __fdiv_rn(t, 127.0f) : 1.0f;
            s_scale = s;
            as_tok[tok] = s;
        }
    }
    __syncthreads();
    const float s = s_scale;
    const int Kt = K >> 5;
    for (int kt = warp; kt < Kt; kt += 32) {
        const float v = row[kt * 32 + lane];
        const int qv = quantise_one(v, s);
        int sum = half_sum16(qv);
        sum += __shfl_xor_sync(0xffffffffu, sum, 16);
        const size_t blk = (size_t)kt * T + tok;
        aq[blk * 32 + lane] = (int8_t)qv;
        if (lane == 0) {
            as[blk] = s;
            asum[blk] = sum;
        }
    }
}

// The same result in one pass for rows of at most 8192 values: a thread keeps its (up to) two
// float4 of the row in registers between the maximum and the quantisation, so the kernel is
// one global round trip, the block reduction and the stores. Eight consecutive lanes hold one
// K32 block; their code sums are added with three shuffles. NT threads with NU float4 each:
// 1024 x 2 for decode batches (shortest chain), 256 x 8 for prefill-sized calls (eight CTAs per
// SM overlap their round trips: 4096 x 5120 in 40 us against 82 us).
template <int NT, int NU>
__global__ void __launch_bounds__(NT)
quant_chunk_pertoken_regs_kernel(const float *__restrict__ x, int K, int T,
                                 int8_t *__restrict__ aq, float *__restrict__ as,
                                 int32_t *__restrict__ asum, float *__restrict__ as_tok,
                                 const SyncArgs sync) {
    pdl_trigger();
    pdl_wait();
    exchange_sync(sync);
    __shared__ float wmax[NT / 32];
    __shared__ float s_scale;
    const int tok = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const float4 *row4 = reinterpret_cast<const float4 *>(x + (size_t)tok * K);
    const int n4 = K >> 2;
    float4 v[NU];
    float m = -INFINITY;
#pragma unroll
    for (int u = 0; u < NU; ++u) {
        const int i = threadIdx.x + u * NT;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < n4) {
            v[u] = row4[i];
            m = fmaxf(m, fmaxf(fmaxf(fabsf(v[u].x), fabsf(v[u].y)), fmaxf(fabsf(v[u].z), fabsf(v[u].w))));
        }
    }
    m = warp_max(m);
    if (lane == 0) wmax[warp] = m;
    __syncthreads();
    if (warp == 0) {
        const float t = warp_max(lane < NT / 32 ? wmax[lane] : -INFINITY);
        if (lane == 0) {
            const float s = (t > 0.0f) ? __fdiv_rn(t, 127.0f) : 1.0f;
            s_scale = s;
            as_tok[tok] = s;
        }
    }
    __syncthreads();
    const float s = s_scale;
#pragma unroll
    for (int u = 0; u < NU; ++u) {
        const int i = threadIdx.x + u * NT;         // float4 index in the row; uniform per warp
        if (i - lane >= n4) break;
        const int q0 = quantise_one(v[u].x, s), q1 = quantise_one(v[u].y, s);
        const int q2 = quantise_one(v[u].z, s), q3 = quantise_one(v[u].w, s);
        int sum = q0 + q1 + q2 + q3;
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
        if (i < n4) {
            const int kt = i >> 3;                   // eight float4 per K32 block
            const size_t blk = (size_t)kt * T + tok;
            const uint32_t packed = (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) |
                                    ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
            reinterpret_cast<uint32_t *>(aq + blk * 32)[i & 7] = packed;
            if ((i & 7) == 0) {
                as[blk] = s;
                asum[blk] = sum;
            }
        }
    }
}

// The same result with a token's row spread over a cluster of C CTAs (grid (C, T), cluster
// (C, 1, 1)): each CTA keeps its K / C values in registers, the CTAs' maxima meet through
// distributed shared memory (every CTA stores its own into all C copies of cmax[], one
// cluster barrier), and each CTA quantises its slice. A maximum does not depend on the order
// it is taken in, so the codes, sums and scales are those of the kernels above, bit for bit;
// a decode batch of 8 tokens now runs on 8 C SMs instead of 8, and a row is read once
// whatever its length.
//
// SRC selects where the row comes from: 0 = x; 1 = the (1+w) RMSNorm of `x` (weights w2),
// every CTA computing the row's sum of squares itself with rmsnorm_chunk_kernel's order of
// additions; 2 = silu(x) * x2. For 1 and 2 the row is also written to `out`, and the result is
// that of the separate kernel followed by the quantiser, bit for bit, in one launch.
struct ClusterSrc {
    const float *x;          // SRC 0: the rows; 1: the rows before the norm; 2: gate
    const float *x2;         // SRC 2: up
    const uint16_t *w;       // SRC 1: bf16 norm weights
    float *out;              // SRC 1, 2: the rows that are quantised
    float eps;
};
template <int SRC>
__global__ void __launch_bounds__(256)
quant_chunk_pertoken_cluster_kernel(const ClusterSrc src, int K, int T,
                                    int8_t *__restrict__ aq, float *__restrict__ as,
                                    int32_t *__restrict__ asum, float *__restrict__ as_tok,
                                    const SyncArgs sync) {
    pdl_trigger();
    pdl_wait();
    exchange_sync(sync);
    __shared__ float wmax[8];
    __shared__ float cmax[8];
    __shared__ float p[256];
    const int C = gridDim.x, c = blockIdx.x, tok = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n4s = (K / C) >> 2;                           // float4 per slice, a multiple of 8
    const size_t row0 = (size_t)tok * K;
    float rms_inv = 0.0f;
    if (SRC == 1) {
        const float *row = src.x + row0;
        float ss = 0.0f;
        for (int i = tid; i < K; i += 256) ss = __fadd_rn(ss, __fmul_rn(row[i], row[i]));
        p[tid] = ss;
        __syncthreads();
        for (int stride = 128; stride >= 1; stride >>= 1) {
            if (tid < stride) p[tid] = __fadd_rn(p[tid], p[tid + stride]);
            __syncthreads();
        }
        rms_inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(p[0], (float)K), src.eps)));
    }
    const float4 *row4 = reinterpret_cast<const float4 *>(src.x + row0) + (size_t)c * n4s;
    float4 v[4];
    float m = -INFINITY;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int i = tid + u * 256;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < n4s) {
            v[u] = row4[i];
            if (SRC == 1) {
                const uint2 w4 = reinterpret_cast<const uint2 *>(src.w)[(size_t)c * n4s + i];   // four bf16
                v[u].x = __fmul_rn(__fmul_rn(v[u].x, rms_inv), __fadd_rn(1.0f, __uint_as_float(w4.x << 16)));
                v[u].y = __fmul_rn(__fmul_rn(v[u].y, rms_inv), __fadd_rn(1.0f, __uint_as_float(w4.x & 0xFFFF0000u)));
                v[u].z = __fmul_rn(__fmul_rn(v[u].z, rms_inv), __fadd_rn(1.0f, __uint_as_float(w4.y << 16)));
                v[u].w = __fmul_rn(__fmul_rn(v[u].w, rms_inv), __fadd_rn(1.0f, __uint_as_float(w4.y & 0xFFFF0000u)));
            }
            if (SRC == 2) {
                const float4 up = (reinterpret_cast<const float4 *>(src.x2 + row0) + (size_t)c * n4s)[i];
                v[u] = make_float4(silu_mul_f(v[u].x, up.x), silu_mul_f(v[u].y, up.y), silu_mul_f(v[u].z, up.z),
                                   silu_mul_f(v[u].w, up.w));
            }
            if (SRC != 0) (reinterpret_cast<float4 *>(src.out + row0) + (size_t)c * n4s)[i] = v[u];
            m = fmaxf(m, fmaxf(fmaxf(fabsf(v[u].x), fabsf(v[u].y)), fmaxf(fabsf(v[u].z), fabsf(v[u].w))));
        }
    }
    m = warp_max(m);
    if (lane == 0) wmax[warp] = m;
    __syncthreads();
    if (warp == 0) {
        const float t = warp_max(lane < 8 ? wmax[lane] : -INFINITY);
        if (lane < C) st_cluster_f32((uint32_t)__cvta_generic_to_shared(&cmax[c]), (uint32_t)lane, t);
    }
    cluster_sync_all();
    float t = cmax[0];
    for (int j = 1; j < C; ++j) t = fmaxf(t, cmax[j]);
    const float s = (t > 0.0f) ? __fdiv_rn(t, 127.0f) : 1.0f;
    if (c == 0 && tid == 0) as_tok[tok] = s;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int i = tid + u * 256;                 // float4 index in the slice; uniform per warp
        if (i - lane >= n4s) break;
        const int q0 = quantise_one(v[u].x, s), q1 = quantise_one(v[u].y, s);
        const int q2 = quantise_one(v[u].z, s), q3 = quantise_one(v[u].w, s);
        int sum = q0 + q1 + q2 + q3;
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
        if (i < n4s) {
            const int gi = c * n4s + i;              // float4 index in the row
            const int kt = gi >> 3;                  // eight float4 per K32 block
            const size_t blk = (size_t)kt * T + tok;
            const uint32_t packed = (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) |
                                    ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
            reinterpret_cast<uint32_t *>(aq + blk * 32)[gi & 7] = packed;
            if ((gi & 7) == 0) {
                as[blk] = s;
                asum[blk] = sum;
            }
        }
    }
}

// The single-row per-token staging (rowmax_partial_kernel + quant_s8_rowscale_kernel) in one
// launch on a cluster of C CTAs: each CTA keeps K / C values of the row in registers, the
// maxima meet through distributed shared memory, and each CTA writes its slice of the
// prepared scratch: linear codes, the permuted tile (a lane's four codes are two even-k and
// two odd-k neighbours there: two 2-byte stores), the scale in every K32 slot, K16 and K32 sums.
template <bool SILU>
__global__ void __launch_bounds__(256)
quant_s8_rowscale_cluster_kernel(const float *__restrict__ x, const float *__restrict__ up,
                                 float *__restrict__ hidden, int K, int8_t *__restrict__ q,
                                 int8_t *__restrict__ qp, float *__restrict__ scale,
                                 int32_t *__restrict__ sum16, int32_t *__restrict__ sum32) {
    pdl_trigger();
    pdl_wait();
    __shared__ float wmax[8];
    __shared__ float cmax[8];
    const int C = gridDim.x, c = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n4s = (K / C) >> 2;                           // float4 per slice, a multiple of 8
    const float4 *row4 = reinterpret_cast<const float4 *>(x) + (size_t)c * n4s;
    float4 v[4];
    float m = -INFINITY;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int i = tid + u * 256;
        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < n4s) {
            v[u] = row4[i];
            if (SILU) {
                const float4 g = (reinterpret_cast<const float4 *>(up) + (size_t)c * n4s)[i];
                v[u] = make_float4(silu_mul_f(v[u].x, g.x), silu_mul_f(v[u].y, g.y), silu_mul_f(v[u].z, g.z),
                                   silu_mul_f(v[u].w, g.w));
                (reinterpret_cast<float4 *>(hidden) + (size_t)c * n4s)[i] = v[u];
            }
            m = fmaxf(m, fmaxf(fmaxf(fabsf(v[u].x), fabsf(v[u].y)), fmaxf(fabsf(v[u].z), fabsf(v[u].w))));
        }
    }
    m = warp_max(m);
    if (lane == 0) wmax[warp] = m;
    __syncthreads();
    if (warp == 0) {
        const float t = warp_max(lane < 8 ? wmax[lane] : -INFINITY);
        if (lane < C) st_cluster_f32((uint32_t)__cvta_generic_to_shared(&cmax[c]), (uint32_t)lane, t);
    }
    cluster_sync_all();
    float t = cmax[0];
    for (int j = 1; j < C; ++j) t = fmaxf(t, cmax[j]);
    const float s = (t > 0.0f) ? __fdiv_rn(t, 127.0f) : 1.0f;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int i = tid + u * 256;                 // float4 index in the slice; uniform per warp
        if (i - lane >= n4s) break;
        const int q0 = quantise_one(v[u].x, s), q1 = quantise_one(v[u].y, s);
        const int q2 = quantise_one(v[u].z, s), q3 = quantise_one(v[u].w, s);
        int sum = q0 + q1 + q2 + q3;
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);                  // K16 half: four lanes
        const int other = __shfl_xor_sync(0xffffffffu, sum, 4);
        if (i < n4s) {
            const int gi = c * n4s + i;              // float4 index in the row
            const int b = gi >> 3, j = gi & 7;       // K32 block, float4 inside it (k = 4j .. 4j+3)
            reinterpret_cast<uint32_t *>(q)[gi] = (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) |
                                                  ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
            uint16_t *tile = reinterpret_cast<uint16_t *>(qp + (size_t)b * 32);
            tile[j] = (uint16_t)((q0 & 0xFF) | ((q2 & 0xFF) << 8));          // permuted_pos(4j), (4j+2)
            tile[8 + j] = (uint16_t)((q1 & 0xFF) | ((q3 & 0xFF) << 8));      // permuted_pos(4j+1), (4j+3)
            if ((j & 3) == 0) sum16[b * 2 + (j >> 2)] = sum;
            if (j == 0) {
                scale[b] = s;
                sum32[b] = sum + other;
            }
        }
    }
}

// K32 code sums of already staged codes (debug helper for the int32 dump).
__global__ void code_sums_kernel(const int8_t *__restrict__ aq, size_t blocks,
                                 int32_t *__restrict__ asum) {
    const size_t blk = (size_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (blk >= blocks) return;
    int v = aq[blk * 32 + (threadIdx.x & 31)];
    v = half_sum16(v);
    v += __shfl_xor_sync(0xffffffffu, v, 16);
    if ((threadIdx.x & 31) == 0) asum[blk] = v;
}

__global__ void silu_mul_kernel(float *__restrict__ out, const float *__restrict__ gate,
                                const float *__restrict__ up, int N) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < N) out[i] = silu_mul_f(gate[i], up[i]);
}

struct ScatterDst {
    float *p[8];
};
// silu(gate) * up of a rank's column slice, stored into the same columns of every rank's
// [T][ld] matrix (plain peer stores; the consumer's exchange point orders them).
__global__ void silu_mul_scatter_kernel(ScatterDst dst, int ndst, const float *__restrict__ gate,
                                        const float *__restrict__ up, int T, int n, size_t ld) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * n) return;
    const int tok = i / n, j = i - tok * n;
    const float v = silu_mul_f(gate[i], up[i]);
    for (int d = 0; d < ndst; ++d) dst.p[d][(size_t)tok * ld + j] = v;
}

__global__ void add_inplace_kernel(float *__restrict__ x, const float *__restrict__ y, int N) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < N) x[i] = __fadd_rn(x[i], y[i]);
}

}  // namespace

void launch_quant_s8(const float *d_x, const float *d_up, float *d_hidden, int K, int8_t *d_q,
                     int8_t *d_qp, float *d_scale, int32_t *d_sum16, int32_t *d_sum32, bool silu) {
    const int blocks = K / 32;
    if (blocks <= 0) return;
    const int grid = (blocks + kWarpsPerBlock - 1) / kWarpsPerBlock;
    if (silu)
        launch_pdl(quant_s8_kernel<true>, dim3(grid), dim3(kWarpsPerBlock * 32), 0, d_x, d_up,
                   d_hidden, blocks, d_q, d_qp, d_scale, d_sum16, d_sum32);
    else
        launch_pdl(quant_s8_kernel<false>, dim3(grid), dim3(kWarpsPerBlock * 32), 0, d_x,
                   (const float *)nullptr, (float *)nullptr, blocks, d_q, d_qp, d_scale, d_sum16,
                   d_sum32);
    TQ_LAUNCH_CHECK("quant_s8_kernel");
}

void launch_quant_s8_pertoken(const float *d_x, const float *d_up, float *d_hidden, int K,
                              int8_t *d_q, int8_t *d_qp, float *d_scale, int32_t *d_sum16,
                              int32_t *d_sum32, float *d_partial, bool silu) {
    if (K < 32) return;
    // one launch on a cluster of 8, 4 or 2 CTAs when the row divides into K32-aligned slices of
    // at most 1024 values (one float4 per thread; on longer rows eight SMs are too few and
    // the two launches below, 68 CTAs at K = 17408, measured faster) and the buffers take
    // vector accesses
    const uintptr_t align16 = reinterpret_cast<uintptr_t>(d_x) | reinterpret_cast<uintptr_t>(d_up) |
                              reinterpret_cast<uintptr_t>(d_hidden);
    if ((align16 & 15) == 0 && (reinterpret_cast<uintptr_t>(d_q) & 3) == 0 &&
        (reinterpret_cast<uintptr_t>(d_qp) & 1) == 0) {
        for (unsigned c = 8; c >= 2; c >>= 1) {
            if (K % (32 * (int)c) || K / (int)c > 1024) continue;
            if (silu)
                launch_pdl_cluster(quant_s8_rowscale_cluster_kernel<true>, dim3(c), dim3(256), c, d_x, d_up,
                                   d_hidden, K, d_q, d_qp, d_scale, d_sum16, d_sum32);
            else
                launch_pdl_cluster(quant_s8_rowscale_cluster_kernel<false>, dim3(c), dim3(256), c, d_x,
                                   (const float *)nullptr, (float *)nullptr, K, d_q, d_qp, d_scale, d_sum16,
                                   d_sum32);
            TQ_LAUNCH_CHECK("quant_s8_rowscale_cluster_kernel");
            return;
        }
    }
    const int nblk = (K + 255) / 256;
    if (silu)
        launch_pdl(rowmax_partial_kernel<true>, dim3(nblk), dim3(256), 0, d_x, d_up, d_hidden, K, d_partial);
    else
        launch_pdl(rowmax_partial_kernel<false>, dim3(nblk), dim3(256), 0, d_x, (const float *)nullptr,
                   (float *)nullptr, K, d_partial);
    TQ_LAUNCH_CHECK("rowmax_partial_kernel");
    launch_pdl(quant_s8_rowscale_kernel, dim3(nblk), dim3(256), 0, silu ? (const float *)d_hidden : d_x, K,
               (const float *)d_partial, nblk, d_q, d_qp, d_scale, d_sum16, d_sum32);
    TQ_LAUNCH_CHECK("quant_s8_rowscale_kernel");
}

void launch_rmsnorm_quant(float *d_out, const float *d_in, const uint16_t *d_w, int H, float eps,
                          float *d_partial, int8_t *d_q, int8_t *d_qp, float *d_scale,
                          int32_t *d_sum16, int32_t *d_sum32) {
    const int nblk = (H + 255) / 256;
    launch_pdl(sumsq_partial_kernel, dim3(nblk), dim3(256), 0, d_in, H, d_partial);
    TQ_LAUNCH_CHECK("sumsq_partial_kernel");
    launch_pdl(rmsnorm_quant_kernel, dim3(nblk), dim3(256), 0, d_out, d_in, d_w, H, eps,
               (const float *)d_partial, nblk, d_q, d_qp, d_scale, d_sum16, d_sum32);
    TQ_LAUNCH_CHECK("rmsnorm_quant_kernel");
}

namespace {
const SyncArgs kNoSync = {};
}

// Prefill-sized calls (64 tokens and more) whose rows split into 128-value units and whose
// buffers take 16-byte loads and 4-byte stores go to the wide kernels.
static bool wide_staging(const float *d_x, int K, int T, const int8_t *d_aq) {
    return T >= 64 && K % 128 == 0 && (reinterpret_cast<uintptr_t>(d_x) & 15) == 0 &&
           (reinterpret_cast<uintptr_t>(d_aq) & 3) == 0;
}
static int sm_count() {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        TQ_CHECK(cudaGetDevice(&dev));
        TQ_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        if (sms <= 0) sms = 148;
    }
    return sms;
}
static unsigned wide_grid(int K, int T) {
    const size_t units = (size_t)T * (size_t)(K >> 7);
    return (unsigned)std::min<size_t>((units + 31) / 32, (size_t)sm_count() * 8);
}

void launch_quant_chunk(const float *d_x, int K, int T, int8_t *d_aq, float *d_as,
                        int32_t *d_asum, const SyncArgs *sync) {
    const size_t blocks = (size_t)(K / 32) * (size_t)T;
    if (!blocks) return;
    if (!sync && wide_staging(d_x, K, T, d_aq)) {
        launch_pdl(quant_chunk_wide_kernel<false>, dim3(wide_grid(K, T)), dim3(256), 0, d_x, K, T, d_aq, d_as,
                   d_asum, (const float *)nullptr);
        TQ_LAUNCH_CHECK("quant_chunk_wide_kernel");
        return;
    }
    const unsigned grid = (unsigned)((blocks + kWarpsPerBlock - 1) / kWarpsPerBlock);
    launch_pdl(quant_chunk_kernel<false>, dim3(grid), dim3(kWarpsPerBlock * 32), 0, d_x, K, T,
               blocks, d_aq, d_as, d_asum, (const float *)nullptr, sync ? *sync : kNoSync);
    TQ_LAUNCH_CHECK("quant_chunk_kernel");
}

void launch_rmsnorm_chunk(float *d_out, const float *d_in, const uint16_t *d_w, int H, int T,
                          float eps, const SyncArgs *sync) {
    launch_pdl(rmsnorm_chunk_kernel, dim3(T), dim3(256), 0, d_out, d_in, d_w, H, eps,
               sync ? *sync : kNoSync);
    TQ_LAUNCH_CHECK("rmsnorm_chunk_kernel");
}

void launch_quant_chunk_s4(const float *d_x, int K, int T, uint8_t *d_aq4, float *d_as4,
                           int32_t *d_asum4) {
    const size_t blocks = (size_t)(K / 64) * (size_t)T;
    if (!blocks) return;
    if (wide_staging(d_x, K, T, reinterpret_cast<const int8_t *>(d_aq4))) {
        launch_pdl(quant_chunk_s4_wide_kernel, dim3(wide_grid(K, T)), dim3(256), 0, d_x, K, T, d_aq4, d_as4,
                   d_asum4);
        TQ_LAUNCH_CHECK("quant_chunk_s4_wide_kernel");
        return;
    }
    const unsigned grid = (unsigned)((blocks + kWarpsPerBlock - 1) / kWarpsPerBlock);
    launch_pdl(quant_chunk_s4_kernel, dim3(grid), dim3(kWarpsPerBlock * 32), 0, d_x, K, T, blocks,
               d_aq4, d_as4, d_asum4);
    TQ_LAUNCH_CHECK("quant_chunk_s4_kernel");
}

// Decode batches: a cluster of 8, 4 or 2 CTAs per token when the row divides into K32-aligned
// slices of at most 4096 values. False: the shape is not covered, nothing was launched.
constexpr int kClusterMaxT = 64;     // above, the per-token and wide kernels measured faster
template <int SRC>
bool launch_quant_cluster(const ClusterSrc &src, int K, int T, int8_t *d_aq, float *d_as, int32_t *d_asum,
                          float *d_as_tok, const SyncArgs &sa) {
    if (T > kClusterMaxT) return false;
    for (unsigned c = 8; c >= 2; c >>= 1) {
        if (K % (32 * (int)c) || K / (int)c > 4096) continue;
        launch_pdl_cluster(quant_chunk_pertoken_cluster_kernel<SRC>, dim3(c, T), dim3(256), c, src, K, T, d_aq,
                           d_as, d_asum, d_as_tok, sa);
        TQ_LAUNCH_CHECK("quant_chunk_pertoken_cluster_kernel");
        return true;
    }
    return false;
}

void launch_rmsnorm_quant_chunk_pertoken(float *d_out, const float *d_in, const uint16_t *d_w, int H, int T,
                                         float eps, int8_t *d_aq, float *d_as, int32_t *d_asum,
                                         float *d_as_tok, const SyncArgs *sync) {
    const SyncArgs sa = sync ? *sync : kNoSync;
    if (launch_quant_cluster<1>(ClusterSrc{d_in, nullptr, d_w, d_out, eps}, H, T, d_aq, d_as, d_asum, d_as_tok, sa))
        return;
    launch_rmsnorm_chunk(d_out, d_in, d_w, H, T, eps, sync);
    launch_quant_chunk_pertoken(d_out, H, T, d_aq, d_as, d_asum, d_as_tok, nullptr);
}

void launch_silu_mul_quant_chunk_pertoken(float *d_out, const float *d_gate, const float *d_up, int K, int T,
                                          int8_t *d_aq, float *d_as, int32_t *d_asum, float *d_as_tok) {
    if (launch_quant_cluster<2>(ClusterSrc{d_gate, d_up, nullptr, d_out, 0.0f}, K, T, d_aq, d_as, d_asum,
                                d_as_tok, kNoSync))
        return;
    launch_silu_mul(d_out, d_gate, d_up, K * T);
    launch_quant_chunk_pertoken(d_out, K, T, d_aq, d_as, d_asum, d_as_tok, nullptr);
}

void launch_quant_chunk_pertoken(const float *d_x, int K, int T, int8_t *d_aq, float *d_as,
                                 int32_t *d_asum, float *d_as_tok, const SyncArgs *sync) {
    const SyncArgs sa = sync ? *sync : kNoSync;
    const size_t blocks = (size_t)(K / 32) * (size_t)T;
    if (!blocks) return;
    if (launch_quant_cluster<0>(ClusterSrc{d_x, nullptr, nullptr, nullptr, 0.0f}, K, T, d_aq, d_as, d_asum,
                                d_as_tok, sa))
        return;
    if (T <= 32 && K <= 8192) {
        launch_pdl(quant_chunk_pertoken_regs_kernel<1024, 2>, dim3(T), dim3(1024), 0, d_x, K, T, d_aq, d_as,
                   d_asum, d_as_tok, sa);
        TQ_LAUNCH_CHECK("quant_chunk_pertoken_regs_kernel");
        return;
    }
    if (T <= 32) {
        launch_pdl(quant_chunk_pertoken_fused_kernel, dim3(T), dim3(1024), 0, d_x, K, T, d_aq, d_as,
                   d_asum, d_as_tok, sa);
        TQ_LAUNCH_CHECK("quant_chunk_pertoken_fused_kernel");
        return;
    }
    if (K <= 8192 && (reinterpret_cast<uintptr_t>(d_x) & 15) == 0 && (reinterpret_cast<uintptr_t>(d_aq) & 3) == 0) {
        // a row fits the registers of one CTA: one pass whatever the token count
        launch_pdl(quant_chunk_pertoken_regs_kernel<256, 8>, dim3(T), dim3(256), 0, d_x, K, T, d_aq, d_as,
                   d_asum, d_as_tok, sa);
        TQ_LAUNCH_CHECK("quant_chunk_pertoken_regs_kernel");
        return;
    }
    launch_pdl(token_scale_kernel, dim3(T), dim3(256), 0, d_x, K, d_as_tok, sa);
    TQ_LAUNCH_CHECK("token_scale_kernel");
    if (wide_staging(d_x, K, T, d_aq)) {
        launch_pdl(quant_chunk_wide_kernel<true>, dim3(wide_grid(K, T)), dim3(256), 0, d_x, K, T, d_aq, d_as,
                   d_asum, (const float *)d_as_tok);
        TQ_LAUNCH_CHECK("quant_chunk_wide_kernel<pertoken>");
        return;
    }
    const unsigned grid = (unsigned)((blocks + kWarpsPerBlock - 1) / kWarpsPerBlock);
    launch_pdl(quant_chunk_kernel<true>, dim3(grid), dim3(kWarpsPerBlock * 32), 0, d_x, K, T,
               blocks, d_aq, d_as, d_asum, (const float *)d_as_tok, kNoSync);
    TQ_LAUNCH_CHECK("quant_chunk_kernel<pertoken>");
}

void launch_code_sums(const int8_t *d_aq, size_t blocks, int32_t *d_asum) {
    if (!blocks) return;
    const unsigned grid = (unsigned)((blocks + kWarpsPerBlock - 1) / kWarpsPerBlock);
    code_sums_kernel<<<grid, kWarpsPerBlock * 32, 0, stream()>>>(d_aq, blocks, d_asum);
    TQ_LAUNCH_CHECK("code_sums_kernel");
}

void launch_silu_mul(float *d_out, const float *d_gate, const float *d_up, int N) {
    silu_mul_kernel<<<(N + 255) / 256, 256, 0, stream()>>>(d_out, d_gate, d_up, N);
    TQ_LAUNCH_CHECK("silu_mul_kernel");
}

void launch_silu_mul_scatter(float *const *dst, int ndst, const float *d_gate, const float *d_up, int T,
                             int n, size_t ld) {
    ScatterDst d{};
    for (int i = 0; i < ndst && i < 8; ++i) d.p[i] = dst[i];
    launch_pdl(silu_mul_scatter_kernel, dim3((T * n + 255) / 256), dim3(256), 0, d, ndst, d_gate, d_up, T, n,
               ld);
    TQ_LAUNCH_CHECK("silu_mul_scatter_kernel");
}

void launch_add_inplace(float *d_x, const float *d_y, int N) {
    add_inplace_kernel<<<(N + 255) / 256, 256, 0, stream()>>>(d_x, d_y, N);
    TQ_LAUNCH_CHECK("add_inplace_kernel");
}

}  // namespace tq
