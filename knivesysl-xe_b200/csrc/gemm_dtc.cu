// gemm_dtc.cu — batched W4A8 GEMM for decode batches (8..64 tokens) on the sm_100a tensor
// cores: tcgen05.mma kind::i8 with int32 accumulators in tensor memory (TMEM).
//
// Replaces x_gemm_w4a8's split path (xpu/src/kernels_dpas.cpp:1379-1489) for the shapes decode
// uses: Y[tok][n] = sum over the k-tiles of a split, ascending, of
// (float)(d - z*asum) * (ws*as) with d the exact int32 dot of one (row, K32 tile), one fp32
// accumulator per output, splits added 0..S-1 from 0.0f (an unsplit weight stores its
// accumulator untouched): the arithmetic and the order of the reference. MODE 1 is the
// per-token form (one activation scale per token row): the int32 dot runs over a whole
// weight-scale group (K32, or both k-tiles of a K64 group) before the promote
// acc = fma((float)(d - z*asum), ws, acc), and y = (sum of the splits) * as_tok.
//
// The kernel is HBM-bound on the packed weight stream; what has to stay small is the number
// of issue slots per 256-byte tile (16 rows x K32). Mapping: 128 weight rows are the M side
// of the MMA (= 128 TMEM lanes), the tokens the N side (8 tokens ride in an N = 16
// instruction whose upper rows are zero), K = 32 = one k-tile per instruction, so one MMA
// yields the per-k-tile int32 dots of 8 row-groups at once and an epilogue THREAD owns one
// weight row: it unpacks that row's scale once per group and promotes its tokens in packed
// f32x2 pairs, where the mma.sync kernels repeat the scale unpack and the activation loads
// in every lane quad. A task is (weight, 128-row block, token window, K-split); CTAs are
// persistent (one per SM) and take tasks round-robin. Roles, connected by mbarriers over a
// ring of four step slots (a step = two k-tiles; operands in shared memory, accumulators in
// TMEM):
//  * producers (4 warps, thread = weight row): cp.async the row's packed 16 bytes per k-tile
//    (and, spread over the threads, the tokens' int8 codes, scales, code sums and the scale
//    lines of the block) into a private raw ring, four stages ahead, so about 64 KB per SM
//    are in flight; every thread later reads back only what it copied itself, so the raw
//    ring needs no barrier. Per step a thread expands its nibbles to bytes q+8 (two logic
//    ops per word) into the canonical no-swizzle K-major core-matrix layout, re-orders its
//    token's 32 codes the same way (even-k bytes, then odd-k: any fixed permutation of k is
//    exact for an integer dot) and copies its share of the per-token {as, asum} pairs;
//  * one MMA thread: two tcgen05.mma (M128 x N x K32) per step on top of accumulators that
//    were pre-filled with the bit pattern of 12582912.0f, then tcgen05.commit;
//  * epilogue (4 or 8 warps): tcgen05.ld the step's accumulators, re-arm them with one
//    tcgen05.st from registers that hold the bias pattern, and per token pair
//    f = fma(-(z+8), asum, bits - 12582912) (exact), acc = fma(f, ws*as, acc).
// Splits of one row block meet in a global scratch: the warp that arrives last adds the S
// partial tiles in the order 0..S-1. With ndst > 1 the final tile is stored into every
// destination (the fused all-gather of a column shard: plain peer stores).
//
// Every mbarrier wait is bounded; on expiry the kernel records a status word, stops issuing
// work, still frees its TMEM and returns.
#include "tc.cuh"

#include <algorithm>

namespace tq {

namespace {

constexpr int kWaitMma = 41, kWaitEpi = 42, kWaitProd = 43;   // status codes of failed waits

template <int TN>
struct Cfg {
    static constexpr int TNP = TN < 16 ? 16 : TN;        // N of the MMA
    static constexpr int EW = TN >= 32 ? 8 : 4;          // epilogue warps
    static constexpr int CT = TN / (EW / 4);             // tokens per epilogue thread
    static constexpr int NC = CT > 16 ? 16 : CT;         // columns per TMEM load
    static constexpr int RS = TN >= 64 ? 2 : 4;          // steps per raw stage
    static constexpr int KPS = 2 * RS;                   // k-tiles per raw stage
    // step slots (operands in shared memory + accumulators in TMEM): two raw stages' worth, so
    // the producers fill one stage's slots while the other's are multiplied and promoted
    static constexpr int kSlots = 2 * RS;
    static constexpr int kRaw = TN == 32 ? 4 : 5;        // raw ring stages (all but one in flight)
    static constexpr int MW = 4;                         // MMA-issuing warps (steps in turn)
    static constexpr int kThreads = (EW + 4 + MW) * 32;
    // step slot: A[2] expanded weights, B[2] activations, S[2] {as0, as1, asum0, asum1} per
    // token pair, W[2] scale words of the 128 rows
    static constexpr int kA = 4096, kB = TNP * 32, kS = TN * 8, kW = 256;
    static constexpr int kSlotBytes = 2 * (kA + kB + kS + kW);
    static constexpr int kRawW = KPS * 2048, kRawA = KPS * TN * 32, kRawS = KPS * TN * 8,
                         kRawL = KPS * 256;
    static constexpr int kRawBytes = kRawW + kRawA + kRawS + kRawL;
    static constexpr int kSmem = kSlots * kSlotBytes + kRaw * kRawBytes;
    static constexpr int kTmemCols = kSlots * 2 * TNP;   // 256, 256, 512, 512
};

struct DtcParams {
    const uint8_t *codes[4];
    const uint16_t *scales[4];
    float *y[8][4];                  // [destination][weight]
    int ndst;
    int M[4], ld[4], splits[4], rboff[5], toff[5];
    int count;
    const int8_t *aq;
    const float *as;
    const float *as_tok;
    const int32_t *asum;
    int Kt, ksh, T, nwin, ntasks;
    float *part;
    int *cnt;
    int *status;
    unsigned long long wait_ns;
#ifdef TQ_DTC_TRACE
    long long *trace;                // [role 0..2][step][8] clock64 stamps of CTA 0
    int dbg;                         // experiment switches (TQ_DTC_DBG)
#endif
};

#ifdef TQ_DTC_TRACE
#define DTC_DBG(bit) (p.dbg & (bit))
#define DTC_STAMP(role, which)                                                              \
    if (blockIdx.x == 0 && p.trace && it < 256 && (threadIdx.x & 31) == 0 &&                    \
        (role != 0 || warp == 0) && (role != 1 || warp == EW))                              \
        p.trace[((role) * 256 + it) * 8 + (which)] = clock64();
#else
#define DTC_STAMP(role, which)
#define DTC_DBG(bit) false
#endif

struct Task {
    int wi, rb, tw, s, kt0, cnt;
};

// Out of line (and the loops around the roles' inner bodies are not unrolled): the three roles
// run different code on the same SM at once, so the kernel's code has to stay small enough
// for the instruction cache - an early version of 100-190 KB per instantiation spent most of
// its time fetching instructions.
template <int MODE>
__device__ __noinline__ Task decode_task(const DtcParams &p, int t) {
    Task k;
    int wi = 0;
    while (wi + 1 < p.count && t >= p.toff[wi + 1]) ++wi;
    int local = t - p.toff[wi];
    const int S = p.splits[wi];
    k.wi = wi;
    k.s = local % S;
    local /= S;
    k.tw = local % p.nwin;
    k.rb = local / p.nwin;
    if (MODE == 1) {                      // splits cut the weight-scale groups
        const int G = p.Kt >> p.ksh;
        k.kt0 = (G * k.s / S) << p.ksh;
        k.cnt = ((G * (k.s + 1) / S) << p.ksh) - k.kt0;
    } else {
        k.kt0 = p.Kt * k.s / S;
        k.cnt = p.Kt * (k.s + 1) / S - k.kt0;
    }
    return k;
}

// Walks the k-tiles of this CTA's tasks in raw-stage units (tasks without k-tiles are skipped).
template <int MODE, int KPS>
struct StageIter {
    int t, off;
    bool valid;
    Task k;
    __device__ __forceinline__ void seek(const DtcParams &p) {
        while ((valid = t < p.ntasks)) {
            k = decode_task<MODE>(p, t);
            if (k.cnt > 0) break;
            t += gridDim.x;
        }
    }
    __device__ __forceinline__ void start(const DtcParams &p) {
        t = blockIdx.x;
        off = 0;
        seek(p);
    }
    __device__ __forceinline__ void next(const DtcParams &p) {
        off += KPS;
        if (off >= k.cnt) {
            off = 0;
            t += gridDim.x;
            seek(p);
        }
    }
};

template <int TN, int MODE>
__global__ void __launch_bounds__(Cfg<TN>::kThreads, 1) gemm_w4a8_dtc_kernel(const DtcParams p) {
    using C = Cfg<TN>;
    constexpr int TNP = C::TNP, EW = C::EW, CT = C::CT, NC = C::NC, RS = C::RS, KPS = C::KPS;
    constexpr int kSlots = C::kSlots, kRaw = C::kRaw;
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ uint64_t bars[3 * 8];           // full[kSlots], accfull[kSlots], empty[kSlots]
    __shared__ uint32_t tmem_base_s;
    __shared__ int dead_s;                     // a wait gave up somewhere in the CTA
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t smem_u = smem_u32(smem);
    const uint32_t full0 = smem_u32(&bars[0]), accfull0 = smem_u32(&bars[kSlots]),
                   empty0 = smem_u32(&bars[2 * kSlots]);
    unsigned char *rawbase = smem + kSlots * C::kSlotBytes;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kSlots; ++s) {
            mbar_init(full0 + s * 8, 4);         // one arrive per producer warp
            mbar_init(accfull0 + s * 8, 1);      // tcgen05.commit
            mbar_init(empty0 + s * 8, EW);       // one arrive per epilogue warp
        }
        dead_s = 0;
        mbar_init_fence();
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&tmem_base_s), C::kTmemCols);
        tmem_relinquish();
    }
    // the activation operand tiles start as zeros (an 8-token call leaves rows 8..15 of the
    // N = 16 tile untouched for the whole kernel)
    for (int i = threadIdx.x; i < kSlots * 2 * (C::kB / 16); i += C::kThreads) {
        const int s = i / (2 * (C::kB / 16)), r = i % (2 * (C::kB / 16));
        *reinterpret_cast<uint4 *>(smem + s * C::kSlotBytes + 2 * C::kA + r * 16) = make_uint4(0, 0, 0, 0);
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;

    if (warp < EW) {       // arm every accumulator column this thread will read
        const uint32_t lane_base = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
        const int col0 = (warp >> 2) * CT;
        for (int b = 0; b < kSlots * 2; ++b)
#pragma unroll
            for (int q = 0; q < CT / NC; ++q) {
                if constexpr (NC == 8) {
                    uint32_t c8[8];
                    make_const_regs(c8, (uint32_t)kMagicBits);
                    tmem_st8(lane_base + b * TNP + col0 + q * NC, c8);
                } else {
                    tmem_st16_const(lane_base + b * TNP + col0 + q * NC, (uint32_t)kMagicBits);
                }
            }
        tmem_wait_st();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    pdl_trigger();

    const int Kt = p.Kt, ksh = p.ksh, Ktg = Kt >> ksh, Ttot = p.T;
    int it = 0;            // steps done by this role: slot it % kSlots

    if (warp < EW) {
        // ================================ epilogue ======================================
        pdl_wait();
        const int q4 = warp & 3, col0 = (warp >> 2) * CT;
        const int rloc = q4 * 32 + lane;                     // row inside the block = TMEM lane
        const uint32_t lane_base = tmem_base + ((uint32_t)(q4 * 32) << 16);
        const f32x2 neg_magic2 = pack2(-kMagicF, -kMagicF);
        uint32_t cmagic[NC];
        make_const_regs(cmagic, (uint32_t)kMagicBits);
        bool dead = false;
        for (int t = blockIdx.x; t < p.ntasks && !dead; t += gridDim.x) {
            const Task k = decode_task<MODE>(p, t);
            f32x2 acc[CT / 2];
#pragma unroll
            for (int i = 0; i < CT / 2; ++i) acc[i] = 0ull;
            const int nsteps = (k.cnt + 1) >> 1;
            for (int st = 0; st < nsteps; ++st, ++it) {
                const int slot = it % kSlots;
                bool ok = !*(volatile int *)&dead_s &&
                          mbar_wait_bounded(accfull0 + slot * 8, (uint32_t)(it / kSlots) & 1u, p.status,
                                            kWaitEpi, p.wait_ns);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) {
                    dead_s = 1;
                    dead = true;
                    break;
                }
                tc_fence_after();
                DTC_STAMP(0, 0)
                const unsigned char *sb = smem + slot * C::kSlotBytes + 2 * C::kA + 2 * C::kB;
                const int nk = min(2, k.cnt - 2 * st);
                const bool one_group = (MODE == 1) && ksh;       // both k-tiles, one promote
                const int nu = one_group ? 1 : nk;               // accumulators to promote
                const bool two = one_group && nk == 2;
                const uint32_t tcol = lane_base + slot * 2 * TNP + col0;
                // one accumulator: the row's scale word, then its tokens in packed pairs
                auto promote = [&](const int u, const int qq, const uint32_t (&d)[NC]) {
                    const uint32_t w = *reinterpret_cast<const uint16_t *>(sb + 2 * C::kS + u * C::kW + rloc * 2);
                    const float ws = __half2float(__ushort_as_half((unsigned short)(w & 0xFFF0u)));
                    const float z8 = (float)(int)((w ^ 8u) & 15u);
                    const f32x2 ws2 = pack2(ws, ws), nz2 = pack2(-z8, -z8);
                    const ulonglong2 *sv = reinterpret_cast<const ulonglong2 *>(sb + u * C::kS) + (col0 >> 1);
                    const ulonglong2 *sv1 = reinterpret_cast<const ulonglong2 *>(sb + C::kS) + (col0 >> 1);
#pragma unroll
                    for (int j = 0; j < NC / 2; ++j) {
                        const ulonglong2 s4 = sv[qq * (NC / 2) + j];     // {as0, as1}, {asum0, asum1}
                        f32x2 smf = s4.y;
                        if (two) smf = add2(smf, sv1[qq * (NC / 2) + j].y);   // exact: small integers
                        const f32x2 f = fma2(nz2, smf, add2(pack2i((int)d[2 * j], (int)d[2 * j + 1]), neg_magic2));
                        if (MODE == 1) fma2_acc(acc[qq * (NC / 2) + j], f, ws2);
                        else fma2_acc(acc[qq * (NC / 2) + j], f, mul2(ws2, s4.x));
                    }
                };
                if (!DTC_DBG(1)) {
#pragma unroll 1
                    for (int u = 0; u < nu; ++u) {
#pragma unroll
                        for (int qq = 0; qq < CT / NC; ++qq) {
                            uint32_t d[NC];
                            if constexpr (NC == 8) {
                                tmem_ld8(tcol + u * TNP + qq * NC, d);
                                tmem_wait_ld8(d);
                                tmem_st8(tcol + u * TNP + qq * NC, cmagic);
                            } else {
                                tmem_ld16(tcol + u * TNP + qq * NC, d);
                                tmem_wait_ld16(d);
                                tmem_st16(tcol + u * TNP + qq * NC, cmagic);
                            }
                            promote(u, qq, d);
                        }
                    }
                }
                tmem_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + slot * 8);
                DTC_STAMP(0, 1)
            }
            if (dead) break;
            // ---- the task's tile: split reduction, then the store(s) ----
            float out[CT];
#pragma unroll
            for (int i = 0; i < CT / 2; ++i) unpack2(acc[i], out[2 * i], out[2 * i + 1]);
            const int S = p.splits[k.wi];
            if (S > 1) {
                const size_t tile = (size_t)(p.rboff[k.wi] + k.rb) * p.nwin + k.tw;
                float *pp = p.part + (tile * S + k.s) * (size_t)(128 * TN) + (size_t)col0 * 128 + rloc;
#pragma unroll
                for (int j = 0; j < CT; ++j) pp[j * 128] = out[j];
                __threadfence();
                __syncwarp();
                int old = 0;
                if (lane == 0) old = atomicAdd(p.cnt + tile * EW + warp, 1);
                old = __shfl_sync(0xffffffffu, old, 0);
                if (old != S - 1) continue;
                __threadfence();
                const float *base = p.part + tile * S * (size_t)(128 * TN) + (size_t)col0 * 128 + rloc;
#pragma unroll
                for (int j = 0; j < CT; ++j) {
                    float sum = 0.0f;
#pragma unroll 1
                    for (int s2 = 0; s2 < S; ++s2)
                        sum = __fadd_rn(sum, __ldcg(base + (size_t)s2 * (128 * TN) + j * 128));
                    out[j] = sum;
                }
                if (lane == 0) p.cnt[tile * EW + warp] = 0;      // ready for the next launch
            }
            const int row = k.rb * 128 + rloc;
            if (row < p.M[k.wi]) {
                const size_t ld = (size_t)p.ld[k.wi];
#pragma unroll
                for (int j = 0; j < CT; ++j) {
                    const int tok = k.tw * TN + col0 + j;
                    float v = out[j];
                    if (MODE == 1) v = __fmul_rn(v, __ldg(p.as_tok + tok));
#pragma unroll 1
                    for (int dd = 0; dd < p.ndst; ++dd) p.y[dd][k.wi][(size_t)tok * ld + row] = v;
                }
            }
        }
    } else if (warp < EW + 4) {
        // ================================ producers =====================================
        const int pr = threadIdx.x - EW * 32;                // row inside the block
        const uint32_t a_off = (uint32_t)((pr >> 3) * kSbo + (pr & 7) * 16);
        const uint64_t pol = l2_policy_evict_first();
        using Iter = StageIter<MODE, KPS>;
        auto raw_w = [&](int r) { return rawbase + r * C::kRawBytes; };
        auto raw_a = [&](int r) { return rawbase + r * C::kRawBytes + C::kRawW; };
        auto raw_s = [&](int r) { return rawbase + r * C::kRawBytes + C::kRawW + C::kRawA; };
        auto raw_l = [&](int r) { return rawbase + r * C::kRawBytes + C::kRawW + C::kRawA + C::kRawS; };
        // packed weights and scale lines of stage `f` (never written by any kernel)
        auto fill_w = [&](const Iter &f, int r) {
            if (!f.valid || DTC_DBG(16)) return;
            const int nkt = min(KPS, f.k.cnt - f.off);
            const int Mt = p.M[f.k.wi] >> 4;
            const int g = min(f.k.rb * 8 + (pr >> 4), Mt - 1);
            const int kt = f.k.kt0 + f.off;
            const uint8_t *src = p.codes[f.k.wi] + ((size_t)g * Kt + kt) * 256u + (pr & 15) * 16;
            const uint32_t dst = smem_u32(raw_w(r)) + pr * 16;
#pragma unroll
            for (int j = 0; j < KPS; ++j)
                if (j < nkt) cp_async16(dst + j * 2048, src + (size_t)j * 256, pol);
            if (pr < nkt * 16) {
                const int j = pr >> 4, c = pr & 15;
                const int gg = min(f.k.rb * 8 + (c >> 1), Mt - 1);
                const uint16_t *sl =
                    p.scales[f.k.wi] + ((size_t)gg * Ktg + ((kt + j) >> ksh)) * 16u + (c & 1) * 8;
                cp_async16_plain(smem_u32(raw_l(r)) + pr * 16, sl);
            }
        };
        // the tokens' codes, scales and code sums of stage `f` (written by the staging kernel)
        auto fill_a = [&](const Iter &f, int r) {
            if (!f.valid) return;
            const int nkt = min(KPS, f.k.cnt - f.off);
            const int kt = f.k.kt0 + f.off, tok0 = f.k.tw * TN;
            const uint32_t da = smem_u32(raw_a(r)), ds = smem_u32(raw_s(r));
            for (int i = pr; i < nkt * TN; i += 128) {
                const int j = i / TN, tok = i % TN;
                const int8_t *src = p.aq + ((size_t)(kt + j) * Ttot + tok0 + tok) * 32;
                cp_async16_plain(da + i * 32, src);
                cp_async16_plain(da + i * 32 + 16, src + 16);
            }
            for (int i = pr; i < nkt * (TN / 4); i += 128) {
                const int j = i / (TN / 4), c4 = i % (TN / 4);
                const size_t idx = (size_t)(kt + j) * Ttot + tok0 + 4 * c4;
                if (MODE == 0) cp_async16_plain(ds + i * 32, p.as + idx);
                cp_async16_plain(ds + i * 32 + 16, p.asum + idx);
            }
        };

        Iter f, c;
        f.start(p);
        c = f;
        {   // weights of the first stages go out before the wait on the previous kernel
            Iter f0 = f;
#pragma unroll 1
            for (int r = 0; r < kRaw - 1; ++r) {
                fill_w(f0, r);
                if (f0.valid) f0.next(p);
            }
        }
        pdl_wait();
#pragma unroll 1
        for (int r = 0; r < kRaw - 1; ++r) {
            fill_a(f, r);
            cp_async_commit();
            if (f.valid) f.next(p);
        }
        int rs = 0;                                   // raw stage that is consumed next
        bool dead = false;
        constexpr int AI = (KPS * TN + 127) / 128;    // token rows a thread converts per stage
        while (c.valid && !dead) {
            DTC_STAMP(1, 4)
            cp_async_wait<kRaw - 2>();
            DTC_STAMP(1, 5)
            {   // refill the stage that was consumed last
                const int rf = (rs + kRaw - 1) % kRaw;
                fill_w(f, rf);
                fill_a(f, rf);
                cp_async_commit();
                if (f.valid) f.next(p);
            }
            DTC_STAMP(1, 6)
            const int nkt = min(KPS, c.k.cnt - c.off);
            const int nst = (nkt + 1) >> 1;
            const unsigned char *rw = raw_w(rs), *ra = raw_a(rs), *rsm = raw_s(rs), *rl = raw_l(rs);
            // (1) everything this thread copied for the stage, loaded back in one batch
            uint4 wr[KPS];
#pragma unroll
            for (int j = 0; j < KPS; ++j)
                wr[j] = (j < nkt) ? *reinterpret_cast<const uint4 *>(rw + (j * 128 + pr) * 16)
                                  : make_uint4(0, 0, 0, 0);
            uint4 aa[AI], ab[AI];
#pragma unroll
            for (int m = 0; m < AI; ++m) {
                const int i = pr + 128 * m;
                aa[m] = ab[m] = make_uint4(0, 0, 0, 0);
                if (i < nkt * TN) {
                    aa[m] = *reinterpret_cast<const uint4 *>(ra + i * 32);
                    ab[m] = *reinterpret_cast<const uint4 *>(ra + i * 32 + 16);
                }
            }
            const bool has_s = pr < nkt * (TN / 4), has_l = pr < nkt * 16;
            float4 sc = make_float4(0.f, 0.f, 0.f, 0.f);
            int4 sm = make_int4(0, 0, 0, 0);
            uint4 ll = make_uint4(0, 0, 0, 0);
            if (has_s) {
                if (MODE == 0) sc = *reinterpret_cast<const float4 *>(rsm + pr * 32);
                sm = *reinterpret_cast<const int4 *>(rsm + pr * 32 + 16);
            }
            if (has_l) ll = *reinterpret_cast<const uint4 *>(rl + pr * 16);
            // (2) the stage's step slots must have been read out
            bool ok = !*(volatile int *)&dead_s;
#pragma unroll 1
            for (int st = 0; st < RS; ++st)
                if (st < nst && ok)
                    ok = mbar_wait_bounded(empty0 + ((it + st) % kSlots) * 8,
                                           ((uint32_t)((it + st) / kSlots) & 1u) ^ 1u, p.status, kWaitProd,
                                           p.wait_ns);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                dead_s = 1;
                dead = true;
                break;
            }
            DTC_STAMP(1, 0)
            // (3) expand the nibbles to bytes q+8 in the core-matrix layout, re-order the
            // token rows the same way, copy the scale pairs and the scale lines
#pragma unroll
            for (int j = 0; j < KPS; ++j)
                if (j < nkt && !DTC_DBG(2)) {
                    unsigned char *sb = smem + ((it + (j >> 1)) % kSlots) * C::kSlotBytes + (j & 1) * C::kA;
                    const uint4 c4 = wr[j];
                    const uint4 lo = make_uint4(nib_plus8(c4.x), nib_plus8(c4.y), nib_plus8(c4.z),
                                                nib_plus8(c4.w));
                    const uint4 hi = make_uint4(nib_plus8(c4.x >> 4), nib_plus8(c4.y >> 4),
                                                nib_plus8(c4.z >> 4), nib_plus8(c4.w >> 4));
                    *reinterpret_cast<uint4 *>(sb + a_off) = lo;            // even-k chunk
                    *reinterpret_cast<uint4 *>(sb + a_off + kLbo) = hi;     // odd-k chunk
                }
            DTC_STAMP(1, 2)
#pragma unroll
            for (int m = 0; m < AI; ++m) {
                const int i = pr + 128 * m;
                if (i < nkt * TN) {
                    const int j = i / TN, tok = i % TN;
                    const uint4 a = aa[m], b = ab[m];
                    const uint4 lo = make_uint4(__byte_perm(a.x, a.y, 0x6420), __byte_perm(a.z, a.w, 0x6420),
                                                __byte_perm(b.x, b.y, 0x6420), __byte_perm(b.z, b.w, 0x6420));
                    const uint4 hi = make_uint4(__byte_perm(a.x, a.y, 0x7531), __byte_perm(a.z, a.w, 0x7531),
                                                __byte_perm(b.x, b.y, 0x7531), __byte_perm(b.z, b.w, 0x7531));
                    unsigned char *dst = smem + ((it + (j >> 1)) % kSlots) * C::kSlotBytes + 2 * C::kA +
                                         (j & 1) * C::kB + (tok >> 3) * 256 + (tok & 7) * 16;
                    *reinterpret_cast<uint4 *>(dst) = lo;
                    *reinterpret_cast<uint4 *>(dst + 128) = hi;
                }
            }
            if (has_s) {   // four tokens' scales and code sums -> two {as0, as1, asum0, asum1} entries
                const int j = pr / (TN / 4), c4 = pr % (TN / 4);
                float4 *dst = reinterpret_cast<float4 *>(smem + ((it + (j >> 1)) % kSlots) * C::kSlotBytes +
                                                         2 * C::kA + 2 * C::kB + (j & 1) * C::kS) + 2 * c4;
                dst[0] = make_float4(sc.x, sc.y, (float)sm.x, (float)sm.y);
                dst[1] = make_float4(sc.z, sc.w, (float)sm.z, (float)sm.w);
            }
            if (has_l) {   // scale lines of the stage's k-tiles
                const int j = pr >> 4, cc = pr & 15;
                *reinterpret_cast<uint4 *>(smem + ((it + (j >> 1)) % kSlots) * C::kSlotBytes + 2 * C::kA +
                                           2 * C::kB + 2 * C::kS + (j & 1) * C::kW + cc * 16) = ll;
            }
            DTC_STAMP(1, 3)
            fence_proxy_async_smem();      // generic-proxy stores -> visible to the MMA
            __syncwarp();                  // ... of every lane, before the warp's one arrival
            if (lane == 0) {
#pragma unroll 1
                for (int st = 0; st < nst; ++st) mbar_arrive(full0 + ((it + st) % kSlots) * 8);
            }
            DTC_STAMP(1, 1)
            it += nst;
            c.next(p);
            rs = (rs + 1) % kRaw;
        }
        cp_async_wait<0>();
    } else {
        // ================================ MMA issuer ====================================
        constexpr uint32_t kIdesc = idesc_i8(128, TNP);
        bool dead = false;
        for (int t = blockIdx.x; t < p.ntasks && !dead; t += gridDim.x) {
            const Task k = decode_task<MODE>(p, t);
            const int nsteps = (k.cnt + 1) >> 1;
            for (int st = 0; st < nsteps; ++st, ++it) {
                // the issuing warps take the steps in turn: a step's wait, two MMAs and commit
                // cost one thread several hundred clocks, more than the tensor pipe needs
                if (it % C::MW != warp - (EW + 4)) continue;
                const int slot = it % kSlots;
                DTC_STAMP(2, 4)
                bool ok = !*(volatile int *)&dead_s &&
                          mbar_wait_bounded(full0 + slot * 8, (uint32_t)(it / kSlots) & 1u, p.status, kWaitMma,
                                            p.wait_ns);
                DTC_STAMP(2, 5)
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) {
                    dead_s = 1;
                    dead = true;
                    break;
                }
                tc_fence_after();
                DTC_STAMP(2, 0)
                if (lane == 0) {
                    const int nk = min(2, k.cnt - 2 * st);
                    const uint32_t sa = smem_u + slot * C::kSlotBytes;
                    for (int u = 0; u < nk; ++u) {
                        if (DTC_DBG(4)) break;
                        if (DTC_DBG(8) && u == 1) break;
                        const int buf = ((MODE == 1) && ksh) ? slot * 2 : slot * 2 + u;
                        tc_mma_i8(tmem_base + buf * TNP, smem_desc(sa + u * C::kA),
                                  smem_desc(sa + 2 * C::kA + u * C::kB), kIdesc, 1u);
                        if (u == 0) { DTC_STAMP(2, 6) }
                    }
                    DTC_STAMP(2, 7)
                    tc_commit(accfull0 + slot * 8);
                }
                DTC_STAMP(2, 1)
                __syncwarp();
            }
        }
    }

    // ---- teardown: every role comes here, also after a failed wait ------------------------
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) tmem_dealloc(tmem_base, C::kTmemCols);
}

struct DtcScratch {
    float *part = nullptr;
    size_t part_floats = 0;
    int *cnt = nullptr;
    int cnt_n = 0;
} g_dtc;

int g_dtc_sms = 0;
#ifdef TQ_DTC_TRACE
long long *g_dtc_trace = nullptr;
#endif

template <int TN, int MODE>
void launch_variant(const DtcParams &p, int grid) {
    using C = Cfg<TN>;
    static bool attr_set = false;
    if (!attr_set) {
        TQ_CHECK(cudaFuncSetAttribute(gemm_w4a8_dtc_kernel<TN, MODE>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem));
        attr_set = true;
    }
    launch_pdl(gemm_w4a8_dtc_kernel<TN, MODE>, dim3(grid), dim3(C::kThreads), (size_t)C::kSmem, p);
    TQ_LAUNCH_CHECK("gemm_w4a8_dtc_kernel");
}

template <int TN>
void launch_tn(const DtcParams &p, int grid, int mode) {
    if (mode) launch_variant<TN, 1>(p, grid);
    else launch_variant<TN, 0>(p, grid);
}

}  // namespace

bool gemm_dtc_covers(const GemmArgs &a) {
    if (a.dump || a.x) return false;
    if (a.count < 1 || a.count > 4 || a.T < 8 || a.T > 64 || (a.T % 8)) return false;
    if (a.npeer < 0 || a.npeer > 8) return false;
    if (a.K % 32) return false;
    if (a.ksh && ((a.K >> 5) & 1)) return false;
    if (a.mode == 1 ? !a.as_tok : !a.as) return false;
    if (!a.aq || !a.asum) return false;
    for (int i = 0; i < a.count; ++i) {
        if (a.seg[i].count != 1 || a.seg[i].split[0] < 1 || a.seg[i].split[0] > 16) return false;
        if (a.M[i] <= 0 || (a.M[i] % 16)) return false;
    }
    return true;
}

void launch_gemm_dtc(const GemmArgs &a) {
    if (!g_dtc_sms) {
        int dev = 0;
        TQ_CHECK(cudaGetDevice(&dev));
        TQ_CHECK(cudaDeviceGetAttribute(&g_dtc_sms, cudaDevAttrMultiProcessorCount, dev));
        if (g_dtc_sms <= 0) g_dtc_sms = 148;
    }
    DtcParams p{};
    p.count = a.count;
    int rbs = 0, maxS = 1;
    long units = 0;                           // (row block, split) pairs
    for (int i = 0; i < a.count; ++i) {
        p.codes[i] = a.codes[i];
        p.scales[i] = a.scales[i];
        p.M[i] = a.M[i];
        p.ld[i] = a.ld[i] ? a.ld[i] : a.M[i];
        p.splits[i] = a.seg[i].split[0];
        p.rboff[i] = rbs;
        rbs += (a.M[i] + 127) / 128;
        units += (long)((a.M[i] + 127) / 128) * p.splits[i];
        maxS = std::max(maxS, p.splits[i]);
    }
    p.rboff[a.count] = rbs;
    // Tokens per task: the widest window that still leaves every SM a task.
    int tn = 8;
    static const int forced = [] {
        const char *e = getenv("TQ_XPU_DTC_TOKENS");
        return e ? atoi(e) : 0;
    }();
    for (int cand : {64, 32, 16, 8}) {
        if (a.T % cand) continue;
        if (forced ? cand == forced : (units * (a.T / cand) >= g_dtc_sms || cand == 8)) {
            tn = cand;
            break;
        }
    }
    p.nwin = a.T / tn;
    int tasks = 0;
    for (int i = 0; i < a.count; ++i) {
        p.toff[i] = tasks;
        tasks += (p.rboff[i + 1] - p.rboff[i]) * p.nwin * p.splits[i];
    }
    p.toff[a.count] = tasks;
    p.ntasks = tasks;
    if (a.npeer > 0) {
        p.ndst = a.npeer;
        for (int d = 0; d < a.npeer; ++d)
            for (int i = 0; i < a.count; ++i) p.y[d][i] = a.ypeer[d][i];
    } else {
        p.ndst = 1;
        for (int i = 0; i < a.count; ++i) p.y[0][i] = a.y[i];
    }
    p.aq = a.aq;
    p.as = a.as;
    p.as_tok = a.as_tok;
    p.asum = a.asum;
    p.Kt = a.K >> 5;
    p.ksh = a.ksh;
    p.T = a.T;
    if (maxS > 1) {
        const size_t tiles = (size_t)rbs * p.nwin;
        const size_t need = tiles * maxS * 128 * tn;
        if (need > g_dtc.part_floats) {
            if (g_dtc.part) tq_dev_free(g_dtc.part);
            g_dtc.part = static_cast<float *>(tq_dev_alloc(need * sizeof(float), "gemm.dtc.partial"));
            g_dtc.part_floats = need;
        }
        const int cn = (int)tiles * 8;
        if (cn > g_dtc.cnt_n) {
            if (g_dtc.cnt) tq_dev_free(g_dtc.cnt);
            g_dtc.cnt = static_cast<int *>(tq_dev_alloc((size_t)cn * sizeof(int), "gemm.dtc.count"));
            TQ_CHECK(cudaMemsetAsync(g_dtc.cnt, 0, (size_t)cn * sizeof(int), stream()));
            g_dtc.cnt_n = cn;
        }
    }
    p.part = g_dtc.part;
    p.cnt = g_dtc.cnt;
    p.status = device_status_word();
    p.wait_ns = wait_limit_ns();
#ifdef TQ_DTC_TRACE
    {
        static long long *tr = nullptr;
        if (!tr) tr = static_cast<long long *>(tq_dev_alloc(3 * 256 * 8 * 8, "dtc.trace"));
        TQ_CHECK(cudaMemsetAsync(tr, 0, 3 * 256 * 8 * 8, stream()));
        p.trace = tr;
        g_dtc_trace = tr;
        const char *e = getenv("TQ_DTC_DBG");
        p.dbg = e ? atoi(e) : 0;
    }
#endif
    const int grid = std::min(g_dtc_sms, tasks);
    switch (tn) {
        case 64: launch_tn<64>(p, grid, a.mode); break;
        case 32: launch_tn<32>(p, grid, a.mode); break;
        case 16: launch_tn<16>(p, grid, a.mode); break;
        default: launch_tn<8>(p, grid, a.mode); break;
    }
}

}  // namespace tq

#ifdef TQ_DTC_TRACE
extern "C" int qwn_dbg_dtc_trace(long long *host_out) {
    if (!tq::g_dtc_trace) return -1;
    tq_d2h(host_out, tq::g_dtc_trace, 3 * 256 * 8 * 8);
    return 0;
}
#endif
