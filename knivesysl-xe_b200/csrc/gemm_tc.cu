// gemm_tc.cu — prefill W4A8 GEMM on the sm_100a tensor cores: tcgen05.mma kind::i8 with
// int32 accumulators in tensor memory (TMEM).
//
// Replaces gemm_rc16 / the unsplit path of x_gemm_w4a8 (xpu/src/kernels_dpas.cpp:1255-1332,
// 1371-1378): Y[tok][n] = sum over k-tiles, ascending, of (float)(d - z*asum) * (ws*as) with
// d the exact int32 dot of one 16-row x K32 tile, accumulated with fma into one fp32
// accumulator per output - the arithmetic and the order of the reference.
//
// Mapping. Weights are the M side of the MMA (128 output rows = 128 TMEM lanes), tokens the
// N side (128 per CTA tile), K = 32 per instruction = one k-tile, so one MMA produces exactly
// the per-k-tile int32 dots the reference promotes. A CTA (12 warps, one per SM, persistent
// over tiles) runs three roles connected by mbarriers (10 operand slots in shared memory, 4
// accumulator buffers in TMEM):
//  * producers (2 warps, thread = two weight rows): load a row's 16 packed bytes of a k-tile,
//    expand the nibbles to signed int8 bytes (three ops per word) and store them as the
//    two 16-byte K-chunks of the row in the canonical no-swizzle K-major core-matrix layout
//    (even-k codes first, then odd-k: any fixed permutation of k inside a tile is exact for
//    an integer dot, and the activation image uses the same one); one thread starts bulk
//    (TMA) copies of the activation image of the tile (4 KiB) and of its per-token
//    {as, as, asum, asum} pairs (1 KiB), prepared by a pre-pass in exactly that layout;
//  * two MMA threads (in two warps, promote groups in turn): tcgen05.mma (M=128, N=128, K=32) into accumulator slot b (the first MMA of a
//    promote group overwrites the slot, a second one accumulates); tcgen05.commit signals
//    the epilogue;
//  * epilogue (8 warps, thread = weight row x 64 tokens): two 32-column tcgen05.ld per
//    promote (every tcgen05 instruction costs its issuing thread on the order of a hundred
//    clocks, so the epilogue issues as few as it can and stores nothing back), then per
//    token pair: the int32 dot becomes fp32 exactly by adding the bit pattern of 12582912.0f
//    as an integer and subtracting 12582912.0f as a float; f = fma(-z, asum, d) (exact;
//    skipped while every zero point of the warp's rows is 0, i.e. for symmetric weights),
//    acc = fma(f, ws*as, acc); 64 fp32 accumulators stay in registers for the whole K loop
//    and are stored at the end (coalesced over rows).
// The epilogue is the wall, as on the reference's hardware: 2 issue slots per output per
// k-tile against 64 tensor-core clocks per 128x128x32 MMA.
//
// Every mbarrier wait is bounded; on expiry the kernel records a status word, stops
// issuing work, still frees its TMEM and returns.
#include "tc.cuh"

#include <cuda_bf16.h>

#include <algorithm>
#include <type_traits>

namespace tq {

namespace {

constexpr int kTM = 128;                 // weight rows per tile (TMEM lanes)
constexpr int kTN = 128;                 // tokens per tile (accumulator columns)
constexpr int kNB = 4;                   // accumulator buffers in TMEM (4 x 128 columns)
constexpr int kNS = 10;                  // operand slots in shared memory
constexpr int kPB = 4;                   // k-tiles a producer thread loads per batch (two rows each)
constexpr int kABytes = kTM * 32;        // expanded int8 weights of one k-tile
constexpr int kBBytes = kTN * 32;        // int8 activations of one k-tile
constexpr int kSBytes = kTN / 2 * 16;    // {as0, as1, asum0, asum1} per token pair
constexpr int kSlotBytes = kABytes + kBBytes + kSBytes;
// Twelve warps: three share a scheduler, so a thread may hold up to 168 registers
// (the epilogue's 64 accumulators and two 32-column TMEM loads do not fit the 128 that a
// fourth warp per scheduler would leave).
constexpr int kEpiWarps = 8, kProdWarps = 2;
// Two MMA-issuing warps take the promote groups in turn: the wait, tcgen05.mma and
// tcgen05.commit of one k-tile cost the issuing thread several hundred clocks (each tcgen05
// instruction about 150, whatever the MMA's N), more than the epilogue needs per k-tile in
// the per-token modes, so one issuing thread was the wall there.
constexpr int kMmaWarps = 2;
constexpr int kThreads = (kEpiWarps + kProdWarps + kMmaWarps) * 32;
constexpr int kRawStages = 4;             // raw ring of the producers: batches of kPB k-tiles
constexpr int kRawBytes = kPB * 2048;     // 128 rows x 16 packed bytes per k-tile
constexpr int kSmemBytes = kNS * kSlotBytes + kRawStages * kRawBytes;   // > half an SM's shared
                                         // memory: one CTA per SM, which the 512-column TMEM
                                         // allocation requires

// instruction descriptor: D = s32 (2), A and B signed 8 bit (1), both K-major, N >> 3 at bit 17, M >> 4 at bit 24
constexpr uint32_t kIdesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kTN >> 3) << 17) |
                            ((uint32_t)(kTM >> 4) << 24);

struct TcParams {
    const uint8_t *codes;
    const uint16_t *scales;
    const uint8_t *img;      // per (k-tile, 128-token block): kBBytes of codes as
                             // [16 token groups][2 K-chunks][8][16], then kSBytes of
                             // {as0, as1, (float)asum0, (float)asum1} per token pair
    void *y;
    const float *as_tok;     // per-token scales (PERTOK kernels)
    int *status;
    unsigned long long wait_ns;   // limit of every mbarrier wait
#ifdef TQ_TC_TRACE
    long long *trace;
#endif
    int M, Kt, ksh, T, Tpad, out_bf16;
};

// Pre-pass: the caller's staging (aq[kt][tok][32], as[kt][tok], asum[kt][tok]) -> the images
// the GEMM tiles copy with one bulk copy each. Tokens >= T are padded with zeros.
__global__ void __launch_bounds__(256)
gemm_tc_prepass_kernel(const int8_t *__restrict__ aq, const float *__restrict__ as,
                       const int32_t *__restrict__ asum, int T, int Tpad, int Kt,
                       uint8_t *__restrict__ img) {
    pdl_trigger();
    const size_t nrow = (size_t)Kt * Tpad;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < nrow; i += (size_t)gridDim.x * 256) {
        const int kt = (int)(i / Tpad), tok = (int)(i % Tpad);
        uint4 lo = make_uint4(0, 0, 0, 0), hi = make_uint4(0, 0, 0, 0);
        if (tok < T) {
            const uint4 *src = reinterpret_cast<const uint4 *>(aq + ((size_t)kt * T + tok) * 32);
            const uint4 a = __ldg(src), b = __ldg(src + 1);    // k = 0..15, 16..31
            // even-k bytes -> chunk 0, odd-k bytes -> chunk 1 (the weight expansion's order)
            lo = make_uint4(__byte_perm(a.x, a.y, 0x6420), __byte_perm(a.z, a.w, 0x6420),
                            __byte_perm(b.x, b.y, 0x6420), __byte_perm(b.z, b.w, 0x6420));
            hi = make_uint4(__byte_perm(a.x, a.y, 0x7531), __byte_perm(a.z, a.w, 0x7531),
                            __byte_perm(b.x, b.y, 0x7531), __byte_perm(b.z, b.w, 0x7531));
        }
        uint8_t *blk = img + ((size_t)kt * (Tpad / kTN) + tok / kTN) * (kBBytes + kSBytes);
        const int tl = tok % kTN;
        uint8_t *dst = blk + (tl >> 3) * 256 + (tl & 7) * 16;
        *reinterpret_cast<uint4 *>(dst) = lo;
        *reinterpret_cast<uint4 *>(dst + 128) = hi;
        if ((tok & 1) == 0) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (tok < T) {
                v.x = as ? as[(size_t)kt * T + tok] : 0.0f;
                v.z = (float)asum[(size_t)kt * T + tok];
            }
            if (tok + 1 < T) {
                v.y = as ? as[(size_t)kt * T + tok + 1] : 0.0f;
                v.w = (float)asum[(size_t)kt * T + tok + 1];
            }
            reinterpret_cast<float4 *>(blk + kBBytes)[tl >> 1] = v;
        }
    }
}

// Four 4-bit two's-complement codes (the low nibble of each byte) -> four int8 bytes.
__device__ __forceinline__ uint32_t sext_nibbles(uint32_t l) {
    l &= 0x0F0F0F0Fu;
    return l | ((l & 0x08080808u) * 0x1Eu);      // a set sign bit fills bits 4..7 of its byte
}

// W4A4 pre-pass: packed int4 activations aq4[kt64][tok][32] (byte b = k 2b, 2b+1 of the 64),
// as4 / asum4 per (kt64, tok) -> the same images as above, two K32 images per K64 block. The
// block's scale and code sum go with its first K32 image; the second one carries zeros, so
// the GEMM that adds the two sums of a promote group gets the block's sum.
__global__ void __launch_bounds__(256)
gemm_tc_prepass_s4_kernel(const uint8_t *__restrict__ aq4, const float *__restrict__ as4,
                          const int32_t *__restrict__ asum4, int T, int Tpad, int Kt,
                          uint8_t *__restrict__ img) {
    pdl_trigger();
    const size_t nrow = (size_t)Kt * Tpad;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < nrow; i += (size_t)gridDim.x * 256) {
        const int kt = (int)(i / Tpad), tok = (int)(i % Tpad);
        const int kg = kt >> 1, half = kt & 1;
        uint4 lo = make_uint4(0, 0, 0, 0), hi = make_uint4(0, 0, 0, 0);
        if (tok < T) {
            const uint4 a = __ldg(reinterpret_cast<const uint4 *>(aq4 + ((size_t)kg * T + tok) * 32) + half);
            // low nibbles = even k -> chunk 0, high nibbles = odd k -> chunk 1
            lo = make_uint4(sext_nibbles(a.x), sext_nibbles(a.y), sext_nibbles(a.z), sext_nibbles(a.w));
            hi = make_uint4(sext_nibbles(a.x >> 4), sext_nibbles(a.y >> 4), sext_nibbles(a.z >> 4),
                            sext_nibbles(a.w >> 4));
        }
        uint8_t *blk = img + ((size_t)kt * (Tpad / kTN) + tok / kTN) * (kBBytes + kSBytes);
        const int tl = tok % kTN;
        uint8_t *dst = blk + (tl >> 3) * 256 + (tl & 7) * 16;
        *reinterpret_cast<uint4 *>(dst) = lo;
        *reinterpret_cast<uint4 *>(dst + 128) = hi;
        if ((tok & 1) == 0) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (half == 0) {
                if (tok < T) {
                    v.x = as4[(size_t)kg * T + tok];
                    v.z = (float)asum4[(size_t)kg * T + tok];
                }
                if (tok + 1 < T) {
                    v.y = as4[(size_t)kg * T + tok + 1];
                    v.w = (float)asum4[(size_t)kg * T + tok + 1];
                }
            }
            reinterpret_cast<float4 *>(blk + kBBytes)[tl >> 1] = v;
        }
    }
}

constexpr int kWaitMma = 21, kWaitEpi = 22, kWaitProd = 23;   // status codes of failed waits
#ifdef TQ_TC_TRACE
#define TC_STAMP(idx, which)                                                                  \
    if (blockIdx.x == 0 && p.trace && (idx) < 256 && threadIdx.x == 0) p.trace[(idx) * 8 + (which)] = clock64();
#else
#define TC_STAMP(idx, which)
#endif

// Four two's-complement nibbles (the low nibble of each byte of w) -> four signed bytes.
__device__ __forceinline__ uint32_t nib_s8(uint32_t w) { return __vsub4(nib_plus8(w), 0x08080808u); }

// GW = k-tiles accumulated in TMEM before one fp32 promote (1: the reference's arithmetic with
// a scale per (token, K32); 2: K64 weight groups with per-token activation scales, or - not
// PERTOK - with one activation scale per (token, K64): the W4A4 arithmetic). PERTOK:
// the activation scale is applied once at the end (y = acc * as_tok).
template <int GW, bool PERTOK>
__global__ void __maxnreg__(168) gemm_w4a8_tc_kernel(const TcParams p) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ uint64_t bars[2 * kNS + 2 * kNB];   // full[kNS], empty[kNS], accfull[kNB], accempty[kNB]
    __shared__ uint32_t tmem_base_s;
    __shared__ int dead_s;                      // a wait gave up somewhere in the CTA
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t smem_u = smem_u32(smem);
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kNS]),
                   acc0 = smem_u32(&bars[2 * kNS]), accempty0 = smem_u32(&bars[2 * kNS + kNB]);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kNS; ++s) {
            mbar_init(full0 + s * 8, kProdWarps * 32);   // every producer thread arrives once
            mbar_init(empty0 + s * 8, kEpiWarps);        // one arrive per epilogue warp
        }
        for (int b = 0; b < kNB; ++b) {
            mbar_init(acc0 + b * 8, 1);                  // tcgen05.commit
            mbar_init(accempty0 + b * 8, kEpiWarps);     // one arrive per epilogue warp
        }
        dead_s = 0;
        mbar_init_fence();
    }
    if (warp == 0) {                                     // one warp allocates all 512 columns
        tmem_alloc(smem_u32(&tmem_base_s), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;

    pdl_trigger();
    pdl_wait();      // everything below reads the images an earlier kernel wrote

    const int Kt = p.Kt, Ktg = Kt >> p.ksh;
    const int row_blocks = p.M / kTM, tok_blocks = p.Tpad / kTN;
    const int ntiles = row_blocks * tok_blocks;
    int it = 0;      // k-tile counter across the tiles of this CTA: operand slot it % kNS,
                     // accumulator buffer it % kNB

    if (warp < kEpiWarps) {
        // ================================ epilogue ======================================
        const int q4 = warp & 3, chalf = (warp >> 2) * 64;
        const int rloc = q4 * 32 + lane;                  // row inside the tile = TMEM lane
        const uint32_t lane_base = tmem_base + ((uint32_t)(q4 * 32) << 16);
        const f32x2 neg_magic2 = pack2(-kMagicF, -kMagicF);
        for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
            const int rb = tile % row_blocks, tb = tile / row_blocks;
            const int row = rb * kTM + rloc;
            const uint16_t *sc = p.scales + ((size_t)(row >> 4) * Ktg) * 16 + (row & 15);
            f32x2 acc[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = 0ull;
            uint32_t scw = __ldg(sc);
            for (int kt = 0; kt < Kt; kt += GW, it += GW) {
                const int ig = it / GW;                       // promote groups done by this CTA
                const int b = ig % kNB, sl = it % kNS;
                const uint32_t ph = (uint32_t)(ig / kNB) & 1u;
                int zp;
                float ws;
                unpack_scale(scw, zp, ws);
                if (kt + GW < Kt) scw = __ldg(sc + (size_t)((kt + GW) >> p.ksh) * 16);
                const f32x2 ws2 = pack2(ws, ws);
                const float nzf = (float)(-zp);
                const f32x2 nz2 = pack2(nzf, nzf);
                // symmetric weights (every zero point of the warp's rows is 0) need no
                // zero-point term at all: the weights enter the MMA as true signed bytes
                const bool anyz = __any_sync(0xffffffffu, zp != 0);
                TC_STAMP(ig, 0)
                bool ok = !*(volatile int *)&dead_s && mbar_wait_bounded(acc0 + b * 8, ph, p.status, kWaitEpi, p.wait_ns);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) {
                    dead_s = 1;
                    break;
                }
                tc_fence_after();
                TC_STAMP(ig, 1)
                const ulonglong2 *sv = reinterpret_cast<const ulonglong2 *>(
                                           smem + (size_t)sl * kSlotBytes + kABytes + kBBytes) +
                                       (chalf >> 1);
                // second k-tile of the group (GW == 2): only its code sums are needed
                const int sl1 = (it + GW - 1) % kNS;
                const ulonglong2 *sv1 = reinterpret_cast<const ulonglong2 *>(
                                            smem + (size_t)sl1 * kSlotBytes + kABytes + kBBytes) +
                                        (chalf >> 1);
                // Two 32-column loads, the second in flight while the first is promoted. The
                // accumulator holds the plain int32 dot (the group's first MMA overwrites it), so
                // nothing has to be stored back; adding the bit pattern of 12582912.0f to the
                // integer and subtracting 12582912.0f from the result as a float converts it
                // exactly (|d| < 2^22) on the integer and packed-fp32 pipes.
                uint32_t da[32], db[32];
                const uint32_t tcol = lane_base + b * kTN + chalf;
                // Straight-line code per variant (ANYZ is a compile-time tag): a test of `anyz`
                // inside the unrolled pair loop splits it into one basic block per pair, and the
                // pairs' short dependency chains then run one after the other.
                auto promote = [&](auto anyz_tag, const int q, uint32_t (&d)[32]) {
                    constexpr bool ANYZ = decltype(anyz_tag)::value;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        f32x2 f = add2(pack2i((int)d[2 * j] + kMagicBits, (int)d[2 * j + 1] + kMagicBits),
                                       neg_magic2);
                        if (PERTOK) {
                            if (ANYZ) {
                                f32x2 smf = sv[q * 16 + j].y;                  // {asum0, asum1}
                                if (GW == 2) smf = add2(smf, sv1[q * 16 + j].y);   // exact: small integers
                                f = fma2(nz2, smf, f);
                            }
                            fma2_acc(acc[q * 16 + j], f, ws2);
                        } else {
                            const ulonglong2 s4 = sv[q * 16 + j];      // {as0, as1}, {asum0, asum1}
                            if (ANYZ) {
                                f32x2 smf = s4.y;
                                if (GW == 2) smf = add2(smf, sv1[q * 16 + j].y);
                                f = fma2(nz2, smf, f);
                            }
                            fma2_acc(acc[q * 16 + j], f, mul2(ws2, s4.x));
                        }
                    }
                };
                auto promote_any = [&](const int q, uint32_t (&d)[32]) {
                    if (anyz) promote(std::true_type{}, q, d);
                    else promote(std::false_type{}, q, d);
                };
                tmem_ld32(tcol, da);
                tmem_wait_ld32(da);
                TC_STAMP(ig, 2)
                tmem_ld32(tcol + 32, db);
                promote_any(0, da);
                TC_STAMP(ig, 3)
                tmem_wait_ld32(db);
                promote_any(1, db);
                TC_STAMP(ig, 4)
                TC_STAMP(ig, 5)
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(accempty0 + b * 8);      // the MMA may overwrite the buffer
                    mbar_arrive(empty0 + sl * 8);        // the producers may refill the slot(s)
                    if (GW == 2) mbar_arrive(empty0 + sl1 * 8);
                }
                TC_STAMP(ig, 6)
            }
            if (*(volatile int *)&dead_s) break;
            // store: thread = row, 64 tokens; rows are contiguous in y, so a warp writes 128 B
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                float v0, v1;
                unpack2(acc[i], v0, v1);
                const int tok = tb * kTN + chalf + 2 * i;
                if (PERTOK) {
                    if (tok < p.T) v0 = __fmul_rn(v0, __ldg(p.as_tok + tok));
                    if (tok + 1 < p.T) v1 = __fmul_rn(v1, __ldg(p.as_tok + tok + 1));
                }
                if (p.out_bf16) {
                    __nv_bfloat16 *y = static_cast<__nv_bfloat16 *>(p.y);
                    if (tok < p.T) y[(size_t)tok * p.M + row] = __float2bfloat16_rn(v0);
                    if (tok + 1 < p.T) y[(size_t)(tok + 1) * p.M + row] = __float2bfloat16_rn(v1);
                } else {
                    float *y = static_cast<float *>(p.y);
                    if (tok < p.T) y[(size_t)tok * p.M + row] = v0;
                    if (tok + 1 < p.T) y[(size_t)(tok + 1) * p.M + row] = v1;
                }
            }
        }
    } else if (warp < kEpiWarps + kProdWarps) {
        // ================================ producers =====================================
        const int pr = threadIdx.x - kEpiWarps * 32;       // rows pr and pr + 64 of the tile
        // destination of a row's two K-chunks in the core-matrix layout (row pr + 64: 8 row
        // groups further)
        const uint32_t a_off = (uint32_t)((pr >> 3) * kSbo + (pr & 7) * 16);
        // Packed weights travel through a private raw ring in shared memory (cp.async, kRawStages
        // batches of kPB k-tiles, all but one in flight): a thread reads back only what it
        // copied itself, so the ring needs no barrier, and the loop below is the producers'
        // whole steady-state code (register double-buffering needed two copies of it, and the
        // kernel's roles were evicting one another from the instruction cache).
        unsigned char *raw = smem + kNS * kSlotBytes;
        const uint32_t raw_u = smem_u + kNS * kSlotBytes;
        const uint64_t pol = l2_policy_evict_first();
        const int nbatch = (Kt + kPB - 1) / kPB;
        const int my_tiles = (ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
        const int total = my_tiles * nbatch;               // batches this CTA produces
        const size_t half_rows = (size_t)4 * Kt * 256;     // 64 rows = 4 row-groups further
        auto fill = [&](int g) {
            if (g < total) {
                const int tile = blockIdx.x + (g / nbatch) * gridDim.x, kt0 = (g % nbatch) * kPB;
                const int row = (tile % row_blocks) * kTM + pr;
                const uint8_t *src = p.codes + ((size_t)(row >> 4) * Kt + kt0) * 256 + (row & 15) * 16;
                const uint32_t dst = raw_u + (uint32_t)(g % kRawStages) * kRawBytes + pr * 16;
#pragma unroll
                for (int j = 0; j < kPB; ++j)
                    if (kt0 + j < Kt) {
                        cp_async16(dst + j * 2048, src + (size_t)j * 256, pol);
                        cp_async16(dst + j * 2048 + 1024, src + half_rows + (size_t)j * 256, pol);
                    }
            }
            cp_async_commit();
        };
#pragma unroll 1
        for (int g = 0; g < kRawStages - 1; ++g) fill(g);
#pragma unroll 1
        for (int g = 0; g < total; ++g) {
            cp_async_wait<kRawStages - 2>();
            fill(g + kRawStages - 1);                      // into the stage consumed last
            const int tb = (blockIdx.x + (g / nbatch) * gridDim.x) / row_blocks, kb = g % nbatch;
            // The whole batch behind ONE round of waits, one proxy fence and one round of
            // arrivals.
            const int nk = min(kPB, Kt - kb * kPB);
            bool ok = !*(volatile int *)&dead_s;
#pragma unroll 1
            for (int j = 0; j < nk && ok; ++j)
                ok = mbar_wait_bounded(empty0 + ((it + j) % kNS) * 8, ((uint32_t)((it + j) / kNS) & 1u) ^ 1u,
                                       p.status, kWaitProd, p.wait_ns);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                dead_s = 1;
                break;
            }
            const unsigned char *rs = raw + (size_t)(g % kRawStages) * kRawBytes + pr * 16;
#pragma unroll
            for (int j = 0; j < kPB; ++j) {
                if (j >= nk) break;
                unsigned char *slot = smem + (size_t)((it + j) % kNS) * kSlotBytes;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint4 c4 = *reinterpret_cast<const uint4 *>(rs + j * 2048 + h * 1024);
                    // nibble -> q + 8 (one logic op per four codes) -> q (one SIMD byte subtract)
                    const uint4 lo = make_uint4(nib_s8(c4.x), nib_s8(c4.y), nib_s8(c4.z), nib_s8(c4.w));
                    const uint4 hi = make_uint4(nib_s8(c4.x >> 4), nib_s8(c4.y >> 4), nib_s8(c4.z >> 4),
                                                nib_s8(c4.w >> 4));
                    *reinterpret_cast<uint4 *>(slot + a_off + h * 8 * kSbo) = lo;          // even-k chunk
                    *reinterpret_cast<uint4 *>(slot + a_off + h * 8 * kSbo + kLbo) = hi;   // odd-k chunk
                }
            }
            fence_proxy_async_smem();   // generic-proxy stores -> visible to the MMA
#pragma unroll 1
            for (int j = 0; j < nk; ++j) {
                const int sl = (it + j) % kNS;
                const uint32_t fb = full0 + sl * 8;
                if (pr == j * 16) {
                    // One bulk copy brings the activation image of this (k-tile, token block);
                    // this thread's arrival also announces its bytes. Each k-tile of the batch
                    // has its own issuing thread: one thread sustains only about two bulk
                    // copies in flight.
                    mbar_expect_tx(fb, kBBytes + kSBytes);
                    bulk_g2s_plain(smem_u + sl * kSlotBytes + kABytes,
                                   p.img + ((size_t)(kb * kPB + j) * (p.Tpad / kTN) + tb) * (kBBytes + kSBytes),
                                   kBBytes + kSBytes, fb);
                } else {
                    mbar_arrive(fb);
                }
            }
            it += nk;
        }
        cp_async_wait<0>();
    } else {
        // ================================ MMA issuer ====================================
        for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
            for (int kt = 0; kt < Kt; ++kt, ++it) {
                const int ig = it / GW;
                if (ig % kMmaWarps != warp - (kEpiWarps + kProdWarps)) continue;   // the other warp's group
                const int b = ig % kNB, sl = it % kNS;
                bool ok = !*(volatile int *)&dead_s &&
                          mbar_wait_bounded(full0 + sl * 8, (uint32_t)(it / kNS) & 1u, p.status, kWaitMma, p.wait_ns);
                // ... and, for the first k-tile of a group, the accumulator buffer has been
                // read out
                if (it % GW == 0)
                    ok = ok && mbar_wait_bounded(accempty0 + b * 8, ((uint32_t)(ig / kNB) & 1u) ^ 1u,
                                                 p.status, kWaitMma, p.wait_ns);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) {
                    dead_s = 1;
                    break;
                }
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t a_addr = smem_u + sl * kSlotBytes;
                    // the first MMA of a promote group overwrites the accumulator
                    tc_mma_i8(tmem_base + b * kTN, smem_desc(a_addr), smem_desc(a_addr + kABytes),
                              kIdesc, (it % GW) ? 1u : 0u);
                    if (it % GW == GW - 1) tc_commit(acc0 + b * 8);
                }
                __syncwarp();
            }
            if (*(volatile int *)&dead_s) break;
        }
    }

    // ---- teardown: every role comes here, also after a failed wait ------------------------
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) tmem_dealloc(tmem_base, 512);
}

struct TcScratch {
    uint8_t *img = nullptr;
    size_t img_bytes = 0;
} g_tc;

int g_tc_sms = 0;
#ifdef TQ_TC_TRACE
long long *g_tc_trace = nullptr;
#endif

}  // namespace

int launch_gemm_tc(const GemmTcArgs &a) {
    // covered: per-block activation scales (the reference's x_gemm_w4a8 arithmetic) or
    // per-token scales, rows a multiple of 128, K64 tier only with an even number of k-tiles
    if (!a.as == !a.as_tok) return -1;          // exactly one kind of activation scale
    if (a.aq4 && (!a.as || !a.ksh)) return -1;  // W4A4: K64 weights, scale per (token, K64)
    if (a.M % kTM || a.K % 32 || a.T < 128) return -1;
    const int Kt = a.K / 32;
    if (a.ksh && (Kt & 1)) return -1;
    if (!g_tc_sms) {
        int dev = 0;
        TQ_CHECK(cudaGetDevice(&dev));
        TQ_CHECK(cudaDeviceGetAttribute(&g_tc_sms, cudaDevAttrMultiProcessorCount, dev));
        if (g_tc_sms <= 0) g_tc_sms = 148;
        TQ_CHECK(cudaFuncSetAttribute(gemm_w4a8_tc_kernel<1, false>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        TQ_CHECK(cudaFuncSetAttribute(gemm_w4a8_tc_kernel<1, true>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        TQ_CHECK(cudaFuncSetAttribute(gemm_w4a8_tc_kernel<2, true>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        TQ_CHECK(cudaFuncSetAttribute(gemm_w4a8_tc_kernel<2, false>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
    }
    const int Tpad = (a.T + kTN - 1) / kTN * kTN;
    const size_t ibytes = (size_t)Kt * (Tpad / kTN) * (kBBytes + kSBytes);
    if (ibytes > g_tc.img_bytes) {
        if (g_tc.img) tq_dev_free(g_tc.img);
        g_tc.img = static_cast<uint8_t *>(tq_dev_alloc(ibytes, "gemm.tc.activation.image"));
        g_tc.img_bytes = ibytes;
    }
    const size_t nrow = (size_t)Kt * Tpad;
    const int pgrid = (int)std::min<size_t>((nrow + 255) / 256, (size_t)g_tc_sms * 8);
    if (a.aq4)
        gemm_tc_prepass_s4_kernel<<<pgrid, 256, 0, stream()>>>(a.aq4, a.as, a.asum, a.T, Tpad, Kt,
                                                              g_tc.img);
    else
        gemm_tc_prepass_kernel<<<pgrid, 256, 0, stream()>>>(a.aq, a.as, a.asum, a.T, Tpad, Kt, g_tc.img);
    TQ_LAUNCH_CHECK("gemm_tc_prepass_kernel");
    TcParams p{};
    p.codes = a.codes; p.scales = a.scales; p.img = g_tc.img; p.y = a.y;
    p.status = device_status_word();
    p.wait_ns = wait_limit_ns();
#ifdef TQ_TC_TRACE
    {
        static long long *tr = nullptr;
        if (!tr) tr = static_cast<long long *>(tq_dev_alloc(256 * 8 * 8, "tc.trace"));
        TQ_CHECK(cudaMemsetAsync(tr, 0, 256 * 8 * 8, stream()));
        p.trace = tr;
        g_tc_trace = tr;
    }
#endif
    p.M = a.M; p.Kt = Kt; p.ksh = a.ksh; p.T = a.T; p.Tpad = Tpad; p.out_bf16 = a.out_bf16;
    const int ntiles = (a.M / kTM) * (Tpad / kTN);
    const int grid = std::min(g_tc_sms, ntiles);
    p.as_tok = a.as_tok;
    if (a.aq4)
        launch_pdl(gemm_w4a8_tc_kernel<2, false>, dim3(grid), dim3(kThreads), (size_t)kSmemBytes, p);
    else if (!a.as_tok)
        launch_pdl(gemm_w4a8_tc_kernel<1, false>, dim3(grid), dim3(kThreads), (size_t)kSmemBytes, p);
    else if (a.ksh)
        launch_pdl(gemm_w4a8_tc_kernel<2, true>, dim3(grid), dim3(kThreads), (size_t)kSmemBytes, p);
    else
        launch_pdl(gemm_w4a8_tc_kernel<1, true>, dim3(grid), dim3(kThreads), (size_t)kSmemBytes, p);
    TQ_LAUNCH_CHECK("gemm_w4a8_tc_kernel");
    return 0;
}

}  // namespace tq

#ifdef TQ_TC_TRACE
extern "C" int qwn_dbg_tc_trace(long long *host_out) {
    if (!tq::g_tc_trace) return -1;
    tq_d2h(host_out, tq::g_tc_trace, 256 * 8 * 8);
    return 0;
}
#endif
