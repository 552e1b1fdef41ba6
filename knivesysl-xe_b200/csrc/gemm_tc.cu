// gemm_tc.cu — prefill W4A8 GEMM on the sm_100a tensor cores: tcgen05.mma kind::f16 on
// integer-valued fp16 operands, fp32 accumulators in tensor memory (TMEM).
//
// Replaces gemm_rc16 / the unsplit path of x_gemm_w4a8 (xpu/src/kernels_dpas.cpp:1255-1332,
// 1371-1378): Y[tok][n] = sum over k-tiles, ascending, of (float)(d - z*asum) * (ws*as) with
// d the exact int32 dot of one 16-row x K32 tile, accumulated with fma into one fp32
// accumulator per output - the arithmetic and the order of the reference.
//
// Why the f16 pipe for an integer dot. The 4-bit codes (-8..7) and the int8 activations are
// exact in fp16, their products (< 2^11) and a k-tile's sum of them (< 2^16; a K64 group:
// < 2^17) are exact in the tensor core's fp32 accumulation, so the accumulator IS (float)d,
// bit for bit, and the epilogue promotes it with one fma per output. With kind::i8 the
// accumulator is int32 and every output costs an integer add and a float add more per k-tile
// on the CUDA cores (the exact conversion), which is what bounded that version of the
// kernel: the tensor pipe, at half the int8 rate, is still far from being the wall.
//
// Mapping. Weights are the M side of the MMA (128 output rows = 128 TMEM lanes), tokens the
// N side (128 per CTA tile), a k-tile (K = 32) is two K = 16 instructions, so one accumulator
// read-out yields exactly the per-k-tile dots the reference promotes. The K loop advances in
// steps of two k-tiles. Both operands come from images that pre-passes write in the operand
// layout (canonical no-swizzle K-major core matrices): the activation image (fp16 codes plus
// as and (float)asum per token) and the weight image - every 4-bit code expanded to fp16 once
// per call (shift, one logic op that isolates two nibbles and sets the exponent of 1024 with
// the sign bit flipped, one packed subtract of 1032; inside a 16-byte K-chunk the codes sit in
// the order 0,4,1,5,2,6,3,7: any fixed permutation of k inside an instruction is exact for a
// dot, and the activation image uses the same one). The weight image costs 4 bytes per code of
// scratch, written and read once per call (3 % of the call); with it the GEMM's CUDA cores
// only promote. Tiles are walked token block fastest, so the CTAs that run together share
// a few row blocks of the weight image while the whole activation image stays in L2.
//
// A CTA (19 warps, one per SM, persistent over tiles) runs three roles connected by
// mbarriers (6 step slots in shared memory, 4 accumulator buffers in TMEM):
//  * one thread starts the bulk (TMA) copies of a step: 16 KiB of weights and 18 KiB of
//    activations, each contiguous in its image;
//  * two MMA threads (in two warps, steps in turn): two tcgen05.mma (M=128, N=128, K=16) per
//    k-tile into accumulator buffer b (the first MMA of a promote group overwrites it);
//    tcgen05.commit signals the workers once per step: a step is one K64 group in one of four
//    128-column buffers, or two K32 groups in the halves of one of two 256-column pairs. The single-thread roles wait with a suspend-time
//    hint: back-to-back polling took a fifth of the schedulers' issue slots;
//  * workers (16 warps): thread = weight row x 32 tokens. Per promote group: wait for the
//    group's accumulator, one 32-column tcgen05.ld, then per token
//    f = fma(-z, asum, d) (exact; only in the kernel variant for weights with zero points),
//    acc = fma(f, ws*as, acc); 32 fp32 accumulators stay in registers for the whole K loop
//    and are stored at the end (coalesced over rows). With five warps per scheduler the loop
//    is bound by issue slots: it is kept to the plain sequence (issuing the next group's
//    load early, behind this group's fma, cost more instructions than the latency it hid).
// What bounds it: issue slots of the worker warps (119 instructions per group, 32 of them fma)
// and the hand-offs between the roles - a trace shows every role busy about half of the time
// and waiting for another one the other half; neither halving the copied bytes, nor a third
// MMA thread, nor spinning instead of suspended waits changes the time by more than 2 %.
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
constexpr int kSS = 6;                   // step slots in shared memory (two k-tile slots each)
constexpr int kABytes = kTM * 64;        // expanded fp16 weights of one k-tile
constexpr int kBBytes = kTN * 64;        // fp16 activations of one k-tile
constexpr int kSBytes = kTN * 8;         // as[128] then (float)asum[128] of the tile's tokens
constexpr int kImgBytes = kBBytes + kSBytes;   // activation image of one (k-tile, token block)
// a step slot: the fp16 weights of its two k-tiles, then their two activation images - the
// order both lie in memory, so a step is two bulk copies
constexpr int kStepBytes = 2 * kABytes + 2 * kImgBytes;
// Nineteen warps: five share a scheduler, whose register file then leaves a thread 96
// registers (32 accumulators and the 32 loaded columns fit). Eight workers of 64 tokens at 168
// registers measured the same in per-token mode and 9 % slower in the reference's arithmetic.
constexpr int kWorkWarps = 16;
constexpr int kWT = kTN / (kWorkWarps / 4);      // tokens of a tile that one worker thread promotes
constexpr int kMaxRegs = 96;
// Two MMA-issuing threads take the promote groups in turn: waits, four tcgen05.mma and the
// tcgen05.commit of a K64 group cost the issuing thread about 700 clocks (every tcgen05
// instruction 80 to 110, whatever the MMA's width), more than a group may take.
constexpr int kMmaWarps = 2;
constexpr int kThreads = (kWorkWarps + 1 + kMmaWarps) * 32;    // + the warp that starts the image copies
constexpr uint32_t kNapNs = 2000;         // suspend-time hint of the single-thread roles' waits
static_assert((kNB & (kNB - 1)) == 0, "accumulator buffers are a mask of the group counter");
constexpr int kSmemBytes = kSS * kStepBytes;   // > half an SM's shared
                                         // memory: one CTA per SM, which the 512-column TMEM
                                         // allocation requires

// fp16 operands: four 16-byte K-chunks per row of a k-tile, 128 bytes apart; row groups of 8
// are 512 bytes apart; the second K = 16 instruction of a k-tile starts two chunks further
constexpr uint32_t kLboH = 128, kSboH = 512;
constexpr uint32_t kIdesc = idesc_f16(kTM, kTN);

struct TcParams {
    const uint8_t *wimg;     // per (128-row block, k-tile): kABytes of fp16 weights in operand layout
    const uint16_t *scales;
    const uint8_t *img;      // per (128-token block, k-tile): kBBytes of fp16 codes as
                             // [16 token groups][4 K-chunks][8 tokens][16 B], then kSBytes:
                             // as[128], (float)asum[128]
    void *y;
    const float *as_tok;     // per-token scales (PERTOK kernels)
    const int *zp_flag;      // written by the pre-pass: some zero point of the weight is not 0
    int *status;
    unsigned long long wait_ns;   // limit of every mbarrier wait
    int M, Kt, ksh, T, Tpad, out_bf16;
};

// Two small integers -> a packed pair of fp16 values (exact for |v| <= 2048).
__device__ __forceinline__ uint32_t h2_of(int lo, int hi) {
    return (uint32_t)__half_as_ushort(__int2half_rn(lo)) | ((uint32_t)__half_as_ushort(__int2half_rn(hi)) << 16);
}

// One token's 32 codes of a k-tile -> its four 16-byte fp16 K-chunks in the image: chunk j
// holds k = 8j + {0,4,1,5,2,6,3,7} (the order the weight expansion produces).
__device__ __forceinline__ void store_token_chunks(uint8_t *blk, int tl, const int (&v)[32]) {
    uint8_t *dst = blk + (tl >> 3) * kSboH + (tl & 7) * 16;
#pragma unroll
    for (int j = 0; j < 4; ++j)
        *reinterpret_cast<uint4 *>(dst + j * kLboH) =
            make_uint4(h2_of(v[8 * j], v[8 * j + 4]), h2_of(v[8 * j + 1], v[8 * j + 5]),
                       h2_of(v[8 * j + 2], v[8 * j + 6]), h2_of(v[8 * j + 3], v[8 * j + 7]));
}

// Part of both pre-passes: sets *flag if any scale word of the weight carries a zero point
// other than 0 (its low nibble). The GEMM is compiled with and without the zero-point term;
// the flag says which of the two kernels does the work.
__device__ __forceinline__ void scan_zero_points(const uint16_t *__restrict__ scales, size_t n,
                                                 int *__restrict__ flag) {
    const uint4 *v = reinterpret_cast<const uint4 *>(scales);      // 8 words at a time (n % 16 == 0)
    uint32_t any = 0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n / 8; i += (size_t)gridDim.x * blockDim.x) {
        const uint4 w = __ldg(v + i);
        any |= (w.x | w.y | w.z | w.w) & 0x000F000Fu;
    }
    if (__any_sync(0xffffffffu, any != 0) && (threadIdx.x & 31) == 0) atomicOr(flag, 1);
}

// Pre-pass: the caller's staging (aq[kt][tok][32], as[kt][tok], asum[kt][tok]) -> the images
// the GEMM tiles copy with one bulk copy each. Tokens >= T are padded with zeros.
__global__ void __launch_bounds__(256)
gemm_tc_prepass_kernel(const int8_t *__restrict__ aq, const float *__restrict__ as,
                       const int32_t *__restrict__ asum, int T, int Tpad, int Kt,
                       uint8_t *__restrict__ img, const uint16_t *__restrict__ scales, size_t nscales,
                       int *__restrict__ zp_flag) {
    pdl_trigger();
    scan_zero_points(scales, nscales, zp_flag);
    const size_t nrow = (size_t)Kt * Tpad;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < nrow; i += (size_t)gridDim.x * 256) {
        const int kt = (int)(i / Tpad), tok = (int)(i % Tpad);
        int v[32];
#pragma unroll
        for (int k = 0; k < 32; ++k) v[k] = 0;
        if (tok < T) {
            const uint4 *src = reinterpret_cast<const uint4 *>(aq + ((size_t)kt * T + tok) * 32);
            const uint4 a = __ldg(src), b = __ldg(src + 1);    // k = 0..15, 16..31
            const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
            for (int k = 0; k < 32; ++k) v[k] = (int)(int8_t)(w[k >> 2] >> ((k & 3) * 8));
        }
        uint8_t *blk = img + ((size_t)(tok / kTN) * Kt + kt) * kImgBytes;
        const int tl = tok % kTN;
        store_token_chunks(blk, tl, v);
        float *sa = reinterpret_cast<float *>(blk + kBBytes);
        sa[tl] = (tok < T && as) ? as[(size_t)kt * T + tok] : 0.0f;
        sa[kTN + tl] = tok < T ? (float)asum[(size_t)kt * T + tok] : 0.0f;
    }
}

// W4A4 pre-pass: packed int4 activations aq4[kt64][tok][32] (byte b = k 2b, 2b+1 of the 64),
// as4 / asum4 per (kt64, tok) -> the same images as above, two K32 images per K64 block. The
// block's scale and code sum go with its first K32 image; the second one carries zeros, so
// the GEMM that adds the two sums of a promote group gets the block's sum.
__global__ void __launch_bounds__(256)
gemm_tc_prepass_s4_kernel(const uint8_t *__restrict__ aq4, const float *__restrict__ as4,
                          const int32_t *__restrict__ asum4, int T, int Tpad, int Kt,
                          uint8_t *__restrict__ img, const uint16_t *__restrict__ scales, size_t nscales,
                          int *__restrict__ zp_flag) {
    pdl_trigger();
    scan_zero_points(scales, nscales, zp_flag);
    const size_t nrow = (size_t)Kt * Tpad;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < nrow; i += (size_t)gridDim.x * 256) {
        const int kt = (int)(i / Tpad), tok = (int)(i % Tpad);
        const int kg = kt >> 1, half = kt & 1;
        int v[32];
#pragma unroll
        for (int k = 0; k < 32; ++k) v[k] = 0;
        if (tok < T) {
            const uint4 a = __ldg(reinterpret_cast<const uint4 *>(aq4 + ((size_t)kg * T + tok) * 32) + half);
            const uint32_t w[4] = {a.x, a.y, a.z, a.w};
            // byte b of the half = k 2b (low nibble), 2b + 1 (high nibble); two's complement
#pragma unroll
            for (int k = 0; k < 32; ++k) v[k] = ((int)(w[k >> 3] << (28 - (k & 7) * 4))) >> 28;
        }
        uint8_t *blk = img + ((size_t)(tok / kTN) * Kt + kt) * kImgBytes;
        const int tl = tok % kTN;
        store_token_chunks(blk, tl, v);
        float *sa = reinterpret_cast<float *>(blk + kBBytes);
        const bool has = half == 0 && tok < T;
        sa[tl] = has ? as4[(size_t)kg * T + tok] : 0.0f;
        sa[kTN + tl] = has ? (float)asum4[(size_t)kg * T + tok] : 0.0f;
    }
}

// Eight two's-complement nibbles of w (nibble i = code k = i) -> eight fp16 values, as four
// words holding the codes (0,4), (1,5), (2,6), (3,7). Per word: the two nibbles land in the
// low bits of the two halves; xor with 0x6408 sets fp16's exponent of 1024 and flips the
// code's sign bit, so the half reads 1024 + (q + 8); subtracting 1032 leaves q. mask and
// bias (0x000F000F, 0x64086408) are passed in registers the caller keeps alive: as literals
// each use costs a move that materialises the constant.
__device__ __forceinline__ uint4 nib8_to_h8(uint32_t w, uint32_t mask, uint32_t bias) {
    uint32_t r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t t;                                        // ((w >> 4i) & mask) ^ bias in one logic op
        asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(t) : "r"(w >> (4 * i)), "r"(mask), "r"(bias));
        asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r[i]) : "r"(t), "r"(bias));
    }
    return make_uint4(r[0], r[1], r[2], r[3]);
}

// Weight pre-pass: packed codes [row group][k-tile][16 rows][16 B] -> per (128-row block,
// k-tile) the kABytes of fp16 values in the operand layout (row groups of 8 are kSboH apart,
// a row's four 16-byte K-chunks kLboH apart), so that a tile's weights of a k-tile are one bulk
// copy. A thread expands one row of one k-tile; 8 consecutive lanes write 128 contiguous bytes
// per chunk. 4 bytes out per code: 178 MB for 17408 x 5120, written and read once per call.
__global__ void __launch_bounds__(256)
gemm_tc_expand_kernel(const uint8_t *__restrict__ codes, int M, int Kt, uint8_t *__restrict__ wimg) {
    pdl_trigger();
    const uint32_t mask = 0x000F000Fu, bias = 0x64086408u;
    const size_t n = (size_t)M * Kt;
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n; i += (size_t)gridDim.x * 256) {
        const int kt = (int)(i / M), m = (int)(i % M);
        const uint4 c4 = ldg_stream_v4(codes + ((size_t)(m >> 4) * Kt + kt) * 256 + (m & 15) * 16);
        const int r = m & (kTM - 1);
        uint8_t *dst = wimg + ((size_t)(m / kTM) * Kt + kt) * kABytes + (r >> 3) * kSboH + (r & 7) * 16;
        *reinterpret_cast<uint4 *>(dst) = nib8_to_h8(c4.x, mask, bias);                 // k 0..7
        *reinterpret_cast<uint4 *>(dst + kLboH) = nib8_to_h8(c4.y, mask, bias);         // k 8..15
        *reinterpret_cast<uint4 *>(dst + 2 * kLboH) = nib8_to_h8(c4.z, mask, bias);     // k 16..23
        *reinterpret_cast<uint4 *>(dst + 3 * kLboH) = nib8_to_h8(c4.w, mask, bias);     // k 24..31
    }
}

constexpr int kWaitMma = 21, kWaitEpi = 22, kWaitProd = 23;   // status codes of failed waits

// Trace build (-DTQ_TC_TRACE): every role of CTA 0 adds up clock64() differences per section
// of its loop (TCT(i) closes section i); qwn_dbg_tc_trace copies the sums out: rows 0..15
// the worker warps, 16 the copy thread, 17 and 18 the MMA threads. Compiled out otherwise.
#ifdef TQ_TC_TRACE
__device__ long long g_tc_trace[20 * 16];
#define TCT_DECL long long tct_[12] = {}; long long tct_t = clock64();
#define TCT(i) { const long long t_ = clock64(); tct_[i] += t_ - tct_t; tct_t = t_; }
#define TCT_OUT(slot) if (blockIdx.x == 0 && lane == 0) { for (int i_ = 0; i_ < 12; ++i_) g_tc_trace[(slot) * 16 + i_] = tct_[i_]; }
#else
#define TCT_DECL
#define TCT(i)
#define TCT_OUT(slot)
#endif

// GW = k-tiles accumulated in TMEM before one fp32 promote (1: the reference's arithmetic with
// a scale per (token, K32); 2: K64 weight groups with per-token activation scales, or - not
// PERTOK - with one activation scale per (token, K64): the W4A4 arithmetic). PERTOK:
// the activation scale is applied once at the end (y = acc * as_tok).
//
// The K loop advances in steps of two k-tiles (K is a multiple of 64); step n of the CTA
// (counted across its tiles) uses step slot n % kSS. A worker warp owns 32 TMEM lanes (rows)
// and 32 of the tile's tokens.
//
// ZP: the kernel applies the zero-point term f = d - z * asum. Both variants are launched;
// the one that does not match the pre-pass's flag returns at once.
template <int GW, bool PERTOK, bool ZP>
__global__ void __maxnreg__(kMaxRegs) gemm_w4a8_tc_kernel(const TcParams p) {
    pdl_trigger();
    pdl_wait();      // everything below reads what earlier kernels wrote (flag, images)
    if ((*p.zp_flag != 0) != ZP) return;
    // per-token scales and no zero points: the promote reads neither as nor asum from the slot
    constexpr bool kSlotFreedByMma = PERTOK && !ZP;
    // One K64 group per step, per-token scales, no zero points: the promote is a bare fma per
    // output, and as packed fma on token pairs it is half as many instructions (5 % faster;
    // in every other mode the packed form measured 8 to 11 % slower than scalar fma).
    constexpr bool kPacked = PERTOK && !ZP && GW == 2;
    // the step loop of that mode is short enough to gain from two copies (1 to 2 %; four lose 4 %,
    // and the other modes lose with two)
    constexpr int kStepUnroll = (PERTOK && GW == 2) ? 2 : 1;
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ uint64_t bars[2 * kSS + 2 * kNB];   // full[kSS], empty[kSS], accfull[kNB], accempty[kNB]
    __shared__ uint32_t tmem_base_s;
    __shared__ int dead_s;                      // a wait gave up somewhere in the CTA
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t smem_u = smem_u32(smem);
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kSS]),
                   acc0 = smem_u32(&bars[2 * kSS]), accempty0 = smem_u32(&bars[2 * kSS + kNB]);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kSS; ++s) {
            mbar_init(full0 + s * 8, 1);                 // the copy thread's arrive with the step's byte count
            // a slot is free when every worker warp has read its activation scales - or, in
            // the variant whose workers read nothing from the slot, when its MMAs are complete
            mbar_init(empty0 + s * 8, kSlotFreedByMma ? 1 : kWorkWarps);
        }
        for (int b = 0; b < kNB; ++b) {
            mbar_init(acc0 + b * 8, 1);                  // tcgen05.commit
            mbar_init(accempty0 + b * 8, kWorkWarps);    // one arrive per worker warp
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

    const int Kt = p.Kt, Ktg = Kt >> p.ksh;
    const int spt = Kt >> 1;                             // steps per tile
    const int row_blocks = p.M / kTM, tok_blocks = p.Tpad / kTN;
    const int ntiles = row_blocks * tok_blocks;
    const int my_tiles = (ntiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int n_total = my_tiles * spt;                  // steps of this CTA

    // A wait that gives up when another role already has: the flag is read on the slow path only.
    auto wait_on = [&](uint32_t bar, uint32_t parity, int code, uint32_t suspend_ns = 0) -> bool {
        if (mbar_test_wait(bar, parity)) return true;
        if (*(volatile int *)&dead_s) return false;
        if (mbar_wait_slow(bar, parity, p.status, code, p.wait_ns, suspend_ns)) return true;
        dead_s = 1;
        return false;
    };

    if (warp < kWorkWarps) {
        // ====================== workers: promote the accumulators ==========================
        const int q4 = warp & 3, chalf = (warp >> 2) * kWT;   // lane quarter, first token
        const int rloc = q4 * 32 + lane;                  // row inside the tile = TMEM lane
        const uint32_t lane_base = tmem_base + ((uint32_t)(q4 * 32) << 16) + chalf;
        // activation scales of this thread's tokens inside a step slot (as four-token
        // vectors: [0, 16) scales, [32, 48) code sums)
        const unsigned char *sv_base = smem + 2 * kABytes + kBBytes + chalf * 4;
        int n = 0;                                        // step counter across the CTA's tiles
        int ss = 0;                                       // n % kSS, kept as a counter
        // The thread's 32 columns of a group's accumulator. (Issuing the load of the next
        // group behind this group's fma, when its barrier had already completed, measured
        // slower than this plain sequence: with five warps per scheduler the other warps cover
        // a load's latency, and every instruction saved counts.)
        uint32_t d[kWT];
        static_assert(kWT == 32, "one 32-column load per group");
        TCT_DECL

        for (int ti = 0; ti < my_tiles; ++ti) {
            const int tile = (int)blockIdx.x + ti * (int)gridDim.x;
            const int tb = tile % tok_blocks, rb = tile / tok_blocks;
            const int row = rb * kTM + rloc;
            const uint16_t *sc = p.scales + ((size_t)(row >> 4) * Ktg) * 16 + (row & 15);
            float acc[kWT];
#pragma unroll
            for (int i = 0; i < kWT; ++i) acc[i] = 0.0f;
            f32x2 accp[kWT / 2];                          // the same as pairs (kPacked)
#pragma unroll
            for (int i = 0; i < kWT / 2; ++i) accp[i] = 0ull;
            uint32_t scw = __ldg(sc);
            const uint16_t *scn = sc;                     // the word of the group being promoted
#pragma unroll kStepUnroll
            for (int s = 0; s < spt; ++s, ++n, ss = (ss + 1 == kSS) ? 0 : ss + 1) {
#pragma unroll
                for (int g = 0; g < (GW == 2 ? 1 : 2); ++g) {
                    TCT(7)
                    const int kt = 2 * s + g;              // first k-tile of the group
                    // One barrier round per step: a K64 group per step uses the four 128-column
                    // buffers in turn; two K32 groups per step share a 256-column buffer pair
                    // (k-tile g in its half), with one wait and one arrival for both.
                    const int b = (GW == 2) ? (n & 3) : (n & 1);
                    const uint32_t par = (GW == 2) ? ((uint32_t)n >> 2) & 1u : ((uint32_t)n >> 1) & 1u;
                    const uint32_t col = (GW == 2) ? b * kTN : (2 * b + g) * kTN;
                    int zp;
                    float ws;
                    unpack_scale(scw, zp, ws);
                    // the next group's word: the next one in the row's run, except inside a K64
                    // pair promoted per k-tile, whose second tile shares the first one's
                    if (GW == 2 || g == 1 || p.ksh == 0) scn += 16;
                    if (kt + GW < Kt) scw = __ldg(scn);
                    const f32x2 ws2 = pack2(ws, ws);
                    const float nzf = (float)(-zp);
                    TCT(0)
                    if (GW == 2 || g == 0) {
                        if (!__all_sync(0xffffffffu, wait_on(acc0 + b * 8, par, kWaitEpi, kNapNs))) goto gave_up;
                        tc_fence_after();
                    }
                    // the accumulator holds (float)d of the group (the group's first MMA
                    // overwrites it): nothing has to be converted or stored back
                    tmem_ld32(lane_base + col, d);
                    TCT(1)
                    const ulonglong2 *sv = reinterpret_cast<const ulonglong2 *>(
                        sv_base + (size_t)ss * kStepBytes + g * kImgBytes);
                    // second k-tile of a K64 group: only its code sums are needed
                    const ulonglong2 *sv1 = reinterpret_cast<const ulonglong2 *>(
                        sv_base + (size_t)ss * kStepBytes + kImgBytes);
                    // symmetric weights need no zero-point term at all (the weights enter the
                    // MMA as true signed values): ZP is a compile-time choice, a test inside the
                    // unrolled loop would split it into one basic block per token group
                    auto promote = [&](int j0, int j1) {
                        if constexpr (kPacked) {
#pragma unroll
                            for (int j = 2 * j0; j < 2 * j1; ++j)
                                fma2_acc(accp[j], pack2(__uint_as_float(d[2 * j]), __uint_as_float(d[2 * j + 1])), ws2);
                        } else {
#pragma unroll
                            for (int j = j0; j < j1; ++j) {     // four tokens at a time
                                // scalar fmas on the loaded registers as they are
                                float f[4];
#pragma unroll
                                for (int i = 0; i < 4; ++i) f[i] = __uint_as_float(d[4 * j + i]);
                                if (ZP) {
                                    ulonglong2 sm = sv[32 + j];                        // four code sums
                                    if (GW == 2) {                                     // exact: small integers
                                        const ulonglong2 sm1 = sv1[32 + j];
                                        sm.x = add2(sm.x, sm1.x);
                                        sm.y = add2(sm.y, sm1.y);
                                    }
                                    float m[4];
                                    unpack2(sm.x, m[0], m[1]);
                                    unpack2(sm.y, m[2], m[3]);
#pragma unroll
                                    for (int i = 0; i < 4; ++i) f[i] = fmaf(nzf, m[i], f[i]);
                                }
                                float w[4] = {ws, ws, ws, ws};
                                if (!PERTOK) {
                                    const ulonglong2 a4 = sv[j];                       // four activation scales
                                    unpack2(mul2(ws2, a4.x), w[0], w[1]);              // ws * as, rounded once
                                    unpack2(mul2(ws2, a4.y), w[2], w[3]);
                                }
#pragma unroll
                                for (int i = 0; i < 4; ++i) acc[4 * j + i] = fmaf(f[i], w[i], acc[4 * j + i]);
                            }
                        }
                    };
                    TCT(2)
                    tmem_wait_ld_all();
                    TCT(3)
                    promote(0, kWT / 4);
                    TCT(4)
                    if (GW == 2 || g == 1) {
                        tc_fence_before();
                        __syncwarp();
                        TCT(5)
                        // one instruction, two barriers: lane 0 tells the MMA that it may overwrite
                        // the buffer, lane 1 the copy thread that the slot's images may be replaced
                        if (!kSlotFreedByMma)
                            mbar_arrive_if(lane == 0 ? accempty0 + b * 8 : empty0 + ss * 8, lane < 2);
                        else
                            mbar_arrive_if(accempty0 + b * 8, lane == 0);
                    }
                    TCT(6)
                }
            }
            // store: thread = row, its tokens; rows are contiguous in y, so a warp writes 128 B
#pragma unroll
            for (int i = 0; i < kWT / 2; ++i) {
                float v0 = acc[2 * i], v1 = acc[2 * i + 1];
                if (kPacked) unpack2(accp[i], v0, v1);
                const int tok = tb * kTN + chalf + 2 * i;
                if (PERTOK) {
                    if (tok < p.T) v0 = __fmul_rn(v0, __ldg(p.as_tok + tok));
                    if (tok + 1 < p.T) v1 = __fmul_rn(v1, __ldg(p.as_tok + tok + 1));
                }
                if (p.out_bf16) {
                    __nv_bfloat16 *y = static_cast<__nv_bfloat16 *>(p.y);
                    if (tok < p.T) __stcs(reinterpret_cast<unsigned short *>(y + (size_t)tok * p.M + row), __bfloat16_as_ushort(__float2bfloat16_rn(v0)));
                    if (tok + 1 < p.T) __stcs(reinterpret_cast<unsigned short *>(y + (size_t)(tok + 1) * p.M + row), __bfloat16_as_ushort(__float2bfloat16_rn(v1)));
                } else {
                    float *y = static_cast<float *>(p.y);
                    if (tok < p.T) __stcs(y + (size_t)tok * p.M + row, v0);
                    if (tok + 1 < p.T) __stcs(y + (size_t)(tok + 1) * p.M + row, v1);
                }
            }
        }
    gave_up:;
        TCT_OUT(warp)
    } else if (warp == kWorkWarps) {
        // ====================== image copies (one thread) =================================
        // Two bulk copies per step: the fp16 weights of the tile's row block and the activation
        // images of its token block, both k-tiles of the step at once; the slot's previous
        // contents must have been promoted by every worker warp (their MMAs are then complete).
        if (lane == 0) {
            int ss = 0;                    // step slot and the parity of its use, kept as counters
            uint32_t ph = 0;
            TCT_DECL
            for (int ti = 0; ti < my_tiles; ++ti) {
                const int tile = (int)blockIdx.x + ti * (int)gridDim.x;
                const int tb = tile % tok_blocks, rb = tile / tok_blocks;
                const uint8_t *src = p.img + (size_t)tb * Kt * kImgBytes;
                const uint8_t *wsrc = p.wimg + (size_t)rb * Kt * kABytes;
                bool ok = true;
                for (int s = 0; s < spt; ++s, src += 2 * kImgBytes, wsrc += 2 * kABytes) {
                    TCT(0)
                    ok = wait_on(empty0 + ss * 8, ph ^ 1u, kWaitProd, kNapNs);
                    TCT(1)
                    if (!ok) break;
                    const uint32_t fb = full0 + ss * 8;
                    const uint32_t dst = smem_u + ss * kStepBytes;
                    mbar_expect_tx(fb, kStepBytes);
                    bulk_g2s_plain(dst, wsrc, 2 * kABytes, fb);
                    bulk_g2s_plain(dst + 2 * kABytes, src, 2 * kImgBytes, fb);
                    if (++ss == kSS) {
                        ss = 0;
                        ph ^= 1u;
                    }
                    TCT(2)
                }
                if (!ok) break;
            }
            // No copy may still be in flight when the CTA gives its shared memory back: wait
            // (bounded) until the last armed use of every slot has all its bytes. On the normal
            // path every one of them was consumed long ago and these tests return at once; after
            // a wait that gave up somewhere, this is where the copies already started drain.
            for (int s2 = 0; s2 < kSS; ++s2) {
                const uint32_t last = (s2 < ss) ? ph : (ph ^ 1u);     // this round's use, or the one before
                if (!mbar_test_wait(full0 + s2 * 8, last))
                    mbar_wait_slow(full0 + s2 * 8, last, p.status, kWaitProd, p.wait_ns, kNapNs);
            }
            TCT_OUT(16)
        }
    } else {
        // ====================== MMA issuers (one thread per warp, steps in turn) ===========
        if (lane == 0) {
            const int mw = warp - (kWorkWarps + 1);
            const uint64_t desc0 = smem_desc_at(smem_u, kLboH, kSboH);
            TCT_DECL
            int ss = mw;                   // step slot and the parity of its use, kept as counters
            uint32_t ph = 0;
            static_assert(kMmaWarps < kSS, "the first step of every MMA thread is in the first round of slots");
            for (int n = mw; n < n_total; n += kMmaWarps) {
                TCT(0)
                if (!wait_on(full0 + ss * 8, ph, kWaitMma, kNapNs)) break;
                TCT(1)
                bool ok = true;
#pragma unroll
                for (int h = 0; h < 2; ++h) {              // the step's two k-tiles
                    const int b = (GW == 2) ? (n & 3) : (n & 1);
                    const uint32_t par = (GW == 2) ? ((uint32_t)n >> 2) & 1u : ((uint32_t)n >> 1) & 1u;
                    const uint32_t col = (GW == 2) ? b * kTN : (2 * b + h) * kTN;
                    // the step's accumulator buffer (or pair) has been read out
                    if (h == 0) {
                        ok = wait_on(accempty0 + b * 8, par ^ 1u, kWaitMma, kNapNs);
                        if (!ok) break;
                        tc_fence_after();
                    }
                    TCT(2)
                    const uint64_t da = desc0 + (uint64_t)((ss * kStepBytes + h * kABytes) >> 4);
                    const uint64_t db = desc0 + (uint64_t)((ss * kStepBytes + 2 * kABytes + h * kImgBytes) >> 4);
                    // the first MMA of a promote group overwrites the accumulator
                    tc_mma_f16(tmem_base + col, da, db, kIdesc, (GW == 2 && h == 1) ? 1u : 0u);
                    tc_mma_f16(tmem_base + col, da + (2 * kLboH >> 4), db + (2 * kLboH >> 4), kIdesc, 1u);
                    if (h == 1) tc_commit(acc0 + b * 8);
                    // the step's operands have been read when its MMAs are complete
                    if (kSlotFreedByMma && h == 1) tc_commit(empty0 + ss * 8);
                    TCT(3)
                }
                if (!ok) break;
                ss += kMmaWarps;
                if (ss >= kSS) {
                    ss -= kSS;
                    ph ^= 1u;
                }
            }
            TCT_OUT(17 + mw)
        }
    }

    // ---- teardown: every role comes here, also after a failed wait ------------------------
    if (warp < kWorkWarps) tmem_wait_ld_all();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) tmem_dealloc(tmem_base, 512);
}

struct TcScratch {
    uint8_t *img = nullptr;
    size_t img_bytes = 0;
    uint8_t *wimg = nullptr;      // fp16 image of the call's weight (4 bytes per code)
    size_t wimg_bytes = 0;
    int *zp_flag = nullptr;
} g_tc;

int g_tc_sms = 0;

}  // namespace

int launch_gemm_tc(const GemmTcArgs &a) {
    // covered: per-block activation scales (the reference's x_gemm_w4a8 arithmetic) or
    // per-token scales, rows a multiple of 128, K a multiple of 64
    if (!a.as == !a.as_tok) return -1;          // exactly one kind of activation scale
    if (a.aq4 && (!a.as || !a.ksh)) return -1;  // W4A4: K64 weights, scale per (token, K64)
    if (a.M % kTM || a.K % 64 || a.T < 128) return -1;     // steps of two k-tiles
    const int Kt = a.K / 32;
    if (!g_tc_sms) {
        int dev = 0;
        TQ_CHECK(cudaGetDevice(&dev));
        TQ_CHECK(cudaDeviceGetAttribute(&g_tc_sms, cudaDevAttrMultiProcessorCount, dev));
        if (g_tc_sms <= 0) g_tc_sms = 148;
        auto big_smem = [](auto kernel) {
            return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        };
        TQ_CHECK(big_smem(gemm_w4a8_tc_kernel<1, false, false>));
        TQ_CHECK(big_smem(gemm_w4a8_tc_kernel<1, false, true>));
        TQ_CHECK(big_smem(gemm_w4a8_tc_kernel<1, true, false>));
        TQ_CHECK(big_smem(gemm_w4a8_tc_kernel<1, true, true>));
        TQ_CHECK(big_smem(gemm_w4a8_tc_kernel<2, true, false>));
        TQ_CHECK(big_smem(gemm_w4a8_tc_kernel<2, true, true>));
        TQ_CHECK(big_smem(gemm_w4a8_tc_kernel<2, false, false>));
        TQ_CHECK(big_smem(gemm_w4a8_tc_kernel<2, false, true>));
        g_tc.zp_flag = static_cast<int *>(tq_dev_alloc(sizeof(int), "gemm.tc.zero-point.flag"));
    }
    ProfScope prof(a.M, a.K, a.T, a.aq4 ? 44 : (a.ksh ? 64 : 4));
    const int Tpad = (a.T + kTN - 1) / kTN * kTN;
    const size_t ibytes = (size_t)Kt * (Tpad / kTN) * kImgBytes;
    if (ibytes > g_tc.img_bytes) {
        if (g_tc.img) tq_dev_free(g_tc.img);
        g_tc.img = static_cast<uint8_t *>(tq_dev_alloc(ibytes, "gemm.tc.activation.image"));
        g_tc.img_bytes = ibytes;
    }
    const size_t wbytes = (size_t)a.M * a.K * 2;
    if (wbytes > g_tc.wimg_bytes) {
        if (g_tc.wimg) tq_dev_free(g_tc.wimg);
        g_tc.wimg = static_cast<uint8_t *>(tq_dev_alloc(wbytes, "gemm.tc.weight.image"));
        g_tc.wimg_bytes = wbytes;
    }
    const size_t nrow = (size_t)Kt * Tpad;
    const int pgrid = (int)std::min<size_t>((nrow + 255) / 256, (size_t)g_tc_sms * 8);
    const size_t nscales = (size_t)a.M * (Kt >> a.ksh);
    TQ_CHECK(cudaMemsetAsync(g_tc.zp_flag, 0, sizeof(int), stream()));
    if (a.aq4)
        gemm_tc_prepass_s4_kernel<<<pgrid, 256, 0, stream()>>>(a.aq4, a.as, a.asum, a.T, Tpad, Kt,
                                                              g_tc.img, a.scales, nscales, g_tc.zp_flag);
    else
        gemm_tc_prepass_kernel<<<pgrid, 256, 0, stream()>>>(a.aq, a.as, a.asum, a.T, Tpad, Kt, g_tc.img,
                                                           a.scales, nscales, g_tc.zp_flag);
    TQ_LAUNCH_CHECK("gemm_tc_prepass_kernel");
    {
        const size_t items = (size_t)a.M * Kt;
        const int egrid = (int)std::min<size_t>((items + 255) / 256, (size_t)g_tc_sms * 16);
        gemm_tc_expand_kernel<<<egrid, 256, 0, stream()>>>(a.codes, a.M, Kt, g_tc.wimg);
        TQ_LAUNCH_CHECK("gemm_tc_expand_kernel");
    }
    TcParams p{};
    p.wimg = g_tc.wimg; p.scales = a.scales; p.img = g_tc.img; p.y = a.y;
    p.status = device_status_word();
    p.wait_ns = wait_limit_ns();
    p.M = a.M; p.Kt = Kt; p.ksh = a.ksh; p.T = a.T; p.Tpad = Tpad; p.out_bf16 = a.out_bf16;
    const int ntiles = (a.M / kTM) * (Tpad / kTN);
    const int grid = std::min(g_tc_sms, ntiles);
    p.as_tok = a.as_tok;
    p.zp_flag = g_tc.zp_flag;
    // both variants of the kernel: the one the flag does not select returns at once
    auto both = [&](auto without_zp, auto with_zp) {
        launch_pdl(without_zp, dim3(grid), dim3(kThreads), (size_t)kSmemBytes, p);
        launch_pdl(with_zp, dim3(grid), dim3(kThreads), (size_t)kSmemBytes, p);
    };
    if (a.aq4)
        both(gemm_w4a8_tc_kernel<2, false, false>, gemm_w4a8_tc_kernel<2, false, true>);
    else if (!a.as_tok)
        both(gemm_w4a8_tc_kernel<1, false, false>, gemm_w4a8_tc_kernel<1, false, true>);
    else if (a.ksh)
        both(gemm_w4a8_tc_kernel<2, true, false>, gemm_w4a8_tc_kernel<2, true, true>);
    else
        both(gemm_w4a8_tc_kernel<1, true, false>, gemm_w4a8_tc_kernel<1, true, true>);
    TQ_LAUNCH_CHECK("gemm_w4a8_tc_kernel");
    return 0;
}

}  // namespace tq

#ifdef TQ_TC_TRACE
extern "C" void qwn_dbg_tc_trace(long long *host) {
    cudaMemcpyFromSymbol(host, tq::g_tc_trace, sizeof(long long) * 320);
}
#endif
