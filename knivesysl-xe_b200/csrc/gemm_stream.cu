// gemm_stream.cu — batched W4A8 GEMM for decode batches (T = 8..64 tokens, one segment)
// on sm_100a. Two persistent kernels: gemm_w4a8_ring_kernel (windows of eight tokens: 32 warps
// per SM, per-warp cp.async ring in shared memory, further down) and gemm_w4a8_stream_kernel
// (the shapes whose window activations do not fit beside the rings, and the int32 dump used by
// the tests), in which every warp streams packed weights from HBM straight into registers, a
// chunk of eight k-tiles ahead of the math.
//
// Replaces x_gemm_w4a8's split path (xpu/src/kernels_dpas.cpp:1379-1489) for the shapes
// decode uses. The kernel is HBM-bound on the packed weight stream; what limits it in
// practice is the shared-memory/L1 data path (128 B per clock per SM) and the issue slots
// spent per 256-byte tile, so the design keeps both small:
//  * one CTA per SM, 16 warps (24 when that saves a pass). All warps of a CTA work on the SAME K-split s (CTA b takes
//    s = b % S), each warp on its own 16-row groups. Lane (r, c) loads word c of rows r
//    and r+8 of a tile (two coalesced 128-byte requests per tile, L1 not allocated) -
//    exactly the A fragment of mma.sync.m16n8k32 - into one of two register buffers of
//    eight tiles: all loads of chunk n+1 are issued before the math of chunk n, so they
//    complete as one batch, and the sequence runs across the row-groups a warp owns, so
//    loads never drain inside the kernel;
//  * a CTA only needs the activations of one K-split: they are staged ONCE per CTA in
//    shared memory in the form the tile loop consumes - int8 codes in MMA B-fragment
//    order, and per (k-tile, token pair) {as0, as1, (float)asum0, (float)asum1}
//    (STAGED). Shapes whose activations do not fit read them through L1 instead;
//  * scale words are fetched one chunk ahead and expanded once per chunk into fp32
//    {ws, -(z+8)} pairs in a small per-warp buffer;
//  * nibbles are used as q+8 (one lop3 per four codes) and the correction folds into the
//    zero-point term: d - z*asum == d' - (z+8)*asum; the MMA accumulator starts at the bit
//    pattern of 12582912.0f, so the exact int32 result becomes fp32 with one add instead
//    of a conversion; (float)(d - z*asum) is formed exactly in fp32 (all terms are integers
//    below 2^24) and the promote term (float)(d - z*asum) * (ws*as) is accumulated with fma
//    in ascending k-tile order on packed f32x2 instructions (two outputs per issue slot);
//  * K-splits of one row-group live in different CTAs. Each writes its partial tile to a
//    small global scratch, and the warp that arrives last (a counter per row-group) adds
//    the S partials in the order 0..S-1 starting from 0.0f and stores y: the reference's
//    summation order, independent of arrival order. An unsplit weight stores its
//    accumulator untouched;
//  * with the fused all-gather (a.npeer > 0) the epilogue stores the tile into the gathered
//    buffer of every rank; the step flag that tells the peers is stored by a one-warp kernel
//    launched right after this one (comm.cu), i.e. at the kernel boundary, so no CTA of
//    this kernel pays for a fence.
// (With 16 warps per SM a shared-memory ring fed by cp.async, and before it by 1-D bulk TMA
// copies, measured slower than the register queue: every weight byte crosses the
// shared-memory data path twice more, and one warp sustains only about two bulk copies in
// flight. The ring pays off once it frees enough registers for 32 warps per SM: the T = 8
// kernel below.)
#include "stream.cuh"

#include <algorithm>
#include <type_traits>

namespace tq {

namespace {

constexpr int kCT = 8;                          // k-tiles per chunk (register queue depth)
constexpr int kWmax = 24;                       // most warps per CTA of any variant
constexpr int kExpBytes = kCT * 16 * 8;         // expanded scales of one chunk, per group
constexpr int kActTileBytes = 256 + 64;         // staged activations per (k-tile, 8 tokens)

__device__ __forceinline__ uint32_t ldg_stream_u16(const uint16_t *p) {
    uint16_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

template <int NTG, bool STAGED, bool DUMP, int kW>
__global__ void __launch_bounds__(kW * 32, 1)
gemm_w4a8_stream_kernel(const GemmArgs a, float *__restrict__ part, int *__restrict__ count) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int T = NTG * 8;              // tokens of this CTA's window
    const int Ttot = a.T;                   // tokens of the call (row stride of the staging)
    const int win = blockIdx.y;             // token window: tokens [tok0, tok0 + T)
    const int tok0 = win * T;
    constexpr int G = 1;   // 16-row groups a warp works on at a time (kept as a loop bound)
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int r = lane >> 2;
    const int c = lane & 3;
    const int row16 = lane & 15, th = lane >> 4;            // roles in the scale expansion
    const int S = a.max_splits;
    const int split = blockIdx.x % S;
    const int cta_i = blockIdx.x / S;                       // index among the CTAs of this split
    const int nctas = (gridDim.x - split + S - 1) / S;      // CTAs that share this split

    float2 *expw = reinterpret_cast<float2 *>(smem) + warp * (G * 128);
    unsigned char *act = smem + (size_t)kW * G * kExpBytes;

    const int groups_all = a.goff[a.count];
    const int units = groups_all / G;                       // a unit = G adjacent row-groups
    const int tgid = cta_i + nctas * warp;                  // first unit of this warp
    const int tstride = nctas * kW;
    const int ntasks = (tgid < units) ? (units - tgid + tstride - 1) / tstride : 0;
    const int Kt = a.K >> 5;
    const int ksh = a.ksh;
    const int Ktg = Kt >> ksh;
    const int kt_begin = Kt * split / S;
    const int cnt = Kt * (split + 1) / S - kt_begin;
    const int nch = (cnt + kCT - 1) / kCT;
    const size_t gstride_c = (size_t)Kt * 256u;             // next row-group: codes, bytes
    const int gstride_s = Ktg * 16;                         // next row-group: scale words

    // ---- producer: descriptor of the chunk that is loaded next ------------------------
    int p_ci = 0, p_u = tgid, p_left = ntasks * nch;
    const uint8_t *t_c = nullptr;      // codes of the producer's task at kt_begin (+ lane part)
    const uint16_t *t_s = nullptr;     // scale words of its first row-group (+ row16)
    const uint8_t *nx_c = nullptr;
    const uint16_t *nx_s = nullptr;
    int nx_nt = 0, nx_kt0 = 0;
    auto advance = [&]() {
        if (p_left == 0) {
            nx_nt = 0;
            return;
        }
        --p_left;
        if (p_ci == 0) {
            const int g0 = p_u * G;
            int wi = 0;
            while (wi + 1 < a.count && g0 >= a.goff[wi + 1]) ++wi;
            const int lg = g0 - a.goff[wi];
            t_c = a.codes[wi] + ((size_t)lg * Kt + kt_begin) * 256u + r * 16 + c * 4;
            t_s = a.scales[wi] + (size_t)lg * Ktg * 16u + row16;
        }
        nx_c = t_c + (size_t)p_ci * (kCT * 256);
        nx_s = t_s;
        nx_nt = min(kCT, cnt - p_ci * kCT);
        nx_kt0 = kt_begin + p_ci * kCT;
        if (++p_ci == nch) {
            p_ci = 0;
            p_u += tstride;
        }
    };

    // Two register buffers of one chunk each (word c of rows r, r+8 of eight tiles per
    // group): the loads of chunk n+1 are all issued before the math of chunk n starts, so
    // a buffer's loads complete as one batch and nothing waits on loads issued after it.
    uint32_t w0[G][kCT][2], w1[G][kCT][2];
    uint32_t sr[G][4];         // scale words of tiles th, th+2, th+4, th+6, row row16
    // Scale words of the chunk described by nx (tiles beyond its end are not touched).
    auto load_scales = [&]() {
#pragma unroll
        for (int m = 0; m < 4; ++m) {
            const int tl = 2 * m + th;
            if (tl < nx_nt) {
                const uint16_t *p = nx_s + ((nx_kt0 + tl) >> ksh) * 16;
#pragma unroll
                for (int g = 0; g < G; ++g) sr[g][m] = ldg_stream_u16(p + g * gstride_s);
            }
        }
    };
    auto load_chunk = [&](uint32_t (&w)[G][kCT][2]) {
#pragma unroll
        for (int u = 0; u < kCT; ++u)
            if (u < nx_nt) {
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const uint8_t *p = nx_c + g * gstride_c + u * 256;
                    w[g][u][0] = ldg_stream_u32(p);
                    w[g][u][1] = ldg_stream_u32(p + 128);
                }
            }
    };

    // first chunk of this warp: fill the queue
    pdl_trigger();
    advance();
    load_chunk(w0);
    load_scales();
    int cur_nt = nx_nt, cur_kt0 = nx_kt0;
    advance();
    // Everything above reads only packed weights; what follows depends on earlier kernels.
    pdl_wait();

    // Stage this split's activations (all warps; the first weight loads are in flight).
    // Layout per (k-tile, token group): 32 lanes x 8 bytes of codes in B-fragment order
    // (lane (r, c): even-k bytes of token r, k = 8c.., then the odd-k bytes), followed by
    // 4 x 16 bytes {as[2c], as[2c+1], (float)asum[2c], (float)asum[2c+1]}.
    if (STAGED) {
        const int items = cnt * NTG * 32;
        for (int i = threadIdx.x; i < items; i += kW * 32) {
            const int kl = i / (NTG * 32);
            const int rem = i - kl * (NTG * 32);             // = tg * 32 + lane'
            const uint2 bb = __ldg(reinterpret_cast<const uint2 *>(
                a.aq + ((size_t)(kt_begin + kl) * Ttot + tok0) * 32 + (size_t)rem * 8));
            uint2 o;
            o.x = __byte_perm(bb.x, bb.y, 0x6420);
            o.y = __byte_perm(bb.x, bb.y, 0x7531);
            *reinterpret_cast<uint2 *>(act + (size_t)(kl * NTG + (rem >> 5)) * kActTileBytes +
                                       (rem & 31) * 8) = o;
        }
        const int pairs = cnt * NTG * 4;
        for (int i = threadIdx.x; i < pairs; i += kW * 32) {
            const int kl = i / (NTG * 4);
            const int rem = i - kl * (NTG * 4);              // = tg * 4 + c'
            const size_t src = (size_t)(kt_begin + kl) * Ttot + tok0 + (size_t)rem * 2;
            const float2 as2 = __ldg(reinterpret_cast<const float2 *>(a.as + src));
            const int2 sm2 = __ldg(reinterpret_cast<const int2 *>(a.asum + src));
            *reinterpret_cast<float4 *>(act + (size_t)(kl * NTG + (rem >> 2)) * kActTileBytes +
                                        256 + (rem & 3) * 16) =
                make_float4(as2.x, as2.y, (float)sm2.x, (float)sm2.y);
        }
        __syncthreads();
    }

    const f32x2 neg_magic2 = pack2(-kMagicF, -kMagicF);
    int cmagic[4];
    make_const_quad(cmagic, kMagicBits);
    int qpar = 0;                          // which buffer holds the current chunk
    for (int j = 0; j < ntasks; ++j) {
        const int g0 = (tgid + j * tstride) * G;
        int wi = 0;
        while (wi + 1 < a.count && g0 >= a.goff[wi + 1]) ++wi;
        const int lg = g0 - a.goff[wi];
        const int M = a.M[wi];

        f32x2 acc01[G][NTG], acc23[G][NTG];
#pragma unroll
        for (int g = 0; g < G; ++g)
#pragma unroll
            for (int t = 0; t < NTG; ++t) acc01[g][t] = acc23[g][t] = 0ull;

        for (int ci = 0; ci < nch; ++ci, qpar ^= 1) {
          auto chunk = [&](uint32_t (&w)[G][kCT][2], uint32_t (&wn)[G][kCT][2]) {
            // Expand this chunk's scale words into fp32 {ws, -(z+8)}: entry (row, tile pair p)
            // = the pair of tile 2p then of tile 2p+1 (16 bytes) at [p][row], so the tile loop
            // reads a row's scales for two tiles with one 16-byte load and never looks at the
            // tier. Loads and stores are conflict-free.
#pragma unroll
            for (int g = 0; g < G; ++g)
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    int zp;
                    float ws;
                    unpack_scale(sr[g][m], zp, ws);
                    expw[g * 128 + (m * 16 + row16) * 2 + th] = make_float2(ws, (float)(-(zp + 8)));
                }
            __syncwarp();
            load_scales();                 // the next chunk's words, a chunk ahead
            load_chunk(wn);                // ... and all of its weight words

            // activations of this chunk: staged copy in shared memory, or global through L1
            const int kl0 = ci * kCT;
            const unsigned char *actp = act + (size_t)kl0 * NTG * kActTileBytes + lane * 8;
            const unsigned char *asq = act + (size_t)kl0 * NTG * kActTileBytes + 256 + c * 16;
            const int8_t *aqp = a.aq + ((size_t)cur_kt0 * Ttot + tok0 + r) * 32 + c * 8;
            const float *asp = a.as + (size_t)cur_kt0 * Ttot + tok0 + 2 * c;
            const int32_t *smp = a.asum + (size_t)cur_kt0 * Ttot + tok0 + 2 * c;

            // Two tiles (2jp, 2jp+1) of every group of the unit. FULL: the chunk has all 8 tiles.
            auto tile_pair = [&](auto full_tag, const int jp) {
                constexpr bool FULL = decltype(full_tag)::value;
                float4 ea[G], eb[G];
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    ea[g] = *reinterpret_cast<const float4 *>(expw + g * 128 + (jp * 16 + r) * 2);
                    eb[g] =
                        *reinterpret_cast<const float4 *>(expw + g * 128 + (jp * 16 + r + 8) * 2);
                }
#pragma unroll
                for (int uu = 0; uu < 2; ++uu) {
                    const int u = 2 * jp + uu;
                    const bool have = FULL || u < cur_nt;
                    uint32_t A[G][4];
                    if (have) {
#pragma unroll
                        for (int g = 0; g < G; ++g) {
                            A[g][0] = nib_plus8(w[g][u][0]);         // rows r,   even k
                            A[g][1] = nib_plus8(w[g][u][1]);         // rows r+8, even k
                            A[g][2] = nib_plus8(w[g][u][0] >> 4);    // rows r,   odd k
                            A[g][3] = nib_plus8(w[g][u][1] >> 4);    // rows r+8, odd k
                        }
                    }
                    if (!have) continue;
#pragma unroll
                    for (int t = 0; t < NTG; ++t) {
                        uint32_t b0, b1;
                        f32x2 as2, smf;
                        int2 sm2 = make_int2(0, 0);
                        if (STAGED) {
                            const uint2 bb = *reinterpret_cast<const uint2 *>(
                                actp + (u * NTG + t) * kActTileBytes);
                            b0 = bb.x; b1 = bb.y;
                            const ulonglong2 av = *reinterpret_cast<const ulonglong2 *>(
                                asq + (u * NTG + t) * kActTileBytes);
                            as2 = av.x; smf = av.y;
                        } else {
                            const uint2 bb =
                                __ldg(reinterpret_cast<const uint2 *>(aqp + ((size_t)u * Ttot + t * 8) * 32));
                            b0 = __byte_perm(bb.x, bb.y, 0x6420);
                            b1 = __byte_perm(bb.x, bb.y, 0x7531);
                            as2 = __ldg(
                                reinterpret_cast<const unsigned long long *>(asp + (size_t)u * Ttot + t * 8));
                            sm2 = __ldg(reinterpret_cast<const int2 *>(smp + (size_t)u * Ttot + t * 8));
                            smf = pack2((float)sm2.x, (float)sm2.y);
                        }
#pragma unroll
                        for (int g = 0; g < G; ++g) {
                            int d[4];
                            mma_s8_c(d, A[g][0], A[g][1], A[g][2], A[g][3], b0, b1, cmagic);
                            if (DUMP) {
                                const size_t Mz = (size_t)a.M[0];
                                const size_t row0 = (size_t)(lg + g) * 16 + r;
                                int32_t *o =
                                    a.dump + ((size_t)(cur_kt0 + u) * Ttot + tok0 + t * 8 + 2 * c) * Mz;
                                o[row0] = d[0] - kMagicBits - 8 * sm2.x;
                                o[Mz + row0] = d[1] - kMagicBits - 8 * sm2.y;
                                o[row0 + 8] = d[2] - kMagicBits - 8 * sm2.x;
                                o[Mz + row0 + 8] = d[3] - kMagicBits - 8 * sm2.y;
                            }
                            const float ws0 = uu ? ea[g].z : ea[g].x, nz0 = uu ? ea[g].w : ea[g].y;
                            const float ws1 = uu ? eb[g].z : eb[g].x, nz1 = uu ? eb[g].w : eb[g].y;
                            // (float)(d - z*asum), exact: every term is an integer below 2^24
                            const f32x2 f01 = fma2(pack2(nz0, nz0), smf,
                                                   add2(pack2i(d[0], d[1]), neg_magic2));
                            const f32x2 f23 = fma2(pack2(nz1, nz1), smf,
                                                   add2(pack2i(d[2], d[3]), neg_magic2));
                            fma2_acc(acc01[g][t], f01, mul2(pack2(ws0, ws0), as2));
                            fma2_acc(acc23[g][t], f23, mul2(pack2(ws1, ws1), as2));
                        }
                    }
                }
            };

            if (cur_nt == kCT) {
#pragma unroll
                for (int jp = 0; jp < kCT / 2; ++jp) tile_pair(std::true_type{}, jp);
            } else {
#pragma unroll
                for (int jp = 0; jp < kCT / 2; ++jp) tile_pair(std::false_type{}, jp);
            }
            __syncwarp();                  // expw is rewritten by the next chunk
            cur_nt = nx_nt;
            cur_kt0 = nx_kt0;
            advance();
          };
          if (qpar) chunk(w1, w0);
          else chunk(w0, w1);
        }
        if constexpr (!DUMP) {
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const int gg = g0 + g;
                float out[NTG][4];
#pragma unroll
                for (int t = 0; t < NTG; ++t) {
                    unpack2(acc01[g][t], out[t][0], out[t][1]);
                    unpack2(acc23[g][t], out[t][2], out[t][3]);
                }
                if (S > 1) {
                    // partial of this split -> scratch; the last split to arrive sums 0..S-1
                    float *pp = part + (((size_t)win * groups_all + gg) * S + split) * (NTG * 128) + lane;
#pragma unroll
                    for (int t = 0; t < NTG; ++t)
#pragma unroll
                        for (int k = 0; k < 4; ++k) pp[(t * 4 + k) * 32] = out[t][k];
                    __threadfence();
                    __syncwarp();
                    int old = 0;
                    if (lane == 0) old = atomicAdd(count + win * groups_all + gg, 1);
                    old = __shfl_sync(0xffffffffu, old, 0);
                    if (old != S - 1) continue;
                    __threadfence();
                    const float *base = part + ((size_t)win * groups_all + gg) * S * (NTG * 128) + lane;
#pragma unroll
                    for (int t = 0; t < NTG; ++t)
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            float sum = 0.0f;
                            for (int s = 0; s < S; ++s)
                                sum = __fadd_rn(sum, __ldcg(base + (size_t)s * (NTG * 128) +
                                                            (t * 4 + k) * 32));
                            out[t][k] = sum;
                        }
                    if (lane == 0) count[win * groups_all + gg] = 0;   // ready for the next launch
                }
                const size_t row = (size_t)(lg + g) * 16 + r;
                if (!a.npeer) {
                    float *y = a.y[wi];
#pragma unroll
                    for (int t = 0; t < NTG; ++t) {
                        const size_t tok = (size_t)tok0 + t * 8 + 2 * c;
                        y[tok * M + row] = out[t][0];
                        y[(tok + 1) * M + row] = out[t][1];
                        y[tok * M + row + 8] = out[t][2];
                        y[(tok + 1) * M + row + 8] = out[t][3];
                    }
                } else {
                    // Fused all-gather: the same slice goes into the gathered buffer of every
                    // rank. The 16 x 8 tile of a token group is transposed through the warp's
                    // scale buffer (free at this point) so that a lane holds four consecutive
                    // rows of one token and every peer gets 16-byte stores (64-byte runs).
                    float *tile = reinterpret_cast<float *>(expw);
#pragma unroll
                    for (int t = 0; t < NTG; ++t) {
                        __syncwarp();
                        tile[(2 * c) * 16 + r] = out[t][0];
                        tile[(2 * c + 1) * 16 + r] = out[t][1];
                        tile[(2 * c) * 16 + r + 8] = out[t][2];
                        tile[(2 * c + 1) * 16 + r + 8] = out[t][3];
                        __syncwarp();
                        const float4 v = *reinterpret_cast<const float4 *>(tile + lane * 4);
                        const size_t tok = (size_t)tok0 + t * 8 + (lane >> 2);
                        const size_t off = tok * M + (size_t)(lg + g) * 16 + (lane & 3) * 4;
                        for (int pi = 0; pi < a.npeer; ++pi)
                            *reinterpret_cast<float4 *>(a.ypeer[pi][wi] + off) = v;
                    }
                    __syncwarp();
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Ring kernel for T = 8, and for T = 16..64 as token windows of 8 on separate CTA columns
// (grid.y; the packed weights are then read once per window, from L2 after the first) when a
// window's activations fit beside the rings: 32 warps per SM at 64 registers. The register queue above leaves
// 16 warps per SM, each of which spends most of its time waiting on its own dependency
// chains; here every warp streams its tiles through a private two-stage shared-memory ring
// filled with cp.async (16 bytes per lane, eight tiles and their scale lines per stage) and
// reads MMA A fragments back with ldmatrix, so the registers hold only one tile pair and
// twice as many warps share an SM. Scale words are read raw from the stage (one 32-byte line
// per tile) and unpacked by the lanes that use them. Task mapping, staged activations, split
// reduction, stores and the fused all-gather are those of the kernel above.
constexpr int kRW = 32;                              // most warps per CTA (a launch may use fewer)
constexpr int kRST = 8;                              // tiles per ring stage (4 and 6 measured slower)
constexpr int kRStage = kRST * 256 + kRST * 32;      // codes, then one scale line per tile
constexpr int kRHead = 64;                           // small per-CTA header in front of the rings

__device__ __forceinline__ uint2 lds_v2(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ ulonglong2 lds_v2u64(uint32_t addr) {
    ulonglong2 v;
    asm volatile("ld.shared.v2.u64 {%0,%1}, [%2];" : "=l"(v.x), "=l"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}

// Packed scale word -> fp32 scale and (float)(z + 8): the 4-bit two's-complement zero point
// with its top bit flipped is z + 8 in [0, 15].
__device__ __forceinline__ void scale_pair(uint32_t packed, float &ws, float &z8) {
    ws = __half2float(__ushort_as_half((unsigned short)(packed & 0xFFF0u)));
    z8 = (float)(int)((packed ^ 8u) & 15u);
}

// PAIR: K64 tier and even split starts - tiles 2j, 2j+1 share a scale line. kRNS: ring stages
// per warp (2 with all 32 warps; more when the call has fewer tasks than warp slots).
// MAXW: most warps the instantiation is launched with (fewer warps leave it more registers).
// PT: per-token activation scales (a.as_tok): one promote per weight-scale group -
// acc = fma((float)(d - z*asum), ws, acc) with d the int32 dot of the whole group (both k-tiles
// of a K64 group chained through the MMA's accumulator input) - splits cut whole groups, and
// the per-token scale multiplies the sum of the splits at the end.
#ifdef TQ_RING_TRACE
__device__ unsigned long long g_ring_trace[1024 * 8];
#define RING_STAMP(i) if (threadIdx.x == 0 && blockIdx.x < 1024) g_ring_trace[blockIdx.x * 8 + (i)] = global_timer_ns();
#define RING_STAMP_END() if (lane == 0 && blockIdx.x < 1024) atomicMax(&g_ring_trace[blockIdx.x * 8 + 5], global_timer_ns());
#else
#define RING_STAMP(i)
#define RING_STAMP_END()
#endif
// NTG: 8-token groups a warp carries per tile (1, 2, 4 or 8): the tile's A fragments, scale
// words and ring traffic are paid once for all of them; the staged activations of group g
// follow those of group g - 1 (`gstride` bytes apart).
template <bool PAIR, int kRNS, int MAXW, bool PT, int NTG = 1>
__global__ void __launch_bounds__(MAXW * 32, 1)
gemm_w4a8_ring_kernel(const GemmArgs a, float *__restrict__ part, int *__restrict__ count) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int r = lane >> 2;
    const int c = lane & 3;
    const int S = a.max_splits;
    const int split = blockIdx.x % S;
    const int cta_i = blockIdx.x / S;
    const int nctas = (gridDim.x - split + S - 1) / S;

    const int groups_all = a.goff[a.count];
    const int tgid = cta_i + nctas * warp;
    const int nw = blockDim.x >> 5;
    const int tstride = nctas * nw;
    const int Kt = a.K >> 5;
    const int ksh = a.ksh;
    const int Ktg = Kt >> ksh;
    const int kt_begin = PT ? ((Ktg * split / S) << ksh) : Kt * split / S;
    const int cnt = (PT ? ((Ktg * (split + 1) / S) << ksh) : Kt * (split + 1) / S) - kt_begin;
    // token window of this CTA column: tokens [tok0, tok0 + 8 NTG) of the call's Ttot
    const int win = blockIdx.y, tok0 = win * 8 * NTG, Ttot = a.T;

    // 64 bytes in front of the rings: the row maxima of the fused per-token quantiser
    int *s_rowmax = reinterpret_cast<int *>(smem);
    unsigned char *ring = smem + kRHead + (size_t)warp * kRNS * kRStage;
    const uint32_t ring_s = smem_u32(ring);
    unsigned char *act = smem + kRHead + (size_t)nw * kRNS * kRStage;
    const uint32_t act_s = smem_u32(act);
    const uint32_t gstride = (uint32_t)cnt * kActTileBytes;          // one token group's staged bytes
    float *xpose = reinterpret_cast<float *>(act + (size_t)NTG * gstride) + warp * 128;
    const uint64_t pol = l2_policy_evict_first();

    // ---- producer: next (row-group, tile offset) to fetch --------------------------------
    int pg = tgid, pi0 = 0;
    uint32_t pdst = ring_s;
    const uint8_t *psrc = nullptr;
    const uint16_t *pscl = nullptr;
    auto producer_group = [&]() {
        if (pg < groups_all) {
            int wi = 0;
            while (wi + 1 < a.count && pg >= a.goff[wi + 1]) ++wi;
            const int lg = pg - a.goff[wi];
            psrc = a.codes[wi] + ((size_t)lg * Kt + kt_begin) * 256u + lane * 16;
            pscl = a.scales[wi] + (size_t)lg * Ktg * 16u + (lane & 1) * 8;
        }
    };
    producer_group();
    auto issue_next = [&]() {
        if (pg < groups_all && cnt > 0) {
            const int left = cnt - pi0;
            const uint16_t *sl = pscl + (size_t)((kt_begin + pi0 + (lane >> 1)) >> ksh) * 16u;
            if (left >= kRST) {
#pragma unroll
                for (int p = 0; p < kRST / 2; ++p)
                    cp_async16(pdst + lane * 16 + p * 512, psrc + p * 512, pol);
                if (lane < 2 * kRST) cp_async16(pdst + kRST * 256 + lane * 16, sl, pol);
            } else {
#pragma unroll
                for (int p = 0; p < kRST / 2; ++p)
                    if (lane + 32 * p < left * 16)
                        cp_async16(pdst + lane * 16 + p * 512, psrc + p * 512, pol);
                if (lane < 2 * left) cp_async16(pdst + kRST * 256 + lane * 16, sl, pol);
            }
            pi0 += kRST;
            psrc += kRST * 256;
            if (pi0 >= cnt) {
                pi0 = 0;
                pg += tstride;
                producer_group();
            }
            pdst = (pdst + kRStage == ring_s + kRNS * kRStage) ? ring_s : pdst + kRStage;
        }
        cp_async_commit();
    };

    RING_STAMP(0)
    pdl_trigger();
#pragma unroll
    for (int i = 0; i < kRNS - 1; ++i) issue_next();
    RING_STAMP(1)
    // Everything above reads only packed weights; what follows depends on earlier kernels.
    pdl_wait();
    RING_STAMP(2)

    // Stage this split's activations (layout of the register-queue kernel for T = 8, but the
    // code sums are stored negated: the tile loop multiplies them by z + 8 >= 0).
    if (a.x) {
        // Fused quantiser: the fp32 rows are quantised here with the rule and the arithmetic
        // of quant_chunk_kernel (per (token, K32) block, or with the row's absmax / 127 in
        // per-token mode), straight into the staged layout. A warp takes one (k-tile, token)
        // block at a time, lane = k.
        const int K = a.K;
        if (a.x_mode == 2) {
            if (threadIdx.x < 8) s_rowmax[threadIdx.x] = __float_as_int(-INFINITY);
            __syncthreads();
            float m[8];
#pragma unroll
            for (int t = 0; t < 8; ++t) m[t] = -INFINITY;
            for (int i = threadIdx.x; i < (K >> 2); i += nw * 32) {
#pragma unroll
                for (int t = 0; t < 8; ++t) {
                    const float4 v = __ldg(reinterpret_cast<const float4 *>(a.x + (size_t)(tok0 + t) * K) + i);
                    m[t] = fmaxf(m[t], fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
                }
            }
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                const float wm = warp_max(m[t]);
                // non-negative floats (and -inf) order like their bit patterns as signed ints
                if (lane == 0) atomicMax(&s_rowmax[t], __float_as_int(wm));
            }
            __syncthreads();
        }
        // kQU blocks per pass, their loads issued together (one load per block and lane)
        constexpr int kQU = 8;
        for (int b0 = warp; b0 < cnt * 8; b0 += nw * kQU) {
            float vv[kQU];
#pragma unroll
            for (int u = 0; u < kQU; ++u) {
                const int b = b0 + u * nw;
                vv[u] = 0.0f;
                if (b < cnt * 8)
                    vv[u] = __ldg(a.x + (size_t)(tok0 + (b & 7)) * K + (size_t)(kt_begin + (b >> 3)) * 32 + lane);
            }
#pragma unroll
            for (int u = 0; u < kQU; ++u) {
                const int b = b0 + u * nw;
                if (b >= cnt * 8) break;
                const int kl = b >> 3, t = b & 7;
                const float v = vv[u];
                float s;
                if (a.x_mode == 2) {
                    const float mx = __int_as_float(s_rowmax[t]);
                    s = (mx > 0.0f) ? __fdiv_rn(mx, 127.0f) : 1.0f;
                } else {
                    const float mx = warp_max(fmaxf(-INFINITY, fabsf(v)));
                    s = (mx > 0.0f) ? __fdiv_rn(mx, 127.0f) : 1.0f;
                }
                const int qv = quantise_one(v, s);
                int sum = half_sum16(qv);
                sum += __shfl_xor_sync(0xffffffffu, sum, 16);
                // B-fragment order: token t, chunk c = k / 8: the chunk's even-k bytes, then its odd-k
                const int c8 = lane >> 3, j = lane & 7;
                act[(size_t)kl * kActTileBytes + (t * 4 + c8) * 8 + ((j & 1) * 4 + (j >> 1))] =
                    (unsigned char)(int8_t)qv;
                if (lane == 0) {
                    float *pv = reinterpret_cast<float *>(act + (size_t)kl * kActTileBytes + 256 + (t >> 1) * 16);
                    pv[t & 1] = s;
                    pv[2 + (t & 1)] = -(float)sum;
                }
            }
        }
        __syncthreads();
    } else {
        // All of a thread's loads of a pass are issued before its first store: the staging is a
        // chain of L2 latencies, and a loop of load-then-store pays one per iteration.
        const int items = cnt * 32, nthr = nw * 32;
        constexpr int kSU = 4;
#pragma unroll 1
        for (int g = 0; g < NTG; ++g) {
            unsigned char *actg = act + (size_t)g * gstride;
            const int tokg = tok0 + 8 * g;
            for (int i0 = threadIdx.x; i0 < items; i0 += nthr * kSU) {
                uint2 bb[kSU];
#pragma unroll
                for (int u = 0; u < kSU; ++u) {
                    const int i = i0 + u * nthr;
                    if (i < items)
                        bb[u] = __ldg(reinterpret_cast<const uint2 *>(
                            a.aq + ((size_t)(kt_begin + (i >> 5)) * Ttot + tokg) * 32 + (size_t)(i & 31) * 8));
                }
#pragma unroll
                for (int u = 0; u < kSU; ++u) {
                    const int i = i0 + u * nthr;
                    if (i < items) {
                        uint2 o;
                        o.x = __byte_perm(bb[u].x, bb[u].y, 0x6420);
                        o.y = __byte_perm(bb[u].x, bb[u].y, 0x7531);
                        *reinterpret_cast<uint2 *>(actg + (size_t)(i >> 5) * kActTileBytes + (i & 31) * 8) = o;
                    }
                }
            }
            const int pairs = cnt * 4;
            for (int i = threadIdx.x; i < pairs; i += nthr) {
                const int kl = i >> 2;
                const int rem = i & 3;
                const size_t src = (size_t)(kt_begin + kl) * Ttot + tokg + (size_t)rem * 2;
                float2 as2 = make_float2(0.f, 0.f);
                if (!PT) as2 = __ldg(reinterpret_cast<const float2 *>(a.as + src));
                int2 sm2 = __ldg(reinterpret_cast<const int2 *>(a.asum + src));
                if (PT && PAIR && !(kl & 1) && kl + 1 < cnt) {      // the K64 group's sum, with its first tile
                    const int2 nx = __ldg(reinterpret_cast<const int2 *>(a.asum + src + Ttot));
                    sm2.x += nx.x;
                    sm2.y += nx.y;
                }
                *reinterpret_cast<float4 *>(actg + (size_t)kl * kActTileBytes + 256 + rem * 16) =
                    make_float4(as2.x, as2.y, -(float)sm2.x, -(float)sm2.y);
            }
        }
        __syncthreads();
    }

    RING_STAMP(3)
    const f32x2 neg_magic2 = pack2(-kMagicF, -kMagicF);
    int cmagic[4];
    make_const_quad(cmagic, kMagicBits);
    uint32_t cst = ring_s;
    const uint32_t lane_a = (lane >> 4) * 256 + (lane & 15) * 16;   // ldmatrix row address
    const uint32_t lane_s = kRST * 256 + r * 2;                     // scale word of row r
    const uint32_t lane_b = act_s + lane * 8;
    const uint32_t lane_v = act_s + 256 + c * 16;

    f32x2 acc01[NTG], acc23[NTG];
    // one tile: A words of rows r, r+8; {ws, z+8} of those rows; activations at bb / vb (+ g * gstride)
    auto tile = [&](uint32_t w_lo, uint32_t w_hi, float ws0, float nz0, float ws1, float nz1,
                    uint32_t bb_addr, uint32_t vb_addr) {
        const uint32_t A0 = nib_plus8(w_lo), A1 = nib_plus8(w_hi);
        const uint32_t A2 = nib_plus8(w_lo >> 4), A3 = nib_plus8(w_hi >> 4);
        const f32x2 nz0p = pack2(nz0, nz0), nz1p = pack2(nz1, nz1), ws0p = pack2(ws0, ws0), ws1p = pack2(ws1, ws1);
#pragma unroll
        for (int g = 0; g < NTG; ++g) {
            const uint2 bb = lds_v2(bb_addr + g * gstride);
            const ulonglong2 av = lds_v2u64(vb_addr + g * gstride);
            int d[4];
            mma_s8_c(d, A0, A1, A2, A3, bb.x, bb.y, cmagic);
            // (float)(d - z*asum) = (z+8) * (-asum) + d', exact: all integers below 2^24
            const f32x2 f01 = fma2(nz0p, av.y, add2(pack2i(d[0], d[1]), neg_magic2));
            const f32x2 f23 = fma2(nz1p, av.y, add2(pack2i(d[2], d[3]), neg_magic2));
            if (PT) {
                fma2_acc(acc01[g], f01, ws0p);
                fma2_acc(acc23[g], f23, ws1p);
            } else {
                fma2_acc(acc01[g], f01, mul2(ws0p, av.x));
                fma2_acc(acc23[g], f23, mul2(ws1p, av.x));
            }
        }
    };
    // both tiles of a K64 group against per-token scales: one int32 dot, one promote
    auto tile_group = [&](uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, float ws0, float nz0, float ws1,
                          float nz1, uint32_t bb_addr, uint32_t vb_addr, bool second) {
        const uint32_t A0 = nib_plus8(w0), A1 = nib_plus8(w1), A2 = nib_plus8(w0 >> 4), A3 = nib_plus8(w1 >> 4);
        const uint32_t B0 = nib_plus8(w2), B1 = nib_plus8(w3), B2 = nib_plus8(w2 >> 4), B3 = nib_plus8(w3 >> 4);
        const f32x2 nz0p = pack2(nz0, nz0), nz1p = pack2(nz1, nz1), ws0p = pack2(ws0, ws0), ws1p = pack2(ws1, ws1);
#pragma unroll
        for (int g = 0; g < NTG; ++g) {
            const uint2 bb = lds_v2(bb_addr + g * gstride);
            const ulonglong2 av = lds_v2u64(vb_addr + g * gstride);
            int d[4];
            mma_s8_c(d, A0, A1, A2, A3, bb.x, bb.y, cmagic);
            if (second) {
                const uint2 bb2 = lds_v2(bb_addr + g * gstride + kActTileBytes);
                mma_s8_acc(d, B0, B1, B2, B3, bb2.x, bb2.y);
            }
            const f32x2 f01 = fma2(nz0p, av.y, add2(pack2i(d[0], d[1]), neg_magic2));
            const f32x2 f23 = fma2(nz1p, av.y, add2(pack2i(d[2], d[3]), neg_magic2));
            fma2_acc(acc01[g], f01, ws0p);
            fma2_acc(acc23[g], f23, ws1p);
        }
    };
    // tiles 2j, 2j+1 of the stage at `cst`; activations of the first one at offset kl_off
    auto tile_pair = [&](uint32_t ab, uint32_t sb, uint32_t bbase, uint32_t vbase, bool second) {
        uint32_t w0, w1, w2, w3;
        ldmatrix_x4(ab, w0, w1, w2, w3);
        float ws0, ws1, nz0, nz1;
        scale_pair(lds_u16(sb), ws0, nz0);
        scale_pair(lds_u16(sb + 16), ws1, nz1);
        if (PT && PAIR) {
            tile_group(w0, w1, w2, w3, ws0, nz0, ws1, nz1, bbase, vbase, second);
            return;
        }
        tile(w0, w1, ws0, nz0, ws1, nz1, bbase, vbase);
        if (second) {
            if (!PAIR) {
                scale_pair(lds_u16(sb + 32), ws0, nz0);
                scale_pair(lds_u16(sb + 48), ws1, nz1);
            }
            tile(w2, w3, ws0, nz0, ws1, nz1, bbase + kActTileBytes, vbase + kActTileBytes);
        }
    };

    for (int g0 = tgid; g0 < groups_all; g0 += tstride) {
        int wi = 0;
        while (wi + 1 < a.count && g0 >= a.goff[wi + 1]) ++wi;
        const int lg = g0 - a.goff[wi];
        const int M = a.M[wi];
#pragma unroll
        for (int g = 0; g < NTG; ++g) acc01[g] = acc23[g] = 0ull;
        uint32_t bbase = lane_b, vbase = lane_v;
        for (int left = cnt; left > 0; left -= kRST) {
            cp_async_wait<kRNS - 2>();
            __syncwarp();                 // the stage is complete; the other slot is free
            issue_next();
            const uint32_t ab = cst + lane_a, sb = cst + lane_s;
            if (left >= kRST) {
#pragma unroll
                for (int j = 0; j < kRST / 2; ++j)
                    tile_pair(ab + j * 512, sb + j * 64, bbase + j * 2 * kActTileBytes,
                              vbase + j * 2 * kActTileBytes, true);
            } else {
                // last, short stage of the split: a plain loop, only its last pair can be half
                const int np = (left + 1) >> 1;
#pragma unroll 1
                for (int j = 0; j < np; ++j)
                    tile_pair(ab + j * 512, sb + j * 64, bbase + j * 2 * kActTileBytes,
                              vbase + j * 2 * kActTileBytes, 2 * j + 1 < left);
            }
            bbase += kRST * kActTileBytes;
            vbase += kRST * kActTileBytes;
            cst = (cst + kRStage == ring_s + kRNS * kRStage) ? ring_s : cst + kRStage;
        }
        const size_t row = (size_t)lg * 16 + r;
        const size_t ldy = a.ld[wi] ? (size_t)a.ld[wi] : (size_t)M;      // row stride of y
        bool last_split = true;
        const size_t slot = (size_t)win * groups_all + g0;              // (window, row-group)
        if (S > 1) {
            // partials of this split -> scratch; the last split to arrive sums 0..S-1
            float *pp = part + (slot * S + split) * (128 * NTG) + lane;
#pragma unroll
            for (int g = 0; g < NTG; ++g) {
                float o[4];
                unpack2(acc01[g], o[0], o[1]);
                unpack2(acc23[g], o[2], o[3]);
#pragma unroll
                for (int k = 0; k < 4; ++k) pp[g * 128 + k * 32] = o[k];
            }
            __threadfence();
            __syncwarp();
            int old = 0;
            if (lane == 0) old = atomicAdd(count + slot, 1);
            old = __shfl_sync(0xffffffffu, old, 0);
            last_split = old == S - 1;
            if (!last_split) continue;
            __threadfence();
        }
#pragma unroll
        for (int g = 0; g < NTG; ++g) {
            float out[4];
            unpack2(acc01[g], out[0], out[1]);
            unpack2(acc23[g], out[2], out[3]);
            if (S > 1) {
                // all of a group's partials are requested before the first add (the adds keep
                // the order 0..S-1): a loop of load-then-add pays an L2 latency per split
                const float *base = part + slot * S * (128 * NTG) + g * 128 + lane;
                float v[4][16];
#pragma unroll
                for (int s2 = 0; s2 < 16; ++s2)
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        v[k][s2] = s2 < S ? __ldcg(base + (size_t)s2 * (128 * NTG) + k * 32) : 0.0f;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    float sum = 0.0f;
#pragma unroll
                    for (int s2 = 0; s2 < 16; ++s2)
                        if (s2 < S) sum = __fadd_rn(sum, v[k][s2]);
                    out[k] = sum;
                }
            }
            const int tokg = tok0 + 8 * g;
            if (PT) {
                const float2 at = __ldg(reinterpret_cast<const float2 *>(a.as_tok + tokg + 2 * c));
                out[0] = __fmul_rn(out[0], at.x);
                out[1] = __fmul_rn(out[1], at.y);
                out[2] = __fmul_rn(out[2], at.x);
                out[3] = __fmul_rn(out[3], at.y);
            }
            if (!a.npeer) {
                float *y = a.y[wi];
                const size_t tok = (size_t)tokg + 2 * c;
                y[tok * ldy + row] = out[0];
                y[(tok + 1) * ldy + row] = out[1];
                y[tok * ldy + row + 8] = out[2];
                y[(tok + 1) * ldy + row + 8] = out[3];
            } else {
                // Fused all-gather: transpose the 16 x 8 tile so that a lane holds four consecutive
                // rows of one token and every peer gets 16-byte stores (64-byte runs).
                __syncwarp();
                xpose[(2 * c) * 16 + r] = out[0];
                xpose[(2 * c + 1) * 16 + r] = out[1];
                xpose[(2 * c) * 16 + r + 8] = out[2];
                xpose[(2 * c + 1) * 16 + r + 8] = out[3];
                __syncwarp();
                const float4 v = *reinterpret_cast<const float4 *>(xpose + lane * 4);
                const size_t off = (size_t)(tokg + (lane >> 2)) * ldy + (size_t)lg * 16 + (lane & 3) * 4;
                for (int pi = 0; pi < a.npeer; ++pi)
                    *reinterpret_cast<float4 *>(a.ypeer[pi][wi] + off) = v;
            }
        }
        if (S > 1 && lane == 0) count[slot] = 0;   // ready for the next launch
    }
    RING_STAMP(4)
    RING_STAMP_END()
}

int g_num_sms = 0;
constexpr size_t kSmemLimit = 227 * 1024;

// Library scratch of the split reduction: partial tiles and one arrival counter per
// row-group (the counterpart of the reference's g_split_partial, kernels_dpas.cpp:150-181).
// Calls are ordered on one stream, so one buffer serves every launch. Counters are zeroed
// when allocated and are left at zero by every launch.
struct StreamScratch {
    float *part = nullptr;
    int *count = nullptr;
    size_t part_floats = 0;
    int count_n = 0;
} g_scratch;

void ensure_scratch(size_t part_floats, int count_n) {
    StreamScratch &s = g_scratch;
    if (part_floats > s.part_floats) {
        if (s.part) tq_dev_free(s.part);
        s.part = static_cast<float *>(tq_dev_alloc(part_floats * sizeof(float), "gemm.split.partial"));
        s.part_floats = part_floats;
    }
    if (count_n > s.count_n) {
        if (s.count) tq_dev_free(s.count);
        s.count = static_cast<int *>(tq_dev_alloc((size_t)count_n * sizeof(int), "gemm.split.count"));
        TQ_CHECK(cudaMemsetAsync(s.count, 0, (size_t)count_n * sizeof(int), stream()));
        s.count_n = count_n;
    }
}

template <int NTG, bool STAGED, bool DUMP, int kW>
void launch_variant(const GemmArgs &a, size_t smem) {
    static bool attr_set = false;
    if (!attr_set) {
        TQ_CHECK(cudaFuncSetAttribute(gemm_w4a8_stream_kernel<NTG, STAGED, DUMP, kW>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)kSmemLimit));
        attr_set = true;
    }
    const int S = a.max_splits;
    const int groups = a.goff[a.count];
    const int nwin = a.T / (NTG * 8);            // token windows (grid.y), one per CTA column
    if (S > 1 && !DUMP)
        ensure_scratch((size_t)nwin * groups * S * NTG * 128, nwin * groups);
    const int want = ((groups + kW - 1) / kW) * S;
    const int grid = std::max(S, std::min(std::max(1, g_num_sms / nwin), want));
    launch_pdl(gemm_w4a8_stream_kernel<NTG, STAGED, DUMP, kW>, dim3(grid, nwin), dim3(kW * 32),
               smem, a, g_scratch.part, g_scratch.count);
    TQ_LAUNCH_CHECK("gemm_w4a8_stream_kernel");
}

template <int NTG>
void launch_ntg(const GemmArgs &a) {
    if (!g_num_sms) {
        int dev = 0;
        TQ_CHECK(cudaGetDevice(&dev));
        TQ_CHECK(cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev));
        if (g_num_sms <= 0) g_num_sms = 148;
    }
    if (a.dump) {
        launch_variant<NTG, false, true, 16>(a, (size_t)16 * kExpBytes);
        return;
    }
    if constexpr (NTG <= 4) {
        // stage this split's activations in shared memory when they fit
        const int Kt = a.K >> 5, S = a.max_splits;
        const size_t act = (size_t)((Kt + S - 1) / S) * NTG * kActTileBytes;
        if ((size_t)kWmax * kExpBytes + act <= kSmemLimit) {
            if constexpr (NTG <= 2) {
                // 24 warps per CTA (fewer registers each) when that saves a whole pass over
                // the row-groups: every (row-group, split) is one indivisible warp task
                const int groups = a.goff[a.count];
                const int ctas = std::max(1, g_num_sms / S);
                const int rounds16 = (groups + ctas * 16 - 1) / (ctas * 16);
                const int rounds24 = (groups + ctas * 24 - 1) / (ctas * 24);
                if (rounds24 < rounds16 && rounds16 <= 3) {
                    launch_variant<NTG, true, false, 24>(a, (size_t)24 * kExpBytes + act);
                    return;
                }
            }
            launch_variant<NTG, true, false, 16>(a, (size_t)16 * kExpBytes + act);
            return;
        }
    }
    launch_variant<NTG, false, false, 16>(a, (size_t)16 * kExpBytes);
}

}  // namespace

bool gemm_stream_covers(const GemmArgs &a) {
    if (a.npeer < 0 || a.npeer > 8) return false;
    for (int i = 0; i < a.count; ++i)
        if (a.ld[i] && a.ld[i] != a.M[i] && a.T != 8) return false;   // only the ring kernel strides y
    if (a.count < 1 || a.T < 8 || a.T > 64 || (a.T % 8)) return false;
    if (a.max_splits > 16) return false;
    if (a.ksh && ((a.K >> 5) & 1)) return false;
    if (a.dump && a.count != 1) return false;
    for (int i = 0; i < a.count; ++i)
        if (a.seg[i].count != 1 || a.seg[i].split[0] != a.max_splits) return false;
    return true;
}

// Tokens per CTA window. Up to 16 tokens a warp carries all of them (weights are fetched
// once). Above that the reference's split rule leaves few (row-group, split) tasks, so the
// tokens are cut into windows handled by different CTAs (grid.y): 16 tokens per window when
// the window's activations of one split fit in shared memory, else 8 if those fit, else 16
// read through L1. A call that feeds the fused all-gather keeps one window.
int window_groups(const GemmArgs &a) {
    const int ntg = a.T / 8;
    if (ntg <= 2 || a.dump || a.npeer) return ntg;
    const int Kt = a.K >> 5, S = a.max_splits;
    const size_t per_tg = (size_t)((Kt + S - 1) / S) * kActTileBytes;
    const size_t room = kSmemLimit - (size_t)kWmax * kExpBytes;
    if (ntg % 2 == 0 && 2 * per_tg <= room) return 2;
    if (per_tg <= room) return 1;
    return (ntg % 2 == 0) ? 2 : 1;
}

// The ring kernel takes T = 8 calls whose split activations fit beside the rings.
// Launch shape of the ring kernel for a call, or false when the call is not its to take.
struct RingPlan {
    int grid, nw, ns, nwin, ntg;
    size_t smem;
};
// Plan with `ntg` token groups per warp (token windows of 8 ntg tokens on CTA columns).
bool ring_plan_ntg(const GemmArgs &a, int ntg, RingPlan &p) {
    p.ntg = ntg;
    p.nwin = a.T / (8 * ntg);                 // token windows: CTA columns (grid.y)
    const int Kt = a.K >> 5, S = a.max_splits;
    const int groups = a.goff[a.count];
    const int ctas = g_num_sms / p.nwin;      // CTAs of one window
    if (S > ctas || groups <= 0) return false;
    const long most = (long)groups * S;
    p.grid = (int)std::max<long>(S, std::min<long>(ctas - ctas % S, most));
    // One task per warp when the call has fewer tasks than warp slots: fewer warps, and the
    // shared memory they leave goes into deeper rings (each warp's chain is then longer
    // than the memory latency its ring covers with two stages).
    const int per_cta = (groups + p.grid / S - 1) / (p.grid / S);      // tasks of the busiest CTA
    p.nw = kRW;
    if (per_cta < kRW) p.nw = std::max(8, (per_cta + 1) / 2 * 2);
    // k-tiles of the longest split (per-token splits cut whole weight-scale groups)
    const int Ktg = Kt >> a.ksh;
    const int span = a.mode ? (((Ktg + S - 1) / S) << a.ksh) : (Kt + S - 1) / S;
    const size_t fixed = kRHead + (size_t)span * ntg * kActTileBytes + (a.npeer ? (size_t)p.nw * 512 : 0);
    if (ntg > 1) {
        // several token groups per warp: one instantiation, at most 20 warps (more registers
        // for the accumulators), three ring stages
        p.nw = std::min(p.nw, 20);
        p.ns = 3;
    } else {
        p.ns = 4;
        while (p.ns > 2 && (size_t)p.nw * p.ns * kRStage + fixed > kSmemLimit) --p.ns;
    }
    p.smem = (size_t)p.nw * p.ns * kRStage + fixed;
    return p.smem <= kSmemLimit;
}
// The widest plan that fits: all of a call's tokens on one warp (weights and their unpacking
// paid once), else windows of 32, 16 or 8 tokens on CTA columns.
bool ring_plan(const GemmArgs &a, RingPlan &p) {
    if (a.T < 8 || a.T > 64 || (a.T % 8) || a.dump) return false;
    if (a.x && (a.T != 8 || a.mode)) return false;   // the fused quantiser serves one window
    if (!g_num_sms) {
        int dev = 0;
        TQ_CHECK(cudaGetDevice(&dev));
        TQ_CHECK(cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev));
        if (g_num_sms <= 0) g_num_sms = 148;
    }
    const int tg = a.T / 8;
    for (int ntg = 8; ntg >= 1; ntg >>= 1)
        if (tg % ntg == 0 && (ntg == 1 || !a.npeer) && ring_plan_ntg(a, ntg, p)) return true;
    return false;
}

bool launch_ring(const GemmArgs &a) {
    RingPlan plan;
    if (!ring_plan(a, plan)) return false;
    const int Kt = a.K >> 5, S = a.max_splits;
    const int groups = a.goff[a.count];
    const int grid = plan.grid, nw = plan.nw, ns = plan.ns;
    const size_t smem = plan.smem;
    bool pair = a.ksh != 0;
    if (!a.mode)      // per-token splits cut whole K64 groups, so they always start on a pair
        for (int s2 = 0; s2 < S; ++s2) pair = pair && ((Kt * s2 / S) % 2 == 0);
    if (S > 1) ensure_scratch((size_t)plan.nwin * groups * S * 128 * plan.ntg, plan.nwin * groups);
    auto go = [&](auto kernel) {
        // every instantiation has the same function type, so remember them by address
        static const void *done[64];
        static int ndone = 0;
        bool seen = false;
        for (int i = 0; i < ndone; ++i) seen = seen || done[i] == (const void *)kernel;
        if (!seen) {
            TQ_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)kSmemLimit));
            if (ndone < 64) done[ndone++] = (const void *)kernel;
        }
        launch_pdl(kernel, dim3(grid, plan.nwin), dim3(nw * 32), smem, a, g_scratch.part, g_scratch.count);
    };
    auto pick = [&](auto pair_tag, auto pt_tag) {
        constexpr bool P = decltype(pair_tag)::value, Q = decltype(pt_tag)::value;
        if (plan.ntg == 8) go(gemm_w4a8_ring_kernel<P, 3, 20, Q, 8>);
        else if (plan.ntg == 4) go(gemm_w4a8_ring_kernel<P, 3, 20, Q, 4>);
        else if (plan.ntg == 2) go(gemm_w4a8_ring_kernel<P, 3, 20, Q, 2>);
        else if (ns == 2) go(gemm_w4a8_ring_kernel<P, 2, kRW, Q>);
        else if (ns == 3) go(gemm_w4a8_ring_kernel<P, 3, kRW, Q>);
        else if (nw <= 20) go(gemm_w4a8_ring_kernel<P, 4, 20, Q>);
        else go(gemm_w4a8_ring_kernel<P, 4, kRW, Q>);
    };
    if (a.mode) {
        if (pair) pick(std::true_type{}, std::true_type{});
        else pick(std::false_type{}, std::true_type{});
    } else {
        if (pair) pick(std::true_type{}, std::false_type{});
        else pick(std::false_type{}, std::false_type{});
    }
    TQ_LAUNCH_CHECK("gemm_w4a8_ring_kernel");
    return true;
}

bool gemm_ring_covers(const GemmArgs &a) {
    RingPlan plan;
    return gemm_stream_covers(a) && ring_plan(a, plan);
}

void launch_gemm_stream(const GemmArgs &a) {
    if (launch_ring(a)) return;
    for (int i = 0; i < a.count; ++i)
        if (a.ld[i] && a.ld[i] != a.M[i]) {      // only the ring kernel strides its output rows
            note_error(cudaErrorInvalidValue, "launch_gemm_stream: strided output outside the ring kernel");
            return;
        }
    switch (window_groups(a)) {
        case 1: launch_ntg<1>(a); break;
        case 2: launch_ntg<2>(a); break;
        case 3: launch_ntg<3>(a); break;
        case 4: launch_ntg<4>(a); break;
        case 5: launch_ntg<5>(a); break;
        case 6: launch_ntg<6>(a); break;
        case 7: launch_ntg<7>(a); break;
        default: launch_ntg<8>(a); break;
    }
}

}  // namespace tq

#ifdef TQ_RING_TRACE
extern "C" int qwn_dbg_ring_trace(unsigned long long *out, int clear) {
    if (clear) {
        static unsigned long long z[1024 * 8];
        return (int)cudaMemcpyToSymbol(tq::g_ring_trace, z, sizeof(z));
    }
    return (int)cudaMemcpyFromSymbol(out, tq::g_ring_trace, 1024 * 8 * 8);
}
#endif
