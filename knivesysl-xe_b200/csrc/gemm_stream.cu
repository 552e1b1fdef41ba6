// gemm_stream.cu — batched W4A8 GEMM for decode batches (T = 8..64 tokens, one segment)
// on sm_100a: a persistent kernel in which every warp streams packed weights through its
// own asynchronous-copy ring.
//
// Replaces x_gemm_w4a8's split path (xpu/src/kernels_dpas.cpp:1379-1489) for the shapes
// decode uses. The kernel is HBM-bound on the packed weight stream, so the design is about
// bytes in flight per SM and about issue slots per 256-byte tile:
//  * one CTA per SM, 16 warps. All warps of a CTA work on the SAME K-split s (CTA b takes
//    s = b % S), each warp on its own 16-row groups; a row-group's K run is contiguous in
//    the packed layout, so a warp streams its span with 16-byte cp.async copies (L1
//    bypassed, evict-first in L2) into a private ring of stages (8 tiles + their scale
//    lines per stage) tracked with commit / wait groups: nothing spins. The ring keeps
//    running across the row-groups a warp owns, so the pipeline never drains;
//  * because a CTA only needs the activations of one K-split, they are staged ONCE per CTA
//    in shared memory in the form the tile loop consumes: the int8 codes already in MMA
//    B-fragment order, and per (k-tile, token pair) the packed pair {as0, as1} and the
//    code sums as fp32 {asum0, asum1} (STAGED = true). Shapes whose activations do not fit
//    read them through L1 instead (STAGED = false);
//  * one ldmatrix.x4 turns two 256-byte tiles into the A fragments of two
//    mma.sync.m16n8k32.s8 (weights = 16 rows, tokens = 8 columns); nibbles are used as q+8
//    (xor 8) and the correction folds into the zero-point term: d - z*asum == d' -
//    (z+8)*asum;
//  * the MMA accumulator starts at the bit pattern of 12582912.0f, so the exact int32
//    result becomes fp32 with one add instead of a conversion; (float)(d - z*asum) is then
//    formed exactly in fp32 (all terms are integers below 2^24) and the promote term
//    (float)(d - z*asum) * (ws*as) is accumulated with fma in ascending k-tile order, all
//    on packed f32x2 instructions (two outputs per issue slot);
//  * K-splits of one row-group live in different CTAs. Each writes its partial tile to a
//    small global scratch, and the warp that arrives last (a counter per row-group) adds
//    the S partials in the order 0..S-1 starting from 0.0f and stores y: the reference's
//    summation order, independent of arrival order. An unsplit weight stores its
//    accumulator untouched.
#include "stream.cuh"

#include <algorithm>

namespace tq {

namespace {

constexpr int kST = 8;                          // k-tiles per ring stage
constexpr int kStageBytes = kST * 256 + 256;    // codes + up to 8 scale lines
constexpr int kW = 16;                          // warps per CTA
constexpr int kExpBytes = kST * 16 * 8;         // expanded scales of one stage, per warp
constexpr int kActTileBytes = 256 + 64;         // staged activations per (k-tile, 8 tokens)

template <int NTG, bool STAGED, bool DUMP>
__global__ void __launch_bounds__(kW * 32, 1)
gemm_w4a8_stream_kernel(const GemmArgs a, const int NS, float *__restrict__ part,
                        int *__restrict__ count) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int T = NTG * 8;
    constexpr bool kPermA = (NTG >= 3) && !STAGED;   // where the even/odd-k shuffle is paid
    constexpr int kUnrollPairs = (NTG <= 2) ? 4 : 1;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int r = lane >> 2;
    const int c = lane & 3;
    const int S = a.max_splits;
    const int split = blockIdx.x % S;
    const int cta_i = blockIdx.x / S;                       // index among the CTAs of this split
    const int nctas = (gridDim.x - split + S - 1) / S;      // CTAs that share this split

    unsigned char *ring = smem + (size_t)warp * NS * kStageBytes;
    const uint32_t ring_u32 = smem_u32(ring);
    float2 *expw = reinterpret_cast<float2 *>(smem + (size_t)kW * NS * kStageBytes) + warp * 128;
    unsigned char *act = smem + (size_t)kW * NS * kStageBytes + kW * kExpBytes;

    const int groups = a.goff[a.count];
    const int tgid = cta_i + nctas * warp;                  // first row-group of this warp
    const int tstride = nctas * kW;
    const int ntasks = (tgid < groups) ? (groups - tgid + tstride - 1) / tstride : 0;
    const int Kt = a.K >> 5;
    const int ksh = a.ksh;
    const int Ktg = Kt >> ksh;
    const int kt_begin = Kt * split / S;
    const int cnt = Kt * (split + 1) / S - kt_begin;
    const int nst = (cnt + kST - 1) / kST;
    const int total_stages = ntasks * nst;
    const uint64_t pol = l2_policy_evict_first();

    // Producer side. The copy sequence of this warp is (task 0: stages 0..nst-1), (task 1:
    // ...), always NS stages ahead of the consumer; its position is kept as running
    // counters. Lane l copies bytes [16 l, 16 l + 16) of every 512-byte pair of tiles,
    // lanes below 2 * (scale lines) one 16-byte piece of the scales.
    int p_i = 0, p_slot = 0, p_g = tgid;
    const uint8_t *p_codes = nullptr;
    const uint8_t *p_scales = nullptr;
    auto issue_next = [&]() {
        if (p_i == 0) {
            int wi = 0;
            while (wi + 1 < a.count && p_g >= a.goff[wi + 1]) ++wi;
            const int lg = p_g - a.goff[wi];
            p_codes = a.codes[wi] + ((size_t)lg * Kt + kt_begin) * 256u + lane * 16;
            p_scales = reinterpret_cast<const uint8_t *>(a.scales[wi]) +
                       (size_t)lg * Ktg * 32u + lane * 16;
        }
        const int kt0 = kt_begin + p_i * kST;
        const int nt = min(kST, cnt - p_i * kST);
        const int sg0 = kt0 >> ksh;
        const int nsg = ((kt0 + nt - 1) >> ksh) + 1 - sg0;
        const uint32_t dst = ring_u32 + p_slot * kStageBytes + lane * 16;
        const uint8_t *src = p_codes + (size_t)p_i * (kST * 256);
        const int half = lane >> 4;
#pragma unroll
        for (int k = 0; k < kST / 2; ++k)
            if (2 * k + half < nt) cp_async16(dst + k * 512, src + k * 512, pol);
        if (lane < 2 * nsg) cp_async16(dst + kST * 256, p_scales + (size_t)sg0 * 32u, pol);
        if (++p_slot == NS) p_slot = 0;
        if (++p_i == nst) {
            p_i = 0;
            p_g += tstride;
        }
    };
    int issued = 0;                       // stages whose copies have been started
#pragma unroll 1
    for (int s = 0; s < NS; ++s) {        // always NS groups, empty ones included
        if (issued < total_stages) {
            issue_next();
            ++issued;
        }
        cp_async_commit();
    }

    // Stage this split's activations (all warps; the weight copies above are in flight).
    // Layout per (k-tile, token group): 32 lanes x 8 bytes of codes in B-fragment order
    // (lane (r, c): even-k bytes of token r, k = 8c.., then the odd-k bytes), followed by
    // 4 x 16 bytes {as[2c], as[2c+1], (float)asum[2c], (float)asum[2c+1]}.
    if (STAGED) {
        const int items = cnt * NTG * 32;
        for (int i = threadIdx.x; i < items; i += kW * 32) {
            const int kl = i / (NTG * 32);
            const int rem = i - kl * (NTG * 32);             // = tg * 32 + lane'
            const uint2 bb = __ldg(reinterpret_cast<const uint2 *>(
                a.aq + ((size_t)(kt_begin + kl) * T) * 32 + (size_t)rem * 8));
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
            const size_t src = (size_t)(kt_begin + kl) * T + (size_t)rem * 2;
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
    int slot = 0;
    for (int j = 0; j < ntasks; ++j) {
        const int g = tgid + j * tstride;
        int wi = 0;
        while (wi + 1 < a.count && g >= a.goff[wi + 1]) ++wi;
        const int lg = g - a.goff[wi];
        const int M = a.M[wi];

        f32x2 acc01[NTG], acc23[NTG];
#pragma unroll
        for (int t = 0; t < NTG; ++t) acc01[t] = acc23[t] = 0ull;

        for (int i = 0; i < nst; ++i) {
            const int cur = slot;
            if (++slot == NS) slot = 0;
            // this lane's pieces of the oldest stage have landed ...
            if (NS == 4) cp_async_wait<3>();
            else if (NS == 3) cp_async_wait<2>();
            else cp_async_wait<1>();
            __syncwarp();                 // ... and everybody else's
            const uint32_t cbase = ring_u32 + cur * kStageBytes + lane * 16;
            const int kt0 = kt_begin + i * kST;
            const int nt = min(kST, cnt - i * kST);

            // Expand this stage's scale words once into fp32 {ws, -(z+8)}. Entry (row, tile
            // pair p) = {ws, nz} of tile 2p followed by {ws, nz} of tile 2p+1, 16 bytes, stored
            // at [p][row]: the tile loop reads its two rows for TWO tiles with one 16-byte
            // load each, and never looks at the tier. Lane l converts row l & 15 of tiles
            // (l >> 4) + 2m, m = 0..3; loads and stores are conflict-free.
            {
                const int row = lane & 15, th = lane >> 4;
                const uint16_t *raw16 = reinterpret_cast<const uint16_t *>(
                    ring + cur * kStageBytes + kST * 256);
                const int par = kt0 & 1;
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    const int tl = 2 * m + th;
                    const int line = ksh ? ((tl + par) >> 1) : tl;
                    int zp;
                    float ws;
                    unpack_scale(raw16[line * 16 + row], zp, ws);
                    expw[(m * 16 + row) * 2 + th] =
                        make_float2(ws, (float)(-(zp + 8)));
                }
            }
            __syncwarp();

            // activations of this stage: staged copy in shared memory, or global through L1
            const unsigned char *actp =
                act + (size_t)(i * kST) * NTG * kActTileBytes + lane * 8;
            const unsigned char *asq = act + (size_t)(i * kST) * NTG * kActTileBytes + 256 + c * 16;
            const int8_t *aqp = a.aq + ((size_t)kt0 * T + r) * 32 + c * 8;
            const float *asp = a.as + (size_t)kt0 * T + 2 * c;
            const int32_t *smp = a.asum + (size_t)kt0 * T + 2 * c;

            // One 16-row x K32 tile against all token groups. jj = tile inside the stage.
            auto tile = [&](const int jj, const uint32_t w0, const uint32_t w1, const float ws0,
                            const float nz0, const float ws1, const float nz1) {
                const uint32_t x0 = (w0 & 0x0F0F0F0Fu) ^ 0x08080808u;          // even k
                const uint32_t y0 = ((w0 >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;   // odd k
                const uint32_t x1 = (w1 & 0x0F0F0F0Fu) ^ 0x08080808u;
                const uint32_t y1 = ((w1 >> 4) & 0x0F0F0F0Fu) ^ 0x08080808u;
                uint32_t a0, a1, a2, a3;
                if (kPermA) {   // k order restored on the weight side: B is the natural bytes
                    a0 = __byte_perm(x0, y0, 0x5140);
                    a2 = __byte_perm(x0, y0, 0x7362);
                    a1 = __byte_perm(x1, y1, 0x5140);
                    a3 = __byte_perm(x1, y1, 0x7362);
                } else {
                    a0 = x0; a1 = x1; a2 = y0; a3 = y1;
                }
                const f32x2 ws0x2 = pack2(ws0, ws0), nz0x2 = pack2(nz0, nz0);
                const f32x2 ws1x2 = pack2(ws1, ws1), nz1x2 = pack2(nz1, nz1);
#pragma unroll
                for (int t = 0; t < NTG; ++t) {
                    uint32_t b0, b1;
                    f32x2 as2, smf;
                    int2 sm2 = make_int2(0, 0);
                    if (STAGED) {
                        const uint2 bb = *reinterpret_cast<const uint2 *>(
                            actp + (jj * NTG + t) * kActTileBytes);
                        b0 = bb.x; b1 = bb.y;
                        const ulonglong2 av = *reinterpret_cast<const ulonglong2 *>(
                            asq + (jj * NTG + t) * kActTileBytes);
                        as2 = av.x; smf = av.y;
                    } else {
                        const uint2 bb =
                            __ldg(reinterpret_cast<const uint2 *>(aqp + (jj * T + t * 8) * 32));
                        if (kPermA) {
                            b0 = bb.x; b1 = bb.y;
                        } else {
                            b0 = __byte_perm(bb.x, bb.y, 0x6420);
                            b1 = __byte_perm(bb.x, bb.y, 0x7531);
                        }
                        as2 = __ldg(
                            reinterpret_cast<const unsigned long long *>(asp + jj * T + t * 8));
                        sm2 = __ldg(reinterpret_cast<const int2 *>(smp + jj * T + t * 8));
                        smf = pack2((float)sm2.x, (float)sm2.y);
                    }
                    int d[4];
                    mma_s8_c(d, a0, a1, a2, a3, b0, b1, cmagic);
                    if (DUMP) {
                        const size_t Mz = (size_t)a.M[0];
                        const size_t row0 = (size_t)lg * 16 + r;
                        int32_t *o = a.dump + ((size_t)(kt0 + jj) * T + t * 8 + 2 * c) * Mz;
                        o[row0] = d[0] - kMagicBits - 8 * sm2.x;
                        o[Mz + row0] = d[1] - kMagicBits - 8 * sm2.y;
                        o[row0 + 8] = d[2] - kMagicBits - 8 * sm2.x;
                        o[Mz + row0 + 8] = d[3] - kMagicBits - 8 * sm2.y;
                    }
                    // (float)(d - z*asum), exact: every term is an integer below 2^24
                    const f32x2 f01 = fma2(nz0x2, smf, add2(pack2i(d[0], d[1]), neg_magic2));
                    const f32x2 f23 = fma2(nz1x2, smf, add2(pack2i(d[2], d[3]), neg_magic2));
                    acc01[t] = fma2(f01, mul2(ws0x2, as2), acc01[t]);
                    acc23[t] = fma2(f23, mul2(ws1x2, as2), acc23[t]);
                }
            };

            if (nt == kST) {
#pragma unroll kUnrollPairs
                for (int jp = 0; jp < kST / 2; ++jp) {
                    uint32_t w00, w01, w10, w11;
                    ldmatrix_x4(cbase + jp * 512, w00, w01, w10, w11);
                    const float4 ea = *reinterpret_cast<const float4 *>(expw + (jp * 16 + r) * 2);
                    const float4 eb =
                        *reinterpret_cast<const float4 *>(expw + (jp * 16 + r + 8) * 2);
                    tile(2 * jp, w00, w01, ea.x, ea.y, eb.x, eb.y);
                    tile(2 * jp + 1, w10, w11, ea.z, ea.w, eb.z, eb.w);
                }
            } else {
                for (int jj = 0; jj < nt; jj += 2) {
                    uint32_t w00, w01, w10, w11;
                    ldmatrix_x4(cbase + jj * 256, w00, w01, w10, w11);
                    const float4 ea =
                        *reinterpret_cast<const float4 *>(expw + ((jj >> 1) * 16 + r) * 2);
                    const float4 eb =
                        *reinterpret_cast<const float4 *>(expw + ((jj >> 1) * 16 + r + 8) * 2);
                    tile(jj, w00, w01, ea.x, ea.y, eb.x, eb.y);
                    if (jj + 1 < nt) tile(jj + 1, w10, w11, ea.z, ea.w, eb.z, eb.w);
                }
            }
            __syncwarp();                 // all reads of this slot done before it is refilled
            if (issued < total_stages) {
                issue_next();
                ++issued;
            }
            cp_async_commit();
        }
        if constexpr (!DUMP) {
            float out[NTG][4];
#pragma unroll
            for (int t = 0; t < NTG; ++t) {
                unpack2(acc01[t], out[t][0], out[t][1]);
                unpack2(acc23[t], out[t][2], out[t][3]);
            }
            if (S > 1) {
                // partial of this split -> scratch; the last split to arrive sums 0..S-1
                float *pp = part + ((size_t)g * S + split) * (NTG * 128) + lane;
#pragma unroll
                for (int t = 0; t < NTG; ++t)
#pragma unroll
                    for (int k = 0; k < 4; ++k) pp[(t * 4 + k) * 32] = out[t][k];
                __threadfence();
                __syncwarp();
                int old = 0;
                if (lane == 0) old = atomicAdd(count + g, 1);
                old = __shfl_sync(0xffffffffu, old, 0);
                if (old != S - 1) continue;
                __threadfence();
                const float *base = part + (size_t)g * S * (NTG * 128) + lane;
#pragma unroll
                for (int t = 0; t < NTG; ++t)
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        float sum = 0.0f;
                        for (int s = 0; s < S; ++s)
                            sum = __fadd_rn(sum, __ldcg(base + (size_t)s * (NTG * 128) + (t * 4 + k) * 32));
                        out[t][k] = sum;
                    }
                if (lane == 0) count[g] = 0;   // ready for the next launch
            }
            float *y = a.y[wi];
            const size_t row = (size_t)lg * 16 + r;
#pragma unroll
            for (int t = 0; t < NTG; ++t) {
                const size_t tok = (size_t)t * 8 + 2 * c;
                y[tok * M + row] = out[t][0];
                y[(tok + 1) * M + row] = out[t][1];
                y[tok * M + row + 8] = out[t][2];
                y[(tok + 1) * M + row + 8] = out[t][3];
            }
        }
    }
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

size_t ring_bytes(int NS) { return (size_t)kW * NS * kStageBytes + (size_t)kW * kExpBytes; }

template <int NTG, bool STAGED, bool DUMP>
void launch_variant(const GemmArgs &a, int NS, size_t smem) {
    static bool attr_set = false;
    if (!attr_set) {
        TQ_CHECK(cudaFuncSetAttribute(gemm_w4a8_stream_kernel<NTG, STAGED, DUMP>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)kSmemLimit));
        attr_set = true;
    }
    const int S = a.max_splits;
    const int groups = a.goff[a.count];
    if (S > 1 && !DUMP) ensure_scratch((size_t)groups * S * NTG * 128, groups);
    const int want = ((groups + kW - 1) / kW) * S;
    const int grid = std::max(S, std::min(g_num_sms, want));
    gemm_w4a8_stream_kernel<NTG, STAGED, DUMP>
        <<<grid, kW * 32, smem, stream()>>>(a, NS, g_scratch.part, g_scratch.count);
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
        launch_variant<NTG, false, true>(a, 4, ring_bytes(4));
        return;
    }
    if (NTG <= 4) {
        // Deepest ring that still leaves room for this split's staged activations.
        const int Kt = a.K >> 5, S = a.max_splits;
        const size_t act = (size_t)((Kt + S - 1) / S) * NTG * kActTileBytes;
        for (int NS = 4; NS >= 2; --NS) {
            if (ring_bytes(NS) + act <= kSmemLimit) {
                launch_variant<(NTG <= 4 ? NTG : 1), true, false>(a, NS, ring_bytes(NS) + act);
                return;
            }
        }
    }
    launch_variant<NTG, false, false>(a, 4, ring_bytes(4));
}

}  // namespace

bool gemm_stream_covers(const GemmArgs &a) {
    if (a.count < 1 || a.T < 8 || a.T > 64 || (a.T % 8)) return false;
    if (a.max_splits > 16) return false;
    if (a.ksh && ((a.K >> 5) & 1)) return false;
    if (a.dump && a.count != 1) return false;
    for (int i = 0; i < a.count; ++i)
        if (a.seg[i].count != 1 || a.seg[i].split[0] != a.max_splits) return false;
    return true;
}

void launch_gemm_stream(const GemmArgs &a) {
    switch (a.T / 8) {
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
