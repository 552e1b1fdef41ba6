// tc_peak.cu — issue-rate measurement of tcgen05.mma kind::i8 on this GPU: the dense int8
// tensor peak the prefill GEMM's fractions are quoted against. No counterpart in the
// reference (its roofs come from its own DPAS probes, xpu/probe/dpas_probe.cpp).
//
// Every SM runs one CTA whose single issuing thread queues `iters` MMAs of shape
// M128 x N x K32 (int8 x int8 -> int32 in TMEM) over two alternating accumulators, reading
// the same two operand tiles from shared memory every time; there is no epilogue and nothing
// is read back, so the time is the tensor pipe's. Operands are zeros: the pipe's rate does
// not depend on values.
#include "tc.cuh"

namespace tq {
namespace {

__global__ void __launch_bounds__(128, 1)
tc_int8_peak_kernel(int n, int iters, int accs, int tiles, long long *clocks, int *status, unsigned long long wait_ns) {
    extern __shared__ __align__(1024) unsigned char smem[];
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_base_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < tiles * (4096 + 8192) / 16; i += 128)
        reinterpret_cast<uint4 *>(smem)[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        mbar_init_fence();
    }
    if (warp == 0) {
        tmem_alloc(smem_u32(&tmem_base_s), 512);
        tmem_relinquish();
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    if (warp == 0) {
        long long t0 = 0, t1 = 0;
        if (lane == 0) {
            const uint32_t a = smem_u32(smem), b = a + 4096;
            const uint32_t idesc = idesc_i8(128, n);
            t0 = clock64();
            for (int i = 0; i < iters; ++i) {
                const uint32_t off = (uint32_t)(i % tiles) * (4096 + 8192);
                tc_mma_i8(tmem_base + (uint32_t)(i % accs) * (uint32_t)n, smem_desc(a + off), smem_desc(b + off),
                          idesc, i >= accs ? 1u : 0u);
            }
            t1 = clock64();
            tc_commit(smem_u32(&bar));
        }
        __syncwarp();
        bool ok = mbar_wait_bounded(smem_u32(&bar), 0, status, 51, wait_ns);
        (void)ok;
        if (lane == 0 && clocks) {
            clocks[blockIdx.x * 2] = t1 - t0;            // issue time of the whole queue
            clocks[blockIdx.x * 2 + 1] = clock64() - t0;  // ... until the last MMA has completed
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) tmem_dealloc(tmem_base, 512);
}

}  // namespace
}  // namespace tq

// Dense int8 TOP/s (2 * M * N * K per MMA) that `iters` queued MMAs of width n (multiple of
// 16, 16..256) reach on all SMs; accs (1..512/n) accumulators are used in turn. clocks_out, if
// not NULL, receives {issue clocks, clocks to completion} of SM 0's queue. Returns < 0 on a
// bad argument or a failed launch.
extern "C" double qwn_tc_int8_probe(int n, int iters, int accs, long long *clocks_out) {
    using namespace tq;
    // TQ_XPU_PEAK_TILES distinct operand tile pairs are read in turn (1..9; default 1)
    static const int tiles = [] {
        const char *e = getenv("TQ_XPU_PEAK_TILES");
        const int v = (e && *e) ? atoi(e) : 1;
        return v < 1 ? 1 : (v > 9 ? 9 : v);
    }();
    if (n < 16 || n > 256 || (n % 16) || iters < 1 || accs < 1 || accs * n > 512) return -1.0;
    int dev = 0, sms = 0;
    TQ_CHECK(cudaGetDevice(&dev));
    TQ_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    if (sms <= 0) return -2.0;
    long long *d_clk = static_cast<long long *>(tq_dev_alloc((size_t)sms * 16, "tc.peak.clocks"));
    const size_t smem = 120 * 1024;     // more than half an SM: one CTA per SM
    TQ_CHECK(cudaFuncSetAttribute(tc_int8_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaEvent_t e0, e1;
    TQ_CHECK(cudaEventCreate(&e0));
    TQ_CHECK(cudaEventCreate(&e1));
    for (int rep = 0; rep < 2; ++rep) {          // first run warms up
        TQ_CHECK(cudaEventRecord(e0, stream()));
        tc_int8_peak_kernel<<<sms, 128, smem, stream()>>>(n, iters, accs, tiles, d_clk, device_status_word(),
                                                         wait_limit_ns());
        TQ_LAUNCH_CHECK("tc_int8_peak_kernel");
        TQ_CHECK(cudaEventRecord(e1, stream()));
    }
    tq_sync();
    float ms = 0.0f;
    TQ_CHECK(cudaEventElapsedTime(&ms, e0, e1));
    if (clocks_out) tq_d2h(clocks_out, d_clk, 16);
    tq_dev_free(d_clk);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (ms <= 0.0f) return -3.0;
    return 2.0 * 128.0 * n * 32.0 * iters * sms / (ms * 1e-3) / 1e12;
}

extern "C" double qwn_tc_int8_peak(int iters) { return qwn_tc_int8_probe(256, iters < 1 ? 4000 : iters, 2, nullptr); }
