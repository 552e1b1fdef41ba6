// gemv_static.cu — a single-row W4A8 GEMV that never allocates.
//
// The ordinary x_gemv_w4a8 stages the quantised activation in scratch buffers that the
// library grows with cudaMalloc on demand. Some callers cannot tolerate that: code that
// runs inside a region where device allocation is forbidden or would synchronise the
// whole device (a latency-critical serving loop that pre-allocated everything, a caller
// whose memory pool owns the entire GPU so cudaMalloc would fail, a host thread that
// must not take the driver's allocation lock). For them the staging scratch of this
// variant is a fixed array in the library's own device image: it exists from the
// moment the library is loaded on a GPU until the process exits, about 80 KiB per GPU,
// and bounds the reduction length at kStaticMaxK.
//
// Consequences a caller must know:
//  * K above kStaticMaxK is rejected (return -30); nothing is launched.
//  * Every call shares the one array. Calls are ordered on the library's stream, so
//    back-to-back calls are safe; two calls made to overlap on the GPU (another stream,
//    another host thread) would race on it. Nothing in it has to start at zero: each
//    call rewrites every byte it later reads, so stale contents are harmless.
//  * The first call on a device looks up the array's device address (set-up). Make that
//    first call before starting any stream capture.
#include "common.cuh"

namespace {

constexpr int kStaticMaxK = 32768;
constexpr int kMaxDevices = 64;

struct StaticActScratch {
    int8_t qp[kStaticMaxK];             // codes, even-k / odd-k split per 32-byte tile
    int8_t q[kStaticMaxK];              // codes in natural order
    float scale[kStaticMaxK / 32];      // one scale per K32 block
    int32_t sum16[kStaticMaxK / 16];    // code sums per K16
    int32_t sum32[kStaticMaxK / 32];    // code sums per K32
};

// In host code this name is only a handle for the runtime, not a device address.
static __device__ __align__(256) StaticActScratch g_static_act;

// Device address of g_static_act per device, looked up once with that device current.
StaticActScratch *g_static_ptr[kMaxDevices] = {};

StaticActScratch *static_scratch_for_current_device() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    if (!g_static_ptr[dev]) {
        void *p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_act);
        if (e != cudaSuccess || !p) {
            tq::note_error(e, "cudaGetSymbolAddress(g_static_act)");
            return nullptr;
        }
        g_static_ptr[dev] = static_cast<StaticActScratch *>(p);
    }
    return g_static_ptr[dev];
}

}  // namespace

extern "C" int qwn_x_gemv_w4a8_static(const tq_qmma_weight_t *w, const float *d_x, float *d_y) {
    if (!w || !d_x || !d_y || !w->s4_ready || !w->d_s4 || !w->d_s4_scale) return -1;
    if (w->s4_k16) return -20;
    if (w->M <= 0 || w->K <= 0 || (w->M % 16) || (w->K % 32)) return -1;
    if (w->K > kStaticMaxK) {
        fprintf(stderr,
                "qwn_x_gemv_w4a8_static: K=%d exceeds the built-in scratch (max K %d); use "
                "x_gemv_w4a8 or rebuild with a larger kStaticMaxK\n", w->K, kStaticMaxK);
        return -30;
    }
    tq::stream();   // binds the library's device; created at tq_set_device in normal use
    StaticActScratch *s = static_scratch_for_current_device();
    if (!s) return -31;
    tq::launch_quant_s8(d_x, nullptr, nullptr, w->K, s->q, s->qp, s->scale, s->sum16, s->sum32,
                        false);
    tq::GemvArgs a{};
    a.codes[0] = w->d_s4;
    a.scales[0] = w->d_s4_scale;
    a.y[0] = d_y;
    a.goff[0] = 0;
    a.goff[1] = w->M / 16;
    a.count = 1;
    a.qp = s->qp;
    a.as = s->scale;
    a.sum32 = s->sum32;
    a.residual = nullptr;
    a.K = w->K;
    a.ksh = w->s4_k64 ? 1 : 0;
    a.splits = tq::choose_gemv_splits(w->M / 16);
    a.serial = 0;
    a.dump = nullptr;
    tq::launch_gemv(a);
    return 0;
}

extern "C" int qwn_static_max_k(void) { return kStaticMaxK; }
