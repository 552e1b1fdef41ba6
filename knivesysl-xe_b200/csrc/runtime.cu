// runtime.cu — device runtime of the projection library: one in-order CUDA stream
// per process/device, checked allocation and copies, the prepared-activation
// scratch, events. Replaces the SYCL queue layer of xpu/src/decode.cpp:40-130.
#include "common.cuh"

#include <vector>

#include <string.h>

namespace tq {

namespace {
cudaStream_t g_stream = nullptr;
int g_device = -1;
int g_sticky_error = 0;
ActScratch g_act;
int *g_status_dev = nullptr;
unsigned long long g_alloc_calls = 0;
unsigned long long g_wait_limit_ns = 2000000000ull;   // bounded device-side waits: 2 s

void init_device_once() {
    if (g_stream) return;
    if (g_device < 0) {
        int dev = 0;
        if (const char *e = getenv("TQ_XPU_DEV")) dev = atoi(e);   // same selector name
        int n = 0;
        if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) {
            fprintf(stderr, "forward_qwen_xpu(b200): no CUDA device found\n");
            abort();
        }
        if (dev < 0 || dev >= n) dev = 0;
        g_device = dev;
    }
    cudaError_t e = cudaSetDevice(g_device);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&g_stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        fprintf(stderr, "forward_qwen_xpu(b200): cannot create stream on device %d: %s\n",
                g_device, cudaGetErrorString(e));
        abort();
    }
}
}  // namespace

cudaStream_t stream() {
    init_device_once();
    return g_stream;
}

void note_error(cudaError_t e, const char *where) {
    if (e == cudaSuccess) return;
    if (!g_sticky_error) {
        g_sticky_error = (int)e;
        fprintf(stderr, "forward_qwen_xpu(b200): CUDA error %d (%s) at %s\n", (int)e,
                cudaGetErrorString(e), where);
    }
}

ActScratch &act_scratch() { return g_act; }

unsigned long long wait_limit_ns() { return g_wait_limit_ns; }

void ensure_act_scratch(int K) {
    ActScratch &s = g_act;
    if (s.cap >= K) return;
    // tq_dev_free waits for the library stream before it frees, so nothing queued can
    // still read the old scratch.
    if (s.q) tq_dev_free(s.q);
    if (s.qp) tq_dev_free(s.qp);
    if (s.scale) tq_dev_free(s.scale);
    if (s.sum16) tq_dev_free(s.sum16);
    if (s.sum32) tq_dev_free(s.sum32);
    if (s.norm_partial) tq_dev_free(s.norm_partial);
    s.q = static_cast<int8_t *>(tq_dev_alloc((size_t)K, "act.q8"));
    s.qp = static_cast<int8_t *>(tq_dev_alloc((size_t)K, "act.q8.permuted"));
    s.scale = static_cast<float *>(tq_dev_alloc((size_t)(K / 32) * sizeof(float), "act.scale"));
    s.sum16 = static_cast<int32_t *>(tq_dev_alloc((size_t)(K / 16) * sizeof(int32_t), "act.sum16"));
    s.sum32 = static_cast<int32_t *>(tq_dev_alloc((size_t)(K / 32) * sizeof(int32_t), "act.sum32"));
    s.norm_partial = static_cast<float *>(
        tq_dev_alloc((size_t)((K + 255) / 256) * sizeof(float), "norm.partial"));
    s.cap = K;
    s.prepared_K = 0;
}

int *device_status_word() {
    if (!g_status_dev) {
        g_status_dev = static_cast<int *>(tq_dev_alloc(sizeof(int), "status"));
        TQ_CHECK(cudaMemsetAsync(g_status_dev, 0, sizeof(int), stream()));
    }
    return g_status_dev;
}

}  // namespace tq

extern "C" {

int tq_set_device(int device) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || device < 0 || device >= n) return -1;
    if (tq::g_stream && device != tq::g_device) return -2;   // one device per process
    tq::g_device = device;
    tq::init_device_once();
    return 0;
}

int tq_device(void) {
    tq::init_device_once();
    return tq::g_device;
}

void *tq_stream(void) { return (void *)tq::stream(); }

void *tq_dev_alloc(size_t bytes, const char *what) {
    tq::init_device_once();
    ++tq::g_alloc_calls;
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes ? bytes : 1);
    if (e != cudaSuccess || !p) {
        fprintf(stderr, "forward_qwen_xpu(b200): device alloc of %zu bytes failed (%s): %s\n",
                bytes, what ? what : "?", cudaGetErrorString(e));
        abort();
    }
    return p;
}

void tq_dev_free(void *p) {
    if (!p) return;
    // Kernels that were launched with programmatic dependent launch may not have started
    // yet; wait for the stream explicitly so that nothing in flight can still touch p.
    if (tq::g_stream) TQ_CHECK(cudaStreamSynchronize(tq::g_stream));
    TQ_CHECK(cudaFree(p));
}

void tq_h2d(void *dst, const void *src, size_t bytes) {
    TQ_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, tq::stream()));
    TQ_CHECK(cudaStreamSynchronize(tq::stream()));
}

void tq_d2h(void *dst, const void *src, size_t bytes) {
    TQ_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, tq::stream()));
    TQ_CHECK(cudaStreamSynchronize(tq::stream()));
}

void tq_dev_zero(void *dst, size_t bytes) {
    TQ_CHECK(cudaMemsetAsync(dst, 0, bytes, tq::stream()));
    TQ_CHECK(cudaStreamSynchronize(tq::stream()));
}

void tq_dev_fill(void *dst, int byte, size_t bytes) {
    TQ_CHECK(cudaMemsetAsync(dst, byte, bytes, tq::stream()));
}

namespace tq {
constexpr int kCopyTickets = 16;
cudaStream_t g_copy_stream = nullptr;                // device to host
cudaStream_t g_up_stream = nullptr;                  // host to device
cudaEvent_t g_copy_ready = nullptr;                 // library stream -> copy stream
cudaEvent_t g_copy_done[kCopyTickets] = {};         // copy stream -> library stream
unsigned g_copy_next = 0;
}  // namespace tq

void tq_sync(void) {
    TQ_CHECK(cudaStreamSynchronize(tq::stream()));
    if (tq::g_copy_stream) TQ_CHECK(cudaStreamSynchronize(tq::g_copy_stream));
    if (tq::g_up_stream) TQ_CHECK(cudaStreamSynchronize(tq::g_up_stream));
    if (tq::g_status_dev && !tq::g_sticky_error) {
        int st = 0;
        if (cudaMemcpy(&st, tq::g_status_dev, sizeof(int), cudaMemcpyDeviceToHost) == cudaSuccess &&
            st != 0) {
            tq::g_sticky_error = 10000 + st;
            fprintf(stderr, "forward_qwen_xpu(b200): device wait gave up, status %d\n", st);
        }
    }
}

int tq_last_error(void) { return tq::g_sticky_error; }

void tq_clear_error(void) {
    if (tq::g_status_dev) {
        TQ_CHECK(cudaStreamSynchronize(tq::stream()));
        TQ_CHECK(cudaMemset(tq::g_status_dev, 0, sizeof(int)));
    }
    tq::g_sticky_error = 0;
}

void tq_set_wait_limit_ms(int ms) {
    tq::g_wait_limit_ns = (unsigned long long)(ms < 1 ? 1 : ms) * 1000000ull;
}

unsigned long long tq_dev_alloc_count(void) { return tq::g_alloc_calls; }

void *tq_host_alloc_pinned(size_t bytes) {
    tq::init_device_once();
    void *p = nullptr;
    if (cudaMallocHost(&p, bytes ? bytes : 1) != cudaSuccess) return nullptr;
    return p;
}

void tq_host_free_pinned(void *p) {
    if (p) TQ_CHECK(cudaFreeHost(p));
}

void tq_h2d_async(void *dst, const void *src, size_t bytes) {
    TQ_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, tq::stream()));
}

void tq_d2h_async(void *dst, const void *src, size_t bytes) {
    TQ_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, tq::stream()));
}

// ---- copies that overlap the calls around them ---------------------------------------
// Two more streams carry copies, one per direction so that both copy engines can run at
// once: a copy waits for what the library stream has queued so far, and the library stream
// only waits for a copy when the caller says so, through a ticket (before it lets a kernel
// overwrite a buffer that is being read back, or read a buffer that is being uploaded).

namespace tq {
int overlapped_copy(void *dst, const void *src, size_t bytes, bool up) {
    cudaStream_t main = stream();
    if (!g_copy_stream) {
        TQ_CHECK(cudaStreamCreateWithFlags(&g_copy_stream, cudaStreamNonBlocking));
        TQ_CHECK(cudaStreamCreateWithFlags(&g_up_stream, cudaStreamNonBlocking));
        TQ_CHECK(cudaEventCreateWithFlags(&g_copy_ready, cudaEventDisableTiming));
        for (auto &e : g_copy_done) TQ_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    }
    if (!g_copy_stream || !g_up_stream) return -1;
    cudaStream_t cs = up ? g_up_stream : g_copy_stream;
    const int ticket = (int)(g_copy_next++ % kCopyTickets);
    TQ_CHECK(cudaEventRecord(g_copy_ready, main));
    TQ_CHECK(cudaStreamWaitEvent(cs, g_copy_ready, 0));
    TQ_CHECK(cudaMemcpyAsync(dst, src, bytes, up ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost, cs));
    TQ_CHECK(cudaEventRecord(g_copy_done[ticket], cs));
    return ticket;
}
}  // namespace tq

int tq_d2h_overlapped(void *dst, const void *src, size_t bytes) {
    return tq::overlapped_copy(dst, src, bytes, false);
}

int tq_h2d_overlapped(void *dst, const void *src, size_t bytes) {
    return tq::overlapped_copy(dst, src, bytes, true);
}

void tq_stream_wait_copy(int ticket) {
    if (ticket < 0 || ticket >= tq::kCopyTickets || !tq::g_copy_stream) return;
    TQ_CHECK(cudaStreamWaitEvent(tq::stream(), tq::g_copy_done[ticket], 0));
}

void tq_d2d_async(void *dst, const void *src, size_t bytes) {
    TQ_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, tq::stream()));
}

void *tq_event_create(void) {
    tq::init_device_once();
    cudaEvent_t ev = nullptr;
    TQ_CHECK(cudaEventCreate(&ev));
    return (void *)ev;
}

void tq_event_destroy(void *ev) {
    if (ev) TQ_CHECK(cudaEventDestroy((cudaEvent_t)ev));
}

void tq_event_record(void *ev) { TQ_CHECK(cudaEventRecord((cudaEvent_t)ev, tq::stream())); }

// Stream capture into a CUDA graph: everything issued on tq_stream() between begin and end
// becomes one replayable graph (no allocation or blocking call may happen in between, so
// warm every entry point up once before capturing).
int tq_graph_capture_begin(void) {
    cudaError_t e = cudaStreamBeginCapture(tq::stream(), cudaStreamCaptureModeThreadLocal);
    tq::note_error(e, "cudaStreamBeginCapture");
    return e == cudaSuccess ? 0 : -1;
}

void *tq_graph_capture_end(void) {
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(tq::stream(), &graph);
    if (e != cudaSuccess || !graph) {
        tq::note_error(e, "cudaStreamEndCapture");
        return nullptr;
    }
    cudaGraphExec_t exec = nullptr;
    e = cudaGraphInstantiate(&exec, graph, 0);
    tq::note_error(e, "cudaGraphInstantiate");
    cudaGraphDestroy(graph);
    return e == cudaSuccess ? (void *)exec : nullptr;
}

void tq_graph_launch(void *exec) {
    if (exec) TQ_CHECK(cudaGraphLaunch((cudaGraphExec_t)exec, tq::stream()));
}

void tq_graph_destroy(void *exec) {
    if (exec) TQ_CHECK(cudaGraphExecDestroy((cudaGraphExec_t)exec));
}

float tq_event_elapsed_ms(void *start, void *stop) {
    float ms = -1.0f;
    TQ_CHECK(cudaEventSynchronize((cudaEvent_t)stop));
    TQ_CHECK(cudaEventElapsedTime(&ms, (cudaEvent_t)start, (cudaEvent_t)stop));
    return ms;
}

}  // extern "C"

// ---- per-projection timers (the reference's profile_projection, xpu/src/decode.cpp:156-219) ----
// The reference waits for the queue and reads the host clock around every projection; here a
// pair of CUDA events goes onto the stream around the call and nothing waits until the report
// is asked for, so profiling does not serialise the steps it measures. Off by default
// (TQ_XPU_PROFILE_PROJ=1 or tq_profile_enable); calls made during stream capture are not timed.
namespace tq {
namespace {
struct ProfSpan {
    int M, K, T, tier;
    cudaEvent_t e0, e1;
};
std::vector<ProfSpan> g_prof_spans;
std::vector<cudaEvent_t> g_prof_free;
int g_prof_on = -1;
constexpr size_t kProfMaxSpans = 1 << 16;

cudaEvent_t prof_event() {
    if (!g_prof_free.empty()) {
        cudaEvent_t e = g_prof_free.back();
        g_prof_free.pop_back();
        return e;
    }
    cudaEvent_t e = nullptr;
    TQ_CHECK(cudaEventCreate(&e));
    return e;
}
}  // namespace

bool profile_on() {
    if (g_prof_on < 0) {
        const char *e = getenv("TQ_XPU_PROFILE_PROJ");
        g_prof_on = (e && *e && *e != '0') ? 1 : 0;
    }
    return g_prof_on > 0;
}

ProfScope::ProfScope(int M, int K, int T, int tier) {
    if (!profile_on() || g_prof_spans.size() >= kProfMaxSpans) return;
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream(), &st) != cudaSuccess || st != cudaStreamCaptureStatusNone) return;
    g_prof_spans.push_back(ProfSpan{M, K, T, tier, prof_event(), prof_event()});
    index_ = (int)g_prof_spans.size() - 1;
    TQ_CHECK(cudaEventRecord(g_prof_spans[index_].e0, stream()));
}
ProfScope::~ProfScope() {
    if (index_ >= 0) TQ_CHECK(cudaEventRecord(g_prof_spans[index_].e1, stream()));
}
}  // namespace tq

extern "C" int tq_profile_enable(int on) {
    const int was = tq::profile_on() ? 1 : 0;
    tq::g_prof_on = on ? 1 : 0;
    return was;
}

// Waits for the stream, adds the recorded spans up per (M, K, T, tier), prints one line per
// projection and clears the record. rows, when not NULL, receives up to max_rows entries of six
// doubles {M, K, T, tier, calls, total microseconds}. Returns the number of distinct
// projections. tier: 4 = W4A8 K32, 64 = K64, 16 = K16, 8 = W8A8, 6 = scalar E2M3, 44 = W4A4.
extern "C" int tq_profile_report(double *rows, int max_rows) {
    using namespace tq;
    tq_sync();
    struct Agg {
        int M, K, T, tier;
        long calls;
        double us;
    };
    std::vector<Agg> agg;
    for (const ProfSpan &sp : g_prof_spans) {
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, sp.e0, sp.e1) != cudaSuccess) ms = 0.0f;
        size_t i = 0;
        while (i < agg.size() && !(agg[i].M == sp.M && agg[i].K == sp.K && agg[i].T == sp.T && agg[i].tier == sp.tier)) ++i;
        if (i == agg.size()) agg.push_back(Agg{sp.M, sp.K, sp.T, sp.tier, 0, 0.0});
        agg[i].calls += 1;
        agg[i].us += (double)ms * 1e3;
        g_prof_free.push_back(sp.e0);
        g_prof_free.push_back(sp.e1);
    }
    g_prof_spans.clear();
    for (size_t i = 0; i < agg.size(); ++i) {
        printf("projection [%d x %d] T=%d tier %d: %ld calls, %.1f us, %.2f us/call\n", agg[i].M, agg[i].K, agg[i].T,
               agg[i].tier, agg[i].calls, agg[i].us, agg[i].us / (double)agg[i].calls);
        if (rows && (int)i < max_rows) {
            double *r = rows + 6 * i;
            r[0] = agg[i].M; r[1] = agg[i].K; r[2] = agg[i].T; r[3] = agg[i].tier;
            r[4] = (double)agg[i].calls; r[5] = agg[i].us;
        }
    }
    return (int)agg.size();
}
