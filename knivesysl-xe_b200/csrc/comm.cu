// comm.cu — the exchange step of a column-sharded projection: an all-gather of the
// ranks' output slices over NVLink. One process per GPU; NCCL is loaded at run time
// (dlopen) so a single-GPU user needs no NCCL at all. The reference's only collective
// is a 2-rank peer-copy all-reduce (xpu/src/decode.cpp:133-154); a column shard needs
// an all-gather instead; the row-parallel (K) shard's partial sums are added with
// tq_comm_allreduce_sum.
#include "common.cuh"

#include <dlfcn.h>
#include <string.h>

namespace {

typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
enum { kNcclInt8 = 0 };   // ncclInt8 / ncclChar

struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
} g_api;

ncclComm_t g_comm = nullptr;
int g_rank = 0, g_world = 1;
tq::GatherState g_gather;

// Publishes a step and waits for everybody's. Runs after the GEMM whose epilogue stored this
// rank's slice on every rank (griddepcontrol.wait returns once that kernel has completed and
// its stores, the peer stores included, have been performed): lane p stores the step number
// into this rank's flag word on rank p behind a system-scope fence, then waits until rank p's
// flag word here has reached the step (bounded: limit_ns of wall clock, two seconds unless
// tq_set_wait_limit_ms changed it, then status 31 and a normal return). Whatever follows on the stream therefore finds every rank's slice in
// the gathered buffer.
struct PeerFlags {
    int *p[8];
};
__global__ void gather_publish_wait_kernel(PeerFlags f, const int *mine, int world, int step,
                                           int *status, unsigned long long limit_ns) {
    tq::pdl_trigger();
    tq::pdl_wait();
    const int p = threadIdx.x;
    if (p >= world) return;
    __threadfence_system();
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(f.p[p]), "r"(step) : "memory");
    unsigned long long t0 = 0;
    for (unsigned polls = 0;; ++polls) {
        int v;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine + p) : "memory");
        if (v - step >= 0) return;
        __nanosleep(100);
        if ((polls & 255u) == 255u) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_ns) break;
        }
    }
    atomicCAS(status, 0, 31);
}

// One thread: the step base of the next pass (see SyncArgs).
__global__ void exchange_advance_kernel(int *base, int n) {
    tq::pdl_trigger();
    tq::pdl_wait();
    if (threadIdx.x == 0) *base += n;
}

// An exchange point on its own (nothing to stage behind it): e.g. before the host reads the
// last gathered result of a pass.
__global__ void exchange_sync_kernel(tq::SyncArgs sa) {
    tq::pdl_trigger();
    tq::pdl_wait();
    tq::exchange_sync(sa);
}

bool load_nccl() {
    if (g_api.handle) return true;
    const char *names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
        g_api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (g_api.handle) break;
    }
    if (!g_api.handle) {
        fprintf(stderr, "forward_qwen_xpu(b200): cannot load NCCL: %s\n", dlerror());
        return false;
    }
    g_api.GetUniqueId = (decltype(g_api.GetUniqueId))dlsym(g_api.handle, "ncclGetUniqueId");
    g_api.CommInitRank = (decltype(g_api.CommInitRank))dlsym(g_api.handle, "ncclCommInitRank");
    g_api.AllGather = (decltype(g_api.AllGather))dlsym(g_api.handle, "ncclAllGather");
    g_api.AllReduce = (decltype(g_api.AllReduce))dlsym(g_api.handle, "ncclAllReduce");
    g_api.CommDestroy = (decltype(g_api.CommDestroy))dlsym(g_api.handle, "ncclCommDestroy");
    g_api.GetErrorString = (decltype(g_api.GetErrorString))dlsym(g_api.handle, "ncclGetErrorString");
    if (!g_api.GetUniqueId || !g_api.CommInitRank || !g_api.AllGather || !g_api.CommDestroy) {
        fprintf(stderr, "forward_qwen_xpu(b200): NCCL symbols missing\n");
        dlclose(g_api.handle);
        g_api.handle = nullptr;
        return false;
    }
    return true;
}

int nccl_fail(ncclResult_t r, const char *where) {
    fprintf(stderr, "forward_qwen_xpu(b200): NCCL error %d at %s: %s\n", r, where,
            g_api.GetErrorString ? g_api.GetErrorString(r) : "?");
    return -10;
}

}  // namespace

namespace tq {
GatherState &gather_state() { return g_gather; }

SyncArgs exchange_point() {
    GatherState &g = g_gather;
    SyncArgs sa{};
    if (g.world < 1 || !g.step_base) return sa;
    for (int p = 0; p < g.world; ++p) sa.peer_flag[p] = g.flag[p] + g.rank;
    sa.mine = g.flag[g.rank];
    sa.base = g.step_base;
    sa.k = ++g.pass_syncs;
    sa.world = g.world;
    sa.status = device_status_word();
    sa.limit_ns = wait_limit_ns();
    return sa;
}

void launch_gather_publish(int step) {
    GatherState &g = g_gather;
    PeerFlags f{};
    for (int p = 0; p < g.world; ++p) f.p[p] = g.flag[p] + g.rank;
    launch_pdl(gather_publish_wait_kernel, dim3(1), dim3(32), 0, f, (const int *)g.flag[g.rank],
               g.world, step, device_status_word(), wait_limit_ns());
    note_error(cudaGetLastError(), "gather_publish_wait_kernel");
}
}  // namespace tq

extern "C" {

int tq_comm_unique_id(void *id128) {
    if (!id128 || !load_nccl()) return -1;
    ncclUniqueId id;
    const ncclResult_t r = g_api.GetUniqueId(&id);
    if (r != 0) return nccl_fail(r, "ncclGetUniqueId");
    memcpy(id128, &id, sizeof id);
    return 0;
}

int tq_comm_init(const void *id128, int rank, int world) {
    if (world < 1 || rank < 0 || rank >= world) return -2;
    if (g_comm) return -3;
    g_rank = rank;
    g_world = world;
    if (world == 1) return 0;
    if (!id128 || !load_nccl()) return -1;
    tq::stream();   // binds the device before the communicator is created
    ncclUniqueId id;
    memcpy(&id, id128, sizeof id);
    const ncclResult_t r = g_api.CommInitRank(&g_comm, world, id, rank);
    if (r != 0) return nccl_fail(r, "ncclCommInitRank");
    return 0;
}

// Every rank contributes bytes_per_rank; d_recv holds world * bytes_per_rank, rank-major.
int tq_comm_allgather(const void *d_send, void *d_recv, size_t bytes_per_rank) {
    if (!d_send || !d_recv) return -1;
    if (g_world == 1) {
        if (d_send != d_recv) tq_d2d_async(d_recv, d_send, bytes_per_rank);
        return 0;
    }
    if (!g_comm) return -3;
    const ncclResult_t r =
        g_api.AllGather(d_send, d_recv, bytes_per_rank, kNcclInt8, g_comm, tq::stream());
    if (r != 0) return nccl_fail(r, "ncclAllGather");
    return 0;
}

// Sum of fp32 partial outputs over the ranks (the exchange of a row-parallel shard,
// x_w4_shard mode 1). In place when d_send == d_recv. The sum order is NCCL's, so results
// match the unsharded projection to fp32 rounding, not bit for bit.
int tq_comm_allreduce_sum(const float *d_send, float *d_recv, size_t count) {
    if (!d_send || !d_recv) return -1;
    if (g_world == 1) {
        if (d_send != d_recv) tq_d2d_async(d_recv, d_send, count * sizeof(float));
        return 0;
    }
    if (!g_comm || !g_api.AllReduce) return -3;
    const ncclResult_t r = g_api.AllReduce(d_send, d_recv, count, /*ncclFloat32*/ 7, /*ncclSum*/ 0,
                                           g_comm, tq::stream());
    if (r != 0) return nccl_fail(r, "ncclAllReduce");
    return 0;
}

// ---- fused all-gather over peer memory ------------------------------------------------
// Each rank owns a gathered buffer [world][block] and a flag array int[world] (zeroed),
// both plain cudaMalloc memory; the other ranks map them through CUDA IPC.
int tq_comm_ipc_export(void *d_ptr, void *handle64) {
    if (!d_ptr || !handle64) return -1;
    cudaIpcMemHandle_t h;
    const cudaError_t e = cudaIpcGetMemHandle(&h, d_ptr);
    if (e != cudaSuccess) {
        tq::note_error(e, "cudaIpcGetMemHandle");
        return -2;
    }
    memcpy(handle64, &h, sizeof h);
    return 0;
}

void *tq_comm_ipc_open(const void *handle64) {
    if (!handle64) return nullptr;
    tq::stream();
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof h);
    void *p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        tq::note_error(e, "cudaIpcOpenMemHandle");
        return nullptr;
    }
    return p;
}

void tq_comm_ipc_close(void *p) {
    if (p) cudaIpcCloseMemHandle(p);
}

// bufs[p], flags[p]: rank p's gathered buffer and flag array as addressable from this
// process (its own allocation for p == rank). world <= 8. Steps count from zero again after
// every setup, so this rank's own flag words are cleared here (blocking); the caller must
// put a host barrier between the setup calls of all ranks and the first gathered call, so
// that no rank publishes step 1 into an array its owner has not cleared yet. The size of
// the buffers (2 * world * block floats for the largest gathered call) cannot be checked
// here and is the caller's to guarantee.
int tq_comm_gather_setup(void *const *bufs, void *const *flags, int world, int rank) {
    if (!bufs || !flags || world < 1 || world > 8 || rank < 0 || rank >= world) return -1;
    tq::GatherState &g = g_gather;
    for (int p = 0; p < world; ++p) {
        if (!bufs[p] || !flags[p]) return -1;
        g.buf[p] = static_cast<float *>(bufs[p]);
        g.flag[p] = static_cast<int *>(flags[p]);
    }
    g.world = world;
    g.rank = rank;
    g.step = 0;
    g.pass_syncs = 0;
    tq_dev_zero(g.flag[rank], (size_t)world * sizeof(int));
    if (!g.step_base) g.step_base = static_cast<int *>(tq_dev_alloc(sizeof(int), "exchange.step.base"));
    tq_dev_zero(g.step_base, sizeof(int));
    return 0;
}

// ptrs[p]: rank p's copy of a symmetric buffer (a [T][ld] fp32 matrix every rank holds in
// full) as addressable from this process; slot 0..15 names it in the scatter calls.
int tq_comm_sym_register(int slot, void *const *ptrs) {
    tq::GatherState &g = g_gather;
    if (slot < 0 || slot >= 16 || !ptrs || g.world < 1) return -1;
    for (int p = 0; p < g.world; ++p) {
        if (!ptrs[p]) return -1;
        g.sym[slot][p] = static_cast<float *>(ptrs[p]);
    }
    return 0;
}

// Closes a pass: the step base moves past the exchange points queued since the last call, so
// the same sequence of calls - or a CUDA graph of it - can run again. Every rank must queue
// the same number of exchange points per pass.
int tq_comm_exchange_advance(void) {
    tq::GatherState &g = g_gather;
    if (g.world < 1 || !g.step_base) return -3;
    tq::launch_pdl(exchange_advance_kernel, dim3(1), dim3(32), 0, g.step_base, g.pass_syncs);
    tq::note_error(cudaGetLastError(), "exchange_advance_kernel");
    g.pass_syncs = 0;
    return 0;
}

// Restarts the count of exchange points of a pass without touching the device (used between
// recording a pass into a CUDA graph and issuing the same pass again).
int tq_comm_exchange_rewind(void) {
    g_gather.pass_syncs = 0;
    return 0;
}

int tq_comm_exchange_sync(void) {
    tq::GatherState &g = g_gather;
    if (g.world < 1 || !g.step_base) return -3;
    tq::launch_pdl(exchange_sync_kernel, dim3(1), dim3(32), 0, tq::exchange_point());
    tq::note_error(cudaGetLastError(), "exchange_sync_kernel");
    return 0;
}

// The wait for every rank's slice is part of the gathered GEMM call (its second, one-warp
// kernel); this entry point remains for callers written against the two-call form.
int tq_comm_gather_wait(void) { return g_gather.world < 1 ? -3 : 0; }

int tq_comm_rank(void) { return g_rank; }
int tq_comm_world(void) { return g_world; }

void tq_comm_destroy(void) {
    if (g_comm) {
        tq_sync();
        g_api.CommDestroy(g_comm);
        g_comm = nullptr;
    }
    g_rank = 0;
    g_world = 1;
}

}  // extern "C"
