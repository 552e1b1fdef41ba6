// stream.cuh — device helpers shared by the streaming GEMV/GEMM kernels: mbarrier,
// cp.async copies into shared memory, ldmatrix, the s8 tensor-core MMA and packed
// two-lane fp32 arithmetic (sm_100a).
#pragma once

#include "common.cuh"

namespace tq {

#ifdef __CUDACC__

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

// Makes freshly initialised barriers visible to the async (bulk copy) proxy.
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}

// The same with a suspend-time hint: the thread may stay suspended up to hint_ns while the
// phase is incomplete.
__device__ __forceinline__ uint32_t mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok;
}

// Non-blocking test of a phase (mbarrier.test_wait never suspends the thread).
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}

// Bounded wait: polls until the phase completes or limit_ns of wall clock have passed
// (%globaltimer; the host passes tq::wait_limit_ns(), two seconds unless
// tq_set_wait_limit_ms changed it), then records `code` in *status (first failure wins) and
// returns false. The result is made warp-uniform by the caller.
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// The polling loop is kept out of line: a pipelined kernel has many waits, and a copy of the
// loop with its clock arithmetic at each of them multiplies the kernel's code size until its
// roles evict one another from the instruction cache.
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, int *status, int code,
                                                   uint64_t limit_ns, uint32_t suspend_ns = 0) {
    // mbarrier.try_wait comes back after some tens of clocks while the phase is incomplete, so
    // a warp that polls back to back takes a fifth or more of its scheduler's issue slots
    // from the warps beside it. A single issuing thread that waits beside working warps
    // passes suspend_ns > 0: the wait then carries that suspend-time hint and the thread
    // stays off the scheduler until the phase completes or the time is up (measured a little
    // faster than a nanosleep between polls, which wakes late). The clock is read every 2048
    // polls, so the limit is noticed within 2048 * suspend_ns.
    uint64_t t0 = 0;
    for (uint32_t polls = 1;; ++polls) {
        if (suspend_ns ? mbar_try_wait_hint(bar, parity, suspend_ns) : mbar_try_wait(bar, parity)) return true;
        if ((polls & 2047u) == 0) {
            const uint64_t now = global_timer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_ns) break;
        }
    }
    atomicCAS(status, 0, code);
    return false;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, int *status,
                                                  int code, uint64_t limit_ns) {
    if (mbar_test_wait(bar, parity)) return true;      // the common case in a pipeline that runs ahead
    return mbar_wait_slow(bar, parity, status, code, limit_ns);
}

__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

// 16-byte asynchronous copy global -> shared that bypasses L1 (per-lane; completion is
// tracked with commit/wait groups, so there is nothing to spin on).
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint64_t policy) {
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;" ::"r"(dst),
                 "l"(src), "l"(policy)
                 : "memory");
}
// The same without a cache hint, and a 4-byte copy (through L1), for small operands that
// should stay cached.
__device__ __forceinline__ void cp_async16_plain(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
    asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Four 8x8 b16 matrices = 32 rows of 16 bytes; lane l supplies the address of row l and
// receives word (l & 3) of rows (l >> 2), 8 + (l >> 2), 16 + ..., 24 + ... in r0..r3.
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t &r0, uint32_t &r1,
                                            uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}

// D = A(16 x 32, s8) * B(32 x 8, s8) + C. C is a register quad the caller keeps alive and
// never writes (see make_const_quad), so no per-call moves are needed to build it.
__device__ __forceinline__ void mma_s8_c(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1,
                                         const int (&c)[4]) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c[0]), "r"(c[1]), "r"(c[2]),
          "r"(c[3]));
}

// The same with the accumulator input taken from a previous result (a chain of MMAs that adds
// several k-tiles into one int32 dot).
__device__ __forceinline__ void mma_s8_acc(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                           uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Four registers holding v that the compiler cannot prove equal (so it keeps them as one
// live quad instead of rebuilding it before every MMA).
__device__ __forceinline__ void make_const_quad(int (&c)[4], int v) {
#pragma unroll
    for (int i = 0; i < 4; ++i) asm volatile("mov.b32 %0, %1;" : "=r"(c[i]) : "r"(v));
}

// Four two's-complement nibbles (the low nibble of each byte of w) -> four bytes q+8:
// (w & 0x0F0F0F0F) ^ 0x08080808 as ONE three-input logic op.
__device__ __forceinline__ uint32_t nib_plus8(uint32_t w) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(d) : "r"(w), "r"(0x0F0F0F0Fu), "r"(0x08080808u));
    return d;
}

// ---- packed pairs of fp32 (one instruction for two IEEE round-to-nearest results) ----
typedef unsigned long long f32x2;

__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 v;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
    return v;
}
__device__ __forceinline__ f32x2 pack2i(int lo, int hi) {
    f32x2 v;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "r"(lo), "r"(hi));
    return v;
}
__device__ __forceinline__ void unpack2(f32x2 v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

// acc = a * b + acc, accumulating in place (no copy of the result into acc)
__device__ __forceinline__ void fma2_acc(f32x2 &acc, f32x2 a, f32x2 b) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}

// Integer n with |n| < 2^22 carried as the fp32 bit pattern of 12582912 + n: adding n to
// kMagicBits is an integer add, and (float)bits - 12582912.0f is exactly (float)n.
constexpr int kMagicBits = 0x4B400000;
constexpr float kMagicF = 12582912.0f;

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

#endif  // __CUDACC__

}  // namespace tq
