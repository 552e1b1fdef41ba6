// gemv_e2m3.cu — single-row GEMV straight from the E2M3 fragment payload: the tier a weight
// is in before it is repacked, and the absolute anchor the repacked tiers are gated against
// (x_gemv_qmma's scalar path, xpu/src/kernels_core.cpp:164-233; qwn_w4_check,
// xpu/src/kernels_dpas.cpp:2696-2737).
//
// Arithmetic of the reference: sixteen lanes stride the columns of a row
// (sum += e2m3(code) * block_scale * x[col], separate multiplies and add), then the lane sums
// are added. The reference leaves the order of that last sum to its sub-group reduction; it
// is fixed here to lane 0..15, the order the CPU oracle uses. One half-warp owns a row; the
// kernel is a plain bandwidth kernel (0.75 bytes per weight) and is not on the decode path.
#include "e2m3.cuh"

namespace tq {

namespace {

__global__ void __launch_bounds__(256)
gemv_e2m3_kernel(const uint8_t *__restrict__ payload, const float *__restrict__ bs, int scale_cols, int M,
                 int K, const float *__restrict__ x, const float *__restrict__ residual,
                 float *__restrict__ y) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x * 16 + (threadIdx.x >> 4);
    const int lane = threadIdx.x & 15;
    if (row >= M) return;                       // M % 16 == 0: whole half-warps leave together
    const int Kt = K >> 5, mt = row >> 4;
    const float *brow = bs + (size_t)(mt >> 3) * scale_cols;
    float sum = 0.0f;
    for (int col = lane; col < K; col += 16) {
        const int kt = col >> 5;
        const float cv = e2m3f(e2m3_code_at(payload, Kt, row, col));
        const float w = __fmul_rn(cv, brow[(scale_cols == Kt) ? kt : (kt >> 2)]);
        sum = __fadd_rn(sum, __fmul_rn(w, x[col]));
    }
    // lane sums added 0..15 (every lane forms the same total; lane 0 stores it)
    float total = 0.0f;
    const unsigned half_mask = 0xFFFFu << (threadIdx.x & 16);
#pragma unroll
    for (int l = 0; l < 16; ++l)
        total = __fadd_rn(total, __shfl_sync(half_mask, sum, (threadIdx.x & 16) + l));
    if (lane == 0) y[row] = residual ? __fadd_rn(total, residual[row]) : total;
}

}  // namespace

// Validation and return codes of the reference's scalar tier (kernels_core.cpp:164-187).
int launch_gemv_e2m3(const tq_qmma_weight_t *w, const float *d_x, const float *d_residual, float *d_y) {
    if (!w->d_A || !w->d_block_scale_inv) return -3;
    if (!w->block_scaled || !w->e2m3 || w->row_major || w->word_major || w->e2m1 || w->e2m3_byte)
        return -4;
    if (w->M != w->Mt * 16 || w->K != w->Kt * 32) return -5;
    const int need_rows = (w->M + 127) >> 7, need_cols = (w->Kt + 3) >> 2;
    if (w->scale_rows < need_rows || (w->scale_cols != w->Kt && w->scale_cols < need_cols)) return -6;
    ProfScope prof(w->M, w->K, 1, 6);
    launch_pdl(gemv_e2m3_kernel, dim3(w->Mt), dim3(256), 0, (const uint8_t *)w->d_A,
               (const float *)w->d_block_scale_inv, w->scale_cols, w->M, w->K, d_x, d_residual, d_y);
    TQ_LAUNCH_CHECK("gemv_e2m3_kernel");
    return 0;
}

}  // namespace tq
