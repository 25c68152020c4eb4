/*
 * gram.cu - cohort statistics of the static Gram shape.
 *
 * The reference's Gram-statistics kernels keep one cohort of up to 32 programs per kernel and
 * accumulate, over all rows, the programs' sums, their full Gram matrix and their cross sums with
 * the targets (projects/secant/secant.h:478-504, host form projects/secant/s_cpu.c:724-848).  Here
 * the runner materializes the predictions of a batch of cohorts for a range of rows with the
 * population evaluator and this kernel reduces them: one warp per statistic, lanes stride the
 * rows, products rounded before they are added (as the host evaluator does), a fixed-order
 * reduction across the lanes, and one read-modify-write of the statistic by that warp alone - so
 * the result does not depend on scheduling.  Not a hot path of this library: predictions go
 * through memory once.
 */
#include "evaluator.cuh"

#include <cuda_runtime.h>

namespace {

constexpr int kGramWarps = 8;

/* statistics of cohort blockIdx.x: [0, A) sums, [A, A + A*A) Gram matrix row-major,
 * [A + A*A, A + A*A + A*T) cross sums [feature][target]; entries of inactive features stay untouched */
__global__ void __launch_bounds__(kGramWarps * 32)
gram_kernel(const float* __restrict__ predictions, size_t prediction_ld, uint32_t rows, const float* __restrict__ targets,
            size_t targets_ld, uint32_t T, uint32_t A, uint32_t batch_programs, float* statistics, size_t statistics_ld) {
    const uint32_t cohort = blockIdx.x;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t s = blockIdx.y * kGramWarps + (threadIdx.x >> 5);
    const uint32_t width = A * (1u + A + T);
    if (s >= width) return;
    const uint32_t first = cohort * A;
    const uint32_t active = batch_programs - first < A ? batch_programs - first : A;
    uint32_t i, j = 0;
    const float* other = nullptr; /* second factor: another program, a target, or none (plain sum) */
    if (s < A) {
        i = s;
    } else if (s < A + A * A) {
        i = (s - A) / A;
        j = (s - A) % A;
        if (j >= active) return;
        other = predictions + (size_t)(first + j) * prediction_ld;
    } else {
        i = (s - A - A * A) / T;
        other = targets + (size_t)((s - A - A * A) % T) * targets_ld;
    }
    if (i >= active) return;
    const float* mine = predictions + (size_t)(first + i) * prediction_ld;
    float sum = 0.0f;
    for (uint32_t r = lane; r < rows; r += 32u) sum = __fadd_rn(sum, other ? __fmul_rn(mine[r], other[r]) : mine[r]);
#pragma unroll
    for (int d = 16; d; d >>= 1) sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, d));
    if (lane == 0) {
        float* out = statistics + (size_t)cohort * statistics_ld + s;
        *out = __fadd_rn(*out, sum);
    }
}

}  // namespace

namespace sb {

cudaError_t launch_gram(const float* predictions, size_t prediction_ld, uint32_t rows, const float* targets, size_t targets_ld,
                        uint32_t num_targets, uint32_t cohort_size, uint32_t batch_programs, float* statistics, size_t statistics_ld,
                        cudaStream_t stream) {
    const uint32_t cohorts = (batch_programs + cohort_size - 1) / cohort_size;
    const uint32_t width = cohort_size * (1u + cohort_size + num_targets);
    const dim3 grid(cohorts, (width + kGramWarps - 1) / kGramWarps);
    gram_kernel<<<grid, kGramWarps * 32, 0, stream>>>(predictions, prediction_ld, rows, targets, targets_ld, num_targets, cohort_size,
                                                     batch_programs, statistics, statistics_ld);
    note_kernel_launches(1);
    return cudaGetLastError();
}

}  // namespace sb
