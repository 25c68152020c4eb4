/*
 * probe.cu - FP32 peak probe: the denominator of the evaluator's roofline.
 *
 * Population scoring is bound by the FP32 pipe, not by HBM or the tensor cores, so its
 * roofline needs the sustained FP32 instruction rate of the device it runs on.  The probe
 * runs independent FFMA chains (eight per thread, fully unrolled) for a fixed number of
 * iterations on every SM and reports executed lane-instructions per second, i.e.
 * SMs x 128 lanes x sustained clock when the pipe is saturated.  Method after the
 * reference's own roofline note
 * (projects/secant/experiments/astaxanthin_batch_reproduction/CPU_GPU_THROUGHPUT.md:82-108).
 */
#include "../../include/secant_b200.h"

#include <cuda_runtime.h>

namespace {

__global__ void __launch_bounds__(256) ffma_chains(float* sink, int iterations, float a, float b) {
    float v0 = threadIdx.x * 1e-3f, v1 = v0 + 1, v2 = v0 + 2, v3 = v0 + 3, v4 = v0 + 4, v5 = v0 + 5, v6 = v0 + 6, v7 = v0 + 7;
#pragma unroll 1
    for (int i = 0; i < iterations; ++i) {
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            v0 = __fmaf_rn(v0, a, b); v1 = __fmaf_rn(v1, a, b); v2 = __fmaf_rn(v2, a, b); v3 = __fmaf_rn(v3, a, b);
            v4 = __fmaf_rn(v4, a, b); v5 = __fmaf_rn(v5, a, b); v6 = __fmaf_rn(v6, a, b); v7 = __fmaf_rn(v7, a, b);
        }
    }
    sink[blockIdx.x * blockDim.x + threadIdx.x] = ((v0 + v1) + (v2 + v3)) + ((v4 + v5) + (v6 + v7));
}

}  // namespace

extern "C" SecantResult secant_b200_fp32_peak_probe(double seconds_budget, double* lane_instructions_per_second) {
    if (!lane_instructions_per_second) return SECANT_ERROR_INVALID_VALUE;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return SECANT_ERROR_DRIVER_FAILED;
    const int blocks = sms * 8, threads = 256;
    float* sink = nullptr;
    cudaEvent_t start, stop;
    if (cudaMalloc(&sink, (size_t)blocks * threads * sizeof(float)) != cudaSuccess) return SECANT_ERROR_DRIVER_FAILED;
    cudaEventCreate(&start);
    cudaEventCreate(&stop);
    int iterations = 2048;
    double best = 0;
    SecantResult result = SECANT_SUCCESS;
    for (int round = 0; round < 6; ++round) {
        cudaEventRecord(start);
        ffma_chains<<<blocks, threads>>>(sink, iterations, 0.999f, 1e-3f);
        cudaEventRecord(stop);
        if (cudaEventSynchronize(stop) != cudaSuccess) { result = SECANT_ERROR_DRIVER_FAILED; break; }
        float ms = 0;
        cudaEventElapsedTime(&ms, start, stop);
        const double rate = (double)blocks * threads * iterations * 128.0 / (ms * 1e-3);
        if (round >= 2 && rate > best) best = rate; /* first rounds warm the clocks up */
        if (ms * 1e-3 < seconds_budget / 8 && iterations < (1 << 24)) iterations *= 2;
    }
    cudaEventDestroy(start);
    cudaEventDestroy(stop);
    cudaFree(sink);
    *lane_instructions_per_second = best;
    return result;
}
