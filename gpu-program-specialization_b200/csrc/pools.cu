/*
 * pools.cu - device side of the ODE engine interface beside scoring: the counter-based random
 * pools and the gather of winners' coefficients.
 *
 * Compiled without floating-point contraction (see the Makefile): the reference builds its pool
 * kernels with --fmad=false (projects/odezza/core/o_philox.c:112), and the normal plane is only
 * reproducible sample for sample when the library functions it calls are built the same way.
 *
 * Pools (projects/odezza/core/o_philox.cu:28-58, projects/odezza/core/odezza.h:400-434): sample i
 * of a plane is word (i mod 4) of Philox4x32-10 with key = seed and counter = {i / 4, domain},
 * domain = 2 * stream for the uniform plane and 2 * stream + 1 for the normal one.  A word
 * becomes a uniform value in the open interval (0, 1) as ((word >> 9) + 0.5) * 2^-23.  Normal
 * samples come in pairs (words 0,1 and 2,3) by Box-Muller in float32: radius = sqrt(-2 ln u0),
 * angle = 2 pi u1, values radius cos(angle) and radius sin(angle).  A pool whose first sample is
 * not a multiple of four starts inside a block and drops the leading words.
 */
#include "evaluator.cuh"

#include <cuda_runtime.h>

#include <algorithm>

namespace {

struct Words {
    unsigned x, y, z, w;
};

/* Philox4x32 with ten rounds (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", 2011) */
__device__ Words philox4x32_10(unsigned long long block, unsigned long long seed, unsigned long long domain) {
    Words c{(unsigned)block, (unsigned)(block >> 32), (unsigned)domain, (unsigned)(domain >> 32)};
    unsigned k0 = (unsigned)seed, k1 = (unsigned)(seed >> 32);
    for (int round = 0; round < 10; ++round) {
        const unsigned hi0 = __umulhi(0xd2511f53u, c.x), lo0 = 0xd2511f53u * c.x;
        const unsigned hi1 = __umulhi(0xcd9e8d57u, c.z), lo1 = 0xcd9e8d57u * c.z;
        c = Words{hi1 ^ c.y ^ k0, lo1, hi0 ^ c.w ^ k1, lo0};
        k0 += 0x9e3779b9u;
        k1 += 0xbb67ae85u;
    }
    return c;
}

__device__ __forceinline__ float open_unit(unsigned word) { return ((float)(word >> 9) + 0.5f) * 1.1920928955078125e-7f; }

template <bool NORMAL>
__global__ void __launch_bounds__(256)
fill_pool_kernel(float* __restrict__ out, unsigned long long size, unsigned long long seed, unsigned long long stream_id,
                 unsigned long long base) {
    const unsigned lead = (unsigned)(base % 4);
    const unsigned long long blocks = (lead + size + 3) / 4, first = base / 4;
    for (unsigned long long b = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; b < blocks;
         b += (unsigned long long)gridDim.x * blockDim.x) {
        const Words bits = philox4x32_10(first + b, seed, (stream_id << 1) | (NORMAL ? 1u : 0u));
        float v[4] = {open_unit(bits.x), open_unit(bits.y), open_unit(bits.z), open_unit(bits.w)};
        if (NORMAL) {
            for (int p = 0; p < 4; p += 2) {
                const float radius = sqrtf(-2.0f * logf(v[p]));
                float s, c;
                sincosf(6.2831853071795864769f * v[p + 1], &s, &c);
                v[p] = radius * c;
                v[p + 1] = radius * s;
            }
        }
        for (unsigned j = 0; j < 4; ++j) {
            const unsigned long long at = b * 4 + j; /* position counted from the start of the first block */
            if (at >= lead && at - lead < size) out[at - lead] = v[j];
        }
    }
}

/* projects/odezza/core/o_sampled_constants.cuh:31-43 */
__device__ float sampled_value(const SecantB200SampledParameter* parameters, const float* uniform_pool, const float* normal_pool,
                               unsigned long long pool_size, unsigned long long which, unsigned long long bank) {
    const SecantB200SampledParameter p = parameters[which];
    if (!p.distribution) return p.shift;
    const unsigned long long delta = bank * p.stride;
    if (p.offset >= pool_size || delta >= pool_size - p.offset) return __int_as_float(0x7fc00000);
    const float* pool = p.distribution == 1 ? uniform_pool : p.distribution == 2 ? normal_pool : nullptr;
    if (!pool) return __int_as_float(0x7fc00000);
    const float value = __fadd_rn(__fmul_rn(pool[p.offset + delta], p.scale), p.shift);
    return fminf(p.upper, fmaxf(p.lower, value));
}

/* projects/odezza/core/o_score_reduce.cu:184-196: one value per (winner, constant); a winner whose
 * index lies outside the grid (an unfilled rank) gathers NaN */
__global__ void __launch_bounds__(256) gather_kernel(sb::GatherProblem g) {
    const unsigned long long total = g.entries * g.constants;
    for (unsigned long long i = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (unsigned long long)gridDim.x * blockDim.x) {
        const unsigned long long index = g.winners[i / g.constants].score_index;
        const unsigned c = (unsigned)(i % g.constants);
        float value = __int_as_float(0x7fc00000);
        if (index < g.score_count) {
            const unsigned long long system = index / g.configurations, bank = (index % g.configurations) >> g.toggle_bits;
            value = g.sampled ? sampled_value(g.sampled, g.uniform_pool, g.normal_pool, g.pool_size, system * g.constants + c, bank)
                              : g.banks[(system * g.bank_count + bank) * g.constants + c];
        }
        g.rows[i] = value;
    }
}

}  // namespace

namespace sb {

cudaError_t fill_pool(float* out, unsigned long long size, unsigned long long seed, unsigned long long stream_id,
                      unsigned long long sample_base, bool normal, cudaStream_t stream) {
    const unsigned long long blocks = (sample_base % 4 + size + 3) / 4;
    const unsigned grid = (unsigned)std::min<unsigned long long>((blocks + 255) / 256, 148ull * 32ull);
    if (normal) fill_pool_kernel<true><<<grid ? grid : 1u, 256, 0, stream>>>(out, size, seed, stream_id, sample_base);
    else fill_pool_kernel<false><<<grid ? grid : 1u, 256, 0, stream>>>(out, size, seed, stream_id, sample_base);
    note_kernel_launches(1);
    return cudaGetLastError();
}

cudaError_t gather_constants(const GatherProblem& problem, cudaStream_t stream) {
    const unsigned long long total = problem.entries * problem.constants;
    if (!total) return cudaSuccess;
    const unsigned grid = (unsigned)std::min<unsigned long long>((total + 255) / 256, 148ull * 32ull);
    gather_kernel<<<grid, 256, 0, stream>>>(problem);
    note_kernel_launches(1);
    return cudaGetLastError();
}

}  // namespace sb
