/*
 * reduce.cu - what happens to the score grid after evaluation, on the device:
 * the best configuration of every program and the global top-k of per-program scores.
 *
 * Rules restated from the reference:
 *   - a score is valid when it is finite and >= 0; the best configuration of a program is
 *     its smallest valid score, the lowest configuration index on ties; no valid score
 *     gives {+inf, UINT64_MAX, 0}   (projects/secant-sr/toggle/src/cpu.c:45-67, the NVRTC
 *     `best` kernel of projects/secant-sr/toggle/src/cuda.c:62-88, SRScore layout
 *     projects/secant-sr/secant_sr.h:68-76);
 *   - ranking across programs orders by (score, index) ascending and an invalid score never
 *     beats a valid one (projects/odezza/core/o_score_reduce.cu:36-39).  The reference's
 *     ranking stops at k = 256 and is built on CUB; this one is a tiled bitonic selection
 *     written for any k up to 2048.
 */
#include "../../include/secant_b200.h"
#include "evaluator.cuh"

#include <cuda_runtime.h>
#include <math_constants.h>

#include <algorithm>

namespace {

constexpr int kBestThreads = 128;

struct Candidate {
    float score;
    unsigned long long index;
    unsigned long long valid;
};

__device__ __forceinline__ bool wins(float s, unsigned long long i, float t, unsigned long long j) {
    return s < t || (s == t && i < j);
}

/* one CTA per score vector */
__global__ void __launch_bounds__(kBestThreads)
best_config_kernel(const float* __restrict__ grid, unsigned long long configs, unsigned long long ld, SecantB200Score* out) {
    const float* row = grid + (size_t)blockIdx.x * ld;
    Candidate c{CUDART_INF_F, ~0ull, 0ull};
    for (unsigned long long i = threadIdx.x; i < configs; i += kBestThreads) {
        const float v = row[i];
        if (v >= 0.0f && v < CUDART_INF_F) { /* finite and non-negative; NaN fails both */
            ++c.valid;
            if (wins(v, i, c.score, c.index)) { c.score = v; c.index = i; }
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float s = __shfl_down_sync(0xffffffffu, c.score, o);
        const unsigned long long i = __shfl_down_sync(0xffffffffu, c.index, o);
        c.valid += __shfl_down_sync(0xffffffffu, c.valid, o);
        if (wins(s, i, c.score, c.index)) { c.score = s; c.index = i; }
    }
    __shared__ Candidate partial[kBestThreads / 32];
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kBestThreads / 32; ++w) {
            c.valid += partial[w].valid;
            if (wins(partial[w].score, partial[w].index, c.score, c.index)) { c.score = partial[w].score; c.index = partial[w].index; }
        }
        SecantB200Score r;
        r.sse = c.score; r.reserved = 0; r.configuration = c.index; r.valid_configurations = c.valid;
        out[blockIdx.x] = r;
    }
}

/* ---- top-k --------------------------------------------------------------------------
 * Every score becomes a 64-bit key: high word = the float's bit pattern (monotonic for
 * non-negative floats; invalid scores map to 0xffffffff), low word = the index.  Smaller
 * key = better rank, and keys are unique.  A CTA sorts a tile of 4096 keys in shared memory
 * (bitonic network) and keeps the k smallest; rounds shrink the candidate list by
 * 4096 / k until one tile is left. */
constexpr int kTile = 4096;
constexpr int kSortThreads = 512;

__device__ __forceinline__ unsigned long long score_key(float v, unsigned long long index) {
    unsigned int hi = 0xffffffffu;
    if (v >= 0.0f && v < CUDART_INF_F) hi = v == 0.0f ? 0u : __float_as_uint(v);
    return ((unsigned long long)hi << 32) | (index & 0xffffffffull);
}

__device__ void sort_tile(unsigned long long* keys) {
    for (int size = 2; size <= kTile; size <<= 1)
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            for (int t = threadIdx.x; t < kTile / 2; t += kSortThreads) {
                const int lo = 2 * t - (t & (stride - 1));
                const int hi = lo + stride;
                const bool ascending = (lo & size) == 0;
                const unsigned long long a = keys[lo], b = keys[hi];
                if ((a > b) == ascending) { keys[lo] = b; keys[hi] = a; }
            }
        }
    __syncthreads();
}

/* first round: tiles of raw scores -> k best keys per tile */
__global__ void __launch_bounds__(kSortThreads)
topk_first_kernel(const float* __restrict__ scores, unsigned long long count, unsigned int k, unsigned long long* out) {
    __shared__ unsigned long long keys[kTile];
    const unsigned long long base = (unsigned long long)blockIdx.x * kTile;
    for (int t = threadIdx.x; t < kTile; t += kSortThreads) {
        const unsigned long long i = base + t;
        keys[t] = i < count ? score_key(scores[i], i) : ~0ull;
    }
    sort_tile(keys);
    for (unsigned int t = threadIdx.x; t < k; t += kSortThreads) out[(size_t)blockIdx.x * k + t] = keys[t];
}

/* later rounds: tiles of candidate keys -> k best keys per tile */
__global__ void __launch_bounds__(kSortThreads)
topk_merge_kernel(const unsigned long long* __restrict__ in, unsigned long long count, unsigned int k, unsigned long long* out) {
    __shared__ unsigned long long keys[kTile];
    const unsigned long long base = (unsigned long long)blockIdx.x * kTile;
    for (int t = threadIdx.x; t < kTile; t += kSortThreads) keys[t] = base + t < count ? in[base + t] : ~0ull;
    sort_tile(keys);
    for (unsigned int t = threadIdx.x; t < k; t += kSortThreads) out[(size_t)blockIdx.x * k + t] = keys[t];
}

__global__ void topk_emit_kernel(const unsigned long long* __restrict__ keys, const float* __restrict__ scores,
                                 unsigned long long count, unsigned int k, unsigned long long* indices, float* values) {
    const unsigned int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= k) return;
    const unsigned long long key = keys[t];
    const bool present = t < count && key != ~0ull;
    const unsigned long long index = key & 0xffffffffull;
    indices[t] = present ? index : ~0ull;
    if (values) values[t] = present ? scores[index] : CUDART_NAN_F;
}

size_t tiles_of(unsigned long long count) { return (size_t)((count + kTile - 1) / kTile); }

/* Fixed scratch of secant_b200_topk_static(): enough for 1,048,576 scores and k = 1024
 * (256 first-round tiles x 1024 keys, plus 64 x 1024 for the second round), 2.5 MiB.  The
 * array lives in every device that loads this library, for the life of the process. */
constexpr size_t kStaticMaxCount = 1u << 20;
constexpr size_t kStaticMaxK = 1024;
constexpr size_t kStaticWords = (kStaticMaxCount / kTile) * kStaticMaxK + ((kStaticMaxCount / kTile) * kStaticMaxK / kTile) * kStaticMaxK;
static __device__ __align__(256) unsigned long long g_topk_static_scratch[kStaticWords];

/* ---- grouped top-k of a [system][configuration] score grid ----------------------------------
 * Rules of the reference engine's reducer (projects/odezza/core/o_score_reduce.cu:36-62,
 * projects/odezza/core/odezza.h:438-486): a score is valid when 0 <= score < FLT_MAX (NaN,
 * infinities, FLT_MAX and negatives are not; -0 is, and orders as +0); winners are ordered by
 * (score, flat index); unfilled ranks are {FLT_MAX, 0, UINT64_MAX}; counts are valid, invalid and
 * finite-negative scores of the group.  Groups: 0 = system, 1 = (system, permutation) over banks,
 * 2 = one global group.  One CTA per group keeps the best k keys in shared memory and merges the
 * group's scores into them 1024 - k at a time with a bitonic sort (the reference sorts with CUB). */
constexpr int kGroupThreads = 256, kGroupKeys = 1024;

__device__ __forceinline__ unsigned long long group_flat_index(unsigned long long group, unsigned long long e, unsigned long long configs,
                                                              unsigned long long perms, unsigned mode) {
    return mode == 2 ? e : mode == 0 ? group * configs + e : (group / perms) * configs + e * perms + group % perms;
}

/* Keeps the k smallest of n keys in keys[0..k), ascending.  Candidates arrive kGroupKeys - k at a
 * time behind the current best k and the whole array is sorted; a batch in which nothing beats
 * the current k-th key is dropped without sorting.  Keys are unique, so the result does not depend
 * on how the candidates were batched or split over CTAs. */
template <class Fetch>
__device__ void select_smallest(unsigned long long* keys, unsigned k, unsigned long long n, Fetch& fetch) {
    const unsigned fresh = kGroupKeys - k;
    for (int i = threadIdx.x; i < kGroupKeys; i += kGroupThreads) keys[i] = ~0ull;
    for (unsigned long long base = 0; base < n; base += fresh) {
        __syncthreads();
        const unsigned long long bar = keys[k - 1];
        int beats = 0;
        for (unsigned i = threadIdx.x; i < fresh; i += kGroupThreads) {
            const unsigned long long e = base + i;
            const unsigned long long key = e < n ? fetch(e) : ~0ull;
            keys[k + i] = key;
            beats |= key < bar;
        }
        if (!__syncthreads_or(beats)) continue;
        for (unsigned size = 2; size <= kGroupKeys; size <<= 1)
            for (unsigned stride = size >> 1; stride > 0; stride >>= 1) {
                __syncthreads();
                for (unsigned t = threadIdx.x; t < kGroupKeys / 2; t += kGroupThreads) {
                    const unsigned lo = 2 * t - (t & (stride - 1)), hi = lo + stride;
                    const bool up = (lo & size) == 0;
                    const unsigned long long a = keys[lo], b = keys[hi];
                    if ((a > b) == up) { keys[lo] = b; keys[hi] = a; }
                }
            }
    }
    __syncthreads();
}

struct RawScores { /* element of a group -> key, tallying validity on the way */
    const float* scores;
    unsigned long long group, first, configs, perms;
    unsigned mode;
    unsigned long long valid, invalid, negative;
    __device__ unsigned long long operator()(unsigned long long e) {
        const unsigned long long element = first + e;
        const float f = scores[group_flat_index(group, element, configs, perms, mode)];
        if (f >= 0.0f && f < 3.402823466e+38f) {
            ++valid;
            return ((unsigned long long)__float_as_uint(f == 0.0f ? 0.0f : f) << 32) | (unsigned)element;
        }
        ++invalid;
        negative += (f < 0.0f && f > -CUDART_INF_F) ? 1 : 0;
        return ~0ull;
    }
};

struct StoredKeys {
    const unsigned long long* keys;
    __device__ unsigned long long operator()(unsigned long long e) const { return keys[e]; }
};

__device__ void emit_winners(const unsigned long long* keys, const float* scores, unsigned long long group, unsigned long long configs,
                             unsigned long long perms, unsigned mode, unsigned k, SecantB200Winner* winners) {
    for (unsigned rank = threadIdx.x; rank < k; rank += kGroupThreads) {
        const unsigned long long key = keys[rank];
        SecantB200Winner w{3.402823466e+38f, 0u, ~0ull};
        if (key != ~0ull) {
            w.score_index = group_flat_index(group, key & 0xffffffffull, configs, perms, mode);
            w.mse = scores[w.score_index]; /* the original bits, signed zero included */
        }
        winners[group * k + rank] = w;
    }
}

/* grid = groups x segments.  With one segment per group the CTA writes the group's winners and
 * counts; otherwise its best k keys and its tallies go to part_keys / part_counts for the merge. */
__global__ void __launch_bounds__(kGroupThreads)
grouped_topk_kernel(const float* __restrict__ scores, unsigned long long elements, unsigned long long configs, unsigned long long perms,
                    unsigned mode, unsigned k, unsigned segments, unsigned long long span, SecantB200Winner* winners,
                    SecantB200ScoreCounts* counts, unsigned long long* part_keys, SecantB200ScoreCounts* part_counts) {
    __shared__ unsigned long long keys[kGroupKeys];
    __shared__ unsigned long long tally[3];
    const unsigned long long group = blockIdx.x / segments;
    const unsigned segment = blockIdx.x % segments;
    const unsigned long long first = (unsigned long long)segment * span;
    const unsigned long long n = first >= elements ? 0ull : (elements - first < span ? elements - first : span);
    if (threadIdx.x < 3) tally[threadIdx.x] = 0;
    RawScores fetch{scores, group, first, configs, perms, mode, 0ull, 0ull, 0ull};
    select_smallest(keys, k, n, fetch);
    atomicAdd(&tally[0], fetch.valid); atomicAdd(&tally[1], fetch.invalid); atomicAdd(&tally[2], fetch.negative);
    __syncthreads();
    if (segments == 1) {
        emit_winners(keys, scores, group, configs, perms, mode, k, winners);
        if (threadIdx.x == 0) counts[group] = SecantB200ScoreCounts{tally[0], tally[1], tally[2]};
    } else {
        for (unsigned rank = threadIdx.x; rank < k; rank += kGroupThreads) part_keys[(size_t)blockIdx.x * k + rank] = keys[rank];
        if (threadIdx.x == 0) part_counts[blockIdx.x] = SecantB200ScoreCounts{tally[0], tally[1], tally[2]};
    }
}

/* one CTA per group: the best k of its segments' keys, and the sum of their tallies */
__global__ void __launch_bounds__(kGroupThreads)
grouped_merge_kernel(const float* __restrict__ scores, unsigned long long configs, unsigned long long perms, unsigned mode, unsigned k,
                     unsigned segments, const unsigned long long* __restrict__ part_keys, const SecantB200ScoreCounts* __restrict__ part_counts,
                     SecantB200Winner* winners, SecantB200ScoreCounts* counts) {
    __shared__ unsigned long long keys[kGroupKeys];
    __shared__ unsigned long long tally[3];
    const unsigned long long group = blockIdx.x;
    if (threadIdx.x < 3) tally[threadIdx.x] = 0;
    StoredKeys fetch{part_keys + (size_t)group * segments * k};
    select_smallest(keys, k, (unsigned long long)segments * k, fetch);
    unsigned long long valid = 0, invalid = 0, negative = 0;
    for (unsigned s = threadIdx.x; s < segments; s += kGroupThreads) {
        const SecantB200ScoreCounts c = part_counts[(size_t)group * segments + s];
        valid += c.valid; invalid += c.invalid; negative += c.negative;
    }
    atomicAdd(&tally[0], valid); atomicAdd(&tally[1], invalid); atomicAdd(&tally[2], negative);
    __syncthreads();
    emit_winners(keys, scores, group, configs, perms, mode, k, winners);
    if (threadIdx.x == 0) counts[group] = SecantB200ScoreCounts{tally[0], tally[1], tally[2]};
}

}  // namespace

/* Runs the selection rounds; `scratch` must hold secant_b200_topk_scratch_elements(count, k)
 * 64-bit words.  Shared by the allocating and the caller-provided-scratch entry points. */
static cudaError_t topk_rounds(const float* scores, unsigned long long count, unsigned int k, unsigned long long* scratch,
                               unsigned long long* indices, float* values, cudaStream_t stream) {
    size_t tiles = tiles_of(count);
    unsigned long long* cur = scratch;
    unsigned long long* nxt = scratch + tiles * k;
    topk_first_kernel<<<(unsigned)tiles, kSortThreads, 0, stream>>>(scores, count, k, cur);
    unsigned launched = 2; /* first + emit */
    unsigned long long have = (unsigned long long)tiles * k;
    while (tiles > 1) {
        tiles = tiles_of(have);
        topk_merge_kernel<<<(unsigned)tiles, kSortThreads, 0, stream>>>(cur, have, k, nxt);
        ++launched;
        have = (unsigned long long)tiles * k;
        unsigned long long* t = cur; cur = nxt; nxt = t;
    }
    topk_emit_kernel<<<(k + 255) / 256, 256, 0, stream>>>(cur, scores, count, k, indices, values);
    sb::note_kernel_launches(launched);
    return cudaGetLastError();
}

/* Grouped top-k with an optional scratch area.  Large groups are cut into segments scored by
 * separate CTAs when `scratch` (8-byte aligned device memory of scratch_bytes) has room for their
 * partial results: segments x (k keys + one tally) per group; without it one CTA walks each group. */
SecantResult sb::grouped_topk(uintptr_t scores, size_t num_systems, size_t num_banks, uint32_t toggle_bits, uint32_t grouping, uint32_t k,
                              uintptr_t winners, uintptr_t counts, uintptr_t scratch, size_t scratch_bytes, cudaStream_t stream) {
    if (!scores || !winners || !counts || scores % 4 || winners % 8 || counts % 8 || scratch % 8 || !num_systems || !num_banks ||
        toggle_bits > 32 || grouping > SECANT_B200_GROUP_GLOBAL || !k || k > 256)
        return SECANT_ERROR_INVALID_VALUE;
    const unsigned long long perms = 1ull << toggle_bits;
    if (num_banks > (~0ull >> toggle_bits) || (num_banks << toggle_bits) > ~0ull / num_systems) return SECANT_ERROR_OVERFLOW;
    const unsigned long long configs = (unsigned long long)num_banks << toggle_bits;
    unsigned long long groups, elements;
    if (grouping == SECANT_B200_GROUP_BY_SYSTEM) { groups = num_systems; elements = configs; }
    else if (grouping == SECANT_B200_GROUP_BY_SYSTEM_PERMUTATION) { groups = num_systems * perms; elements = num_banks; }
    else { groups = 1; elements = configs * num_systems; }
    if (groups > 0x7fffffffull || elements > 0xffffffffull) return SECANT_ERROR_OVERFLOW; /* grid size, 32-bit key index */
    /* segments: enough CTAs for four per SM, at least 4096 elements each, and no more than the scratch holds */
    unsigned long long segments = 1;
    if (scratch && groups < 592) {
        segments = std::min<unsigned long long>((592 + groups - 1) / groups, (elements + 4095) / 4096);
        const unsigned long long per_segment = (unsigned long long)k * 8 + sizeof(SecantB200ScoreCounts);
        segments = std::min<unsigned long long>(segments, scratch_bytes / per_segment / groups);
        if (segments < 2) segments = 1;
    }
    const unsigned long long span = (elements + segments - 1) / segments;
    unsigned long long* part_keys = reinterpret_cast<unsigned long long*>(scratch);
    SecantB200ScoreCounts* part_counts = reinterpret_cast<SecantB200ScoreCounts*>(part_keys + groups * segments * k);
    const float* grid = reinterpret_cast<const float*>(scores);
    grouped_topk_kernel<<<(unsigned)(groups * segments), kGroupThreads, 0, stream>>>(
        grid, elements, configs, perms, grouping, k, (unsigned)segments, span, reinterpret_cast<SecantB200Winner*>(winners),
        reinterpret_cast<SecantB200ScoreCounts*>(counts), part_keys, part_counts);
    unsigned launched = 1;
    if (segments > 1) {
        grouped_merge_kernel<<<(unsigned)groups, kGroupThreads, 0, stream>>>(grid, configs, perms, grouping, k, (unsigned)segments, part_keys,
                                                                             part_counts, reinterpret_cast<SecantB200Winner*>(winners),
                                                                             reinterpret_cast<SecantB200ScoreCounts*>(counts));
        ++launched;
    }
    sb::note_kernel_launches(launched);
    return cudaGetLastError() == cudaSuccess ? SECANT_SUCCESS : SECANT_ERROR_DRIVER_FAILED;
}

extern "C" {

SecantResult secant_b200_grouped_topk(uintptr_t scores, size_t num_systems, size_t num_banks, uint32_t toggle_bits, uint32_t grouping,
                                      uint32_t k, uintptr_t winners, uintptr_t counts, void* stream) {
    return sb::grouped_topk(scores, num_systems, num_banks, toggle_bits, grouping, k, winners, counts, 0, 0, (cudaStream_t)stream);
}

size_t secant_b200_topk_scratch_elements(size_t count, size_t k) {
    const size_t first = tiles_of(count) * k;
    return first + tiles_of(first) * k; /* ping + pong; later rounds only shrink */
}

SecantResult secant_b200_best_config(uintptr_t scores, size_t num_vectors, size_t num_configurations, size_t leading_dimension,
                                     uintptr_t best_out, void* stream) {
    if (!scores || !best_out || !num_vectors || !num_configurations || leading_dimension < num_configurations ||
        num_vectors > 0x7fffffffull || scores % 4 || best_out % 8)
        return SECANT_ERROR_INVALID_VALUE;
    best_config_kernel<<<(unsigned)num_vectors, kBestThreads, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const float*>(scores), num_configurations, leading_dimension, reinterpret_cast<SecantB200Score*>(best_out));
    sb::note_kernel_launches(1);
    return cudaGetLastError() == cudaSuccess ? SECANT_SUCCESS : SECANT_ERROR_DRIVER_FAILED;
}

/* Device address of the static scratch on the current device.  The symbol name is only a
 * host-side handle; the address a kernel may use has to be asked for once per device, with
 * that device current. */
static cudaError_t static_scratch_address(unsigned long long** address) {
    constexpr int kMaxDevices = 64;
    static unsigned long long* table[kMaxDevices] = {nullptr};
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
    unsigned long long* known = __atomic_load_n(&table[device], __ATOMIC_ACQUIRE);
    if (!known) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_topk_static_scratch);
        if (e != cudaSuccess) return e;
        known = static_cast<unsigned long long*>(p);
        __atomic_store_n(&table[device], known, __ATOMIC_RELEASE); /* every thread resolves the same address */
    }
    *address = known;
    return cudaSuccess;
}

SecantResult secant_b200_topk_static(uintptr_t scores, size_t count, size_t k, uintptr_t indices_out, uintptr_t scores_out,
                                     void* stream) {
    if (!scores || !indices_out || !count || !k || scores % 4 || indices_out % 8 || scores_out % 4) return SECANT_ERROR_INVALID_VALUE;
    if (count > kStaticMaxCount || k > kStaticMaxK) return SECANT_ERROR_INSUFFICIENT_BUFFER; /* beyond the fixed scratch */
    if (secant_b200_topk_scratch_elements(count, k) > kStaticWords) return SECANT_ERROR_INSUFFICIENT_BUFFER;
    unsigned long long* scratch = nullptr;
    if (static_scratch_address(&scratch) != cudaSuccess) return SECANT_ERROR_DRIVER_FAILED;
    /* every round writes the keys it later reads, so nothing in the shared array needs clearing */
    const cudaError_t e = topk_rounds(reinterpret_cast<const float*>(scores), count, (unsigned)k, scratch,
                                      reinterpret_cast<unsigned long long*>(indices_out), reinterpret_cast<float*>(scores_out),
                                      (cudaStream_t)stream);
    return e == cudaSuccess ? SECANT_SUCCESS : SECANT_ERROR_DRIVER_FAILED;
}

SecantResult secant_b200_topk(uintptr_t scores, size_t count, size_t k, uintptr_t indices_out, uintptr_t scores_out, void* stream) {
    if (!scores || !indices_out || !count || !k || k > 2048 || count > 0xffffffffull || scores % 4 || indices_out % 8 || scores_out % 4)
        return SECANT_ERROR_INVALID_VALUE;
    unsigned long long* scratch = nullptr;
    const size_t words = secant_b200_topk_scratch_elements(count, k);
    if (cudaMallocAsync(&scratch, words * sizeof(unsigned long long), (cudaStream_t)stream) != cudaSuccess) return SECANT_ERROR_ALLOCATION_FAILED;
    cudaError_t e = topk_rounds(reinterpret_cast<const float*>(scores), count, (unsigned)k, scratch,
                                reinterpret_cast<unsigned long long*>(indices_out), reinterpret_cast<float*>(scores_out),
                                (cudaStream_t)stream);
    const cudaError_t f = cudaFreeAsync(scratch, (cudaStream_t)stream);
    if (e == cudaSuccess) e = f;
    return e == cudaSuccess ? SECANT_SUCCESS : SECANT_ERROR_DRIVER_FAILED;
}

}  // extern "C"
