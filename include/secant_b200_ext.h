/*
 * secant_b200_ext.h - entry points and descriptor fields this library adds to the
 * reference C API.  Included by secant_b200.h; do not include it on its own.
 *
 * None of these has a counterpart in the reference header.  They exist because the
 * population-scoring workloads this library is built for need things the reference API
 * cannot express (per-program coefficient banks, a runner without the NVRTC round trip,
 * device-side best-configuration and top-k reductions, RK4 rollout scoring).
 */
#ifndef SECANT_B200_EXT_H_INCLUDED
#define SECANT_B200_EXT_H_INCLUDED

/*
 * Toggle-SSE run with appended optional fields.  The reference descriptor rule
 * (secant.h:49-56) allows a larger struct_size whose extra fields default to zero, so this
 * struct is passed to secant_cubin_runner_run()/run_batch() like the plain one, with
 * base.header.struct_size = sizeof(SecantB200ToggleSSERun).
 *
 *  program_bank_stride  elements between the coefficient tables of consecutive programs.
 *                       0 (default) = one [bank][slot] table shared by every program,
 *                       which is the reference behaviour (secant.h:506-514).  Non-zero =
 *                       program a reads bank b, slot k at
 *                       constants.address[a*program_bank_stride + b*bank_stride + k].
 *  first_program_index  added to the program index when addressing per-program banks,
 *                       so that a rank holding a slice of a population can point at the
 *                       whole table.  Ignored when program_bank_stride is 0.
 */
typedef struct SecantB200ToggleSSERun {
    SecantCubinToggleSSERun base;
    size_t program_bank_stride;
    size_t first_program_index;
} SecantB200ToggleSSERun;

static inline SecantB200ToggleSSERun secant_b200_toggle_sse_run_init(void) {
    SECANT_B200_ZERO_INIT(SecantB200ToggleSSERun, v);
    v.base = secant_cubin_toggle_sse_run_init();
    v.base.header.struct_size = (uint32_t)sizeof(v);
    return v;
}

/*
 * Creates a runner straight from a recipe, without generating source, compiling it and
 * inspecting a binary first.  Equivalent to the reference sequence source_write -> NVRTC ->
 * plan_init -> runner_create (projects/secant/tests/toggle_cuda_test.c:65-115) with the
 * compile step removed; the runner owns its plan.  Same context rules as
 * secant_cubin_runner_create: the CUDA context current at creation must be current for
 * every run and for destroy.
 */
SECANT_DEC SecantResult secant_b200_runner_create(const SecantCubinRecipeHeader* recipe,
                                                  const SecantCubinRunnerOptions* options,
                                                  SecantCubinRunner* runner_ret);

/*
 * Device-resident populations.  secant_b200_population_create() validates, encodes and
 * uploads a program set once; secant_b200_population_run() then scores it against any
 * run request of the runner's shape (the request's `programs` field is ignored) without
 * re-reading, re-encoding or re-uploading the programs -- the case of a search loop that
 * refits coefficient banks or swaps data for an unchanged population
 * (projects/secant-sr/toggle/src/cuda.c:368-477 scores the same programs with new banks).
 * toggle_bits is the smallest toggle_bits any later run will use.  A population belongs
 * to the runner it was created from and must be destroyed before that runner.
 */
typedef struct SecantB200PopulationImpl* SecantB200Population;
SECANT_DEC SecantResult secant_b200_population_create(SecantCubinRunner runner, const SecantAstProgramSet* programs,
                                                      uint32_t toggle_bits, SecantB200Population* population_ret);
SECANT_DEC SecantResult secant_b200_population_run(SecantB200Population population, const SecantCubinRunHeader* run,
                                                   SecantRunnerStats* stats_ret);
SECANT_DEC SecantResult secant_b200_population_run_batch(SecantB200Population population,
                                                         const SecantCubinRunHeader* const* runs, size_t num_runs,
                                                         SecantRunnerStats* stats_ret);
/* Arithmetic nodes (after routine inlining) summed over the population, for work accounting. */
SECANT_DEC uint64_t secant_b200_population_num_ops(SecantB200Population population);
SECANT_DEC SecantResult secant_b200_population_destroy(SecantB200Population population);

/*
 * Arithmetic of division and of the transcendental functions.
 *   ACCURATE (default): IEEE division, sin/cos/exp/log within 2-2.5 ulp of the correctly rounded
 *       result over the whole float range - the numerics of the reference HOST evaluator
 *       (projects/secant/s_cpu.c:329-352), which the parity tests are held to.
 *   FAST: special-function-unit approximations (__sinf, __expf, __logf, __fdividef, ...), the
 *       lowerings the reference's GPU kernels are compiled with (--use_fast_math,
 *       projects/secant/tests/toggle_cuda_test.c:74).  Sums agree with the host evaluator to
 *       the reference GPU test's tolerance, 2e-4 * (1 + |sum|), on well-conditioned programs.
 * Add, subtract, multiply, min, max, negate and abs are exact in both modes.  Returns
 * INVALID_STATE while a run is in flight.  The RK4 entry point always uses ACCURATE.
 */
enum { SECANT_B200_MATH_ACCURATE = 0, SECANT_B200_MATH_FAST = 1 };
SECANT_DEC SecantResult secant_b200_runner_set_math(SecantCubinRunner runner, uint32_t mode);

/*
 * Scratch memory of a run.  The evaluator splits the rows of a run across thread blocks, keeps one
 * partial sum per (row split, program, target, configuration) in device memory of its own and adds
 * the splits of a bin in a fixed order, so a score never depends on how the blocks were scheduled
 * (the reference adds with atomics, projects/secant/s_cubin_generate_toggle_sse.c:378-381).  The
 * buffer belongs to the runner (one per launch stream, grown on demand, kept between runs,
 * released by destroy).  More row splits mean more, shorter blocks - better balance when there are
 * few programs - and more scratch.  This call caps the scratch of one launch at `bytes`; 0 restores
 * the default of 1 GiB.  A launch whose single-split scratch alone exceeds the cap still runs, with
 * one split.  Returns INVALID_STATE while a run is in flight.
 */
SECANT_DEC SecantResult secant_b200_runner_set_scratch_limit(SecantCubinRunner runner, size_t bytes);

/*
 * RK4 rollout scoring: the population-evaluation path with the program inside an integration
 * loop.  num_systems candidate systems of num_states (<= 8) right-hand-side programs each
 * (programs.asts is system-major: system i, state s at index i*num_states + s; COLUMN s reads
 * state s, BANK_CONSTANT k coefficient k) are integrated with fixed-step RK4 from the first
 * point of every reference trajectory and scored by mean squared error against it.
 * Semantics of the reference engine's scoring kernel
 * (projects/odezza/core/o_generate_scoring_cuda.c:494-588): h = (times[k]-times[k-1]) /
 * steps_per_observation, explicit fmaf in every stage update, score = FLT_MAX (never NaN) as
 * soon as a time step, an initial state, an integrated state or the error sum is not finite.
 *   reference   [state][trajectory * points_per_trajectory + point], device, f32
 *   times       device float[points_per_trajectory], shared by all trajectories
 * Ragged form, the reference engine's launch layout (projects/odezza/core/odezza.h:275-289): when
 * trajectory_offsets is non-zero it addresses device uint32[num_trajectories + 1] partitioning
 * total_points concatenated points (first point of a trajectory = its initial condition),
 * times is device float[total_points] (strictly increasing inside a trajectory, steps may be
 * irregular), reference is [state][concatenated point] and points_per_trajectory is ignored.
 * Offsets that do not start at zero, increase strictly and end at total_points, a non-finite
 * time or reference value anywhere, or no scored value at all give FLT_MAX in every score.  With
 * allow_missing_observations a NaN reference value after a trajectory's first point is an
 * unobserved value: it is skipped, and the mean divides by the values that were observed.
 *   constants   [system][bank][slot]; system_bank_stride 0 = num_banks * bank_stride
 *   output      [system][configuration], configuration = bank * 2^toggle_bits + permutation
 * Blocking; uses the current CUDA device and context; runs on the call's own streams, ordered after
 * the work the caller has queued on the default stream.  Programs are validated before anything is
 * launched; a structural error found later, while a chunk of systems is being encoded, ends the call
 * with its code after earlier chunks may have written their scores.  Transcendental opcodes are allowed in
 * right-hand sides, but only exactly rounded operations (add, sub, mul, div, fma, sqrt, neg,
 * abs, min, max) reproduce a host rollout bit for bit, which chaotic systems need.
 */
/* A coefficient drawn from a shared pool instead of an explicit bank table: layout and rule of the
 * reference engine's OdezzaSampledParameter (projects/odezza/core/odezza.h:304-311,
 * projects/odezza/core/o_sampled_constants_source.h:32-44).  distribution 0: the value is `shift`
 * for every bank; 1 / 2: pool = uniform / normal, value = clamp(pool[offset + bank * stride] * scale
 * + shift, lower, upper) with the multiply and the add rounded separately; an index outside the
 * pool or another distribution gives NaN (and with it an invalid score). */
typedef struct SecantB200SampledParameter {
    uint64_t offset;
    uint32_t stride, distribution;
    float scale, shift, lower, upper;
} SecantB200SampledParameter;

typedef struct SecantB200Rk4Run {
    uint32_t struct_size, version, flags, reserved;   /* version = SECANT_CUBIN_RUN_VERSION_3 */
    SecantAstProgramSet programs;
    size_t num_systems, num_states, num_constants;
    SecantDeviceConstantBanks constants;
    size_t system_bank_stride, num_banks;
    uint32_t toggle_bits, reserved2;
    SecantDeviceMatrixF32 reference;
    size_t num_trajectories, points_per_trajectory;
    uintptr_t times;
    size_t steps_per_observation;
    SecantDeviceMatrixF32 output;
    /* appended fields; a struct_size that ends before them, or zeros, select the uniform form */
    uintptr_t trajectory_offsets;
    size_t total_points;
    uint32_t allow_missing_observations, reserved3;
    /* non-zero sampled_parameters: device SecantB200SampledParameter[num_systems][num_constants];
     * `constants` is then unused and may be zero; the pools hold rng_pool_size floats each */
    uintptr_t sampled_parameters, uniform_pool, normal_pool;
    uint64_t rng_pool_size;
    /* optional device uint64 (8-byte aligned), incremented by the number of (trajectory, observation
     * interval) pairs that were integrated.  A candidate whose score is already FLT_MAX (a state or a
     * step became non-finite) is not integrated further, so this is what the call actually computed;
     * the full count is num_systems * configurations * scored points. */
    uintptr_t integrated_intervals;
} SecantB200Rk4Run;
SECANT_DEC SecantResult secant_b200_rk4_score(const SecantB200Rk4Run* run);
/* The call's record buffers come from a stream-ordered memory pool of the library's own (one per
 * device, created on first use), which keeps what the largest call so far needed: allocating and
 * freeing them with cudaMalloc/cudaFree cost 2 to 300 ms per call.  This returns the cached memory of
 * every device to the driver; buffers of calls in flight are not touched. */
SECANT_DEC SecantResult secant_b200_release_cached_memory(void);

/*
 * Grouped top-k over a score grid [system][configuration] (contiguous, configuration = bank *
 * 2^toggle_bits + permutation), the reduction of the reference engine
 * (projects/odezza/core/odezza.h:438-486, projects/odezza/core/o_score_reduce.cu:36-62):
 * grouping 0 = one group per system, 1 = one per (system, permutation) ranking the banks,
 * 2 = one global group.  A score is valid when 0 <= score < FLT_MAX; winners[group][k] are ordered
 * by (score, flat index) and carry the original score bits and the flat element index; unfilled
 * ranks are {FLT_MAX, 0, UINT64_MAX}; counts[group] = valid, invalid and finite-negative scores.
 * 1 <= k <= 256.  winners and counts are device addresses, 8-byte aligned.  Asynchronous on
 * `stream`; no allocation.
 */
typedef struct SecantB200Winner {
    float mse;
    uint32_t reserved;
    uint64_t score_index;
} SecantB200Winner;
typedef struct SecantB200ScoreCounts {
    uint64_t valid, invalid, negative;
} SecantB200ScoreCounts;
enum { SECANT_B200_GROUP_BY_SYSTEM = 0, SECANT_B200_GROUP_BY_SYSTEM_PERMUTATION = 1, SECANT_B200_GROUP_GLOBAL = 2 };
SECANT_DEC SecantResult secant_b200_grouped_topk(uintptr_t scores, size_t num_systems, size_t num_banks, uint32_t toggle_bits,
                                                 uint32_t grouping, uint32_t k, uintptr_t winners, uintptr_t counts, void* stream);

/*
 * Best configuration of every score vector, on the device.  `scores` is [vector][configuration]
 * float32 with `leading_dimension` elements between vectors (for a toggle-SSE grid with one
 * target: vector = program).  A score is valid when finite and >= 0; the winner is the
 * smallest valid score, lowest configuration on ties; no valid score gives
 * {+inf, UINT64_MAX, 0}.  Layout and rule of the reference consumer's SRScore
 * (projects/secant-sr/secant_sr.h:68-76, projects/secant-sr/toggle/src/cpu.c:45-67).
 * Asynchronous on `stream` (a cudaStream_t, NULL = default stream).
 */
typedef struct SecantB200Score {
    float sse;
    uint32_t reserved;
    uint64_t configuration;
    uint64_t valid_configurations;
} SecantB200Score;
SECANT_DEC SecantResult secant_b200_best_config(uintptr_t scores, size_t num_vectors, size_t num_configurations,
                                                size_t leading_dimension, uintptr_t best_out, void* stream);

/*
 * Global top-k of `count` float32 scores (count < 2^32, k <= 2048): writes the indices of the
 * k best scores to indices_out (uint64[k]) and, when scores_out is non-zero, their values
 * (float[k]).  Order: valid scores (finite, >= 0) before invalid ones, score ascending,
 * index ascending (projects/odezza/core/o_score_reduce.cu:36-39).  Slots beyond `count`
 * receive UINT64_MAX / NaN.  Uses a stream-ordered temporary allocation of
 * secant_b200_topk_scratch_elements(count, k) 64-bit words.  Asynchronous on `stream`.
 */
SECANT_DEC SecantResult secant_b200_topk(uintptr_t scores, size_t count, size_t k, uintptr_t indices_out,
                                         uintptr_t scores_out, void* stream);
SECANT_DEC size_t secant_b200_topk_scratch_elements(size_t count, size_t k);

/*
 * secant_b200_topk() for callers that must not allocate.  No counterpart in the reference.
 *
 * Some hosts cannot let a library call cudaMalloc: a process that has handed all device
 * memory to its own pool (a further allocation fails or fragments the pool), or a steady-
 * state scoring loop that cannot afford the device-wide synchronisation and latency an
 * allocation or free may cost.  This variant runs the same kernels as secant_b200_topk()
 * but keeps its intermediate keys in a fixed 2.5 MiB array compiled into the library, so
 * it calls no cudaMalloc, cudaFree or other allocating routine; inputs and outputs are
 * still the caller's.
 *
 * Limits: count <= 1,048,576 scores and k <= 1,024; anything larger returns
 * SECANT_ERROR_INSUFFICIENT_BUFFER and nothing is launched (use secant_b200_topk()).
 * The array exists once per device and is held until the process exits.  All calls on a
 * device share it: two calls whose kernels overlap on the GPU (different streams, or
 * different host threads) race on the intermediate keys and return garbage, so serialise
 * them.  The first call on each device looks up the array's device address (with that
 * device current); make that first call outside any stream capture.  Results are identical
 * to secant_b200_topk().  Asynchronous on `stream`.
 */
SECANT_DEC SecantResult secant_b200_topk_static(uintptr_t scores, size_t count, size_t k, uintptr_t indices_out,
                                                uintptr_t scores_out, void* stream);

/* Sustained FP32 rate of the current device in lane-instructions per second (one FFMA on
 * one lane = 1), measured with independent FFMA chains for about seconds_budget seconds.
 * This is the denominator of the evaluator's FP32 roofline.  Allocates a small buffer. */
SECANT_DEC SecantResult secant_b200_fp32_peak_probe(double seconds_budget, double* lane_instructions_per_second);

/* Human-readable description of the last CUDA error seen by a runner (empty when none). */
SECANT_DEC const char* secant_b200_runner_last_error(SecantCubinRunner runner);

/* Number of kernels this library has launched in the calling process so far. */
SECANT_DEC uint64_t secant_b200_kernel_launch_count(void);

/* Bytes of dataset rows the evaluator launches of the calling process have been asked to read so
 * far: every launch splits its programs into groups of thread blocks and each group reads every
 * row of every column once ((inputs + targets) x rows x 4 bytes per group).  With a dataset larger
 * than the L2 cache this is the row stream from HBM; benchmarks divide it by the run time. */
SECANT_DEC uint64_t secant_b200_row_stream_bytes(void);

#endif /* SECANT_B200_EXT_H_INCLUDED */
