/*
 * odezza_b200.h - the scoring, random-pool and score-reduction part of the reference ODE engine's C
 * API (projects/odezza/core/odezza.h), provided by libsecant_b200.so over this library's rollout
 * scorer and reducers.
 *
 * Restated interface: type names, field order, enumerator values and function signatures are those
 * of the reference header, so that a caller compiled against either header links to either
 * library for the entry points declared here.  Each declaration cites what it replaces.  What the
 * reference does underneath (generate a CUDA template, compile it with NVRTC, inspect the binary,
 * patch machine code per system, load and unload modules) does not happen here: right-hand sides
 * are translated to this library's records and interpreted by the rollout kernel, so the
 * capacities of the create info are accepted and ignored.
 *
 * Not provided: the template artifact API, the Levenberg-Marquardt engine, the frontend and the
 * multi-GPU runtime of the reference.
 */
#ifndef ODEZZA_B200_H
#define ODEZZA_B200_H

#include <cuda.h>

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef ODEZZA_DEC
#define ODEZZA_DEC __attribute__((visibility("default")))
#endif

#define ODEZZA_MAX_TOGGLE_BITS 32u

/* projects/odezza/core/odezza.h:44-68 */
typedef enum OdezzaResult {
    ODEZZA_SUCCESS = 0,
    ODEZZA_ERROR_INVALID_ARGUMENT = 1,
    ODEZZA_ERROR_INSUFFICIENT_BUFFER = 2,
    ODEZZA_ERROR_OVERFLOW = 3,
    ODEZZA_ERROR_FORMAT = 4,
    ODEZZA_ERROR_ALLOCATION = 5,
    ODEZZA_ERROR_IO = 6,
    ODEZZA_ERROR_UNSUPPORTED = 7,
    ODEZZA_ERROR_COMPILATION = 8,
    ODEZZA_ERROR_COMPILER = 9,
    ODEZZA_ERROR_AST = 10,
    ODEZZA_ERROR_SPECIALIZATION_CAPACITY = 11,
    ODEZZA_ERROR_REGISTER_PRESSURE = 12,
    ODEZZA_ERROR_STATE_LAYOUT = 13,
    ODEZZA_ERROR_QUEUE_FULL = 14,
    ODEZZA_ERROR_CUDA = 15,
    ODEZZA_ERROR_THREAD = 16,
    ODEZZA_ERROR_BUSY = 17,
    ODEZZA_ERROR_CUDA_UNFENCED = 18,
    ODEZZA_RESULT_COUNT
} OdezzaResult;

/* Postorder right-hand-side bytecode: one opcode byte, then its payload (state / constant index: one
 * byte; literal: four bytes, little endian; two-way toggle: bit; four-way toggle: two bits).
 * projects/odezza/core/odezza.h:70-96 */
typedef enum OdezzaAstOpcode {
    ODEZZA_AST_RETURN_F32 = 0x80,
    ODEZZA_AST_STATE_F32 = 0x81,
    ODEZZA_AST_CONSTANT_F32 = 0x82,
    ODEZZA_AST_LITERAL_F32 = 0x83,
    ODEZZA_AST_TOGGLE2_F32 = 0x84,
    ODEZZA_AST_TOGGLE4_F32 = 0x85,
    ODEZZA_AST_ADD_F32 = 0x90,
    ODEZZA_AST_SUB_F32 = 0x91,
    ODEZZA_AST_MUL_F32 = 0x92,
    ODEZZA_AST_DIV_F32 = 0x93,
    ODEZZA_AST_NEG_F32 = 0x94,
    ODEZZA_AST_SQRT_F32 = 0x95,
    ODEZZA_AST_RCP_F32 = 0x96,
    ODEZZA_AST_ABS_F32 = 0x97,
    ODEZZA_AST_MIN_F32 = 0x98,
    ODEZZA_AST_MAX_F32 = 0x99,
    ODEZZA_AST_FMA_F32 = 0x9a,
    ODEZZA_AST_SIN_F32 = 0x9b,
    ODEZZA_AST_COS_F32 = 0x9c,
    ODEZZA_AST_EX2_F32 = 0x9d,
    ODEZZA_AST_LG2_F32 = 0x9e,
    ODEZZA_AST_RSQRT_F32 = 0x9f,
    ODEZZA_AST_TANH_F32 = 0xa0,
    ODEZZA_AST_EXP_F32 = 0xa1,
    ODEZZA_AST_LOG_F32 = 0xa2
} OdezzaAstOpcode;

/* projects/odezza/core/odezza.h:104-119 */
typedef struct OdezzaAstProgram {
    const uint8_t* bytes;
    size_t byte_count;
} OdezzaAstProgram;
typedef struct OdezzaScoringRhs { /* one program and the derivative it writes */
    uint8_t state_index;
    OdezzaAstProgram program;
} OdezzaScoringRhs;
typedef struct OdezzaScoringSystem { /* every derivative not fixed at handle creation */
    const OdezzaScoringRhs* rhs;
    size_t rhs_count;
} OdezzaScoringSystem;

typedef struct OdezzaScoringPipeline OdezzaScoringPipeline;

/* projects/odezza/core/odezza.h:248-267.  sm_version, the capacities, worker_count and
 * cubin_slots_per_worker describe the reference's compiled template and its specialization workers;
 * they are validated for plausibility (non-zero where the reference requires it) and otherwise
 * unused.  state_count is at most 8 here. */
typedef struct OdezzaScoringPipelineCreateInfo {
    uint32_t sm_version;
    size_t state_count;
    size_t state_capacity;
    uint32_t constant_count;
    uint32_t constant_capacity;
    const OdezzaScoringRhs* fixed_rhs;
    size_t fixed_rhs_count;
    uint32_t system_capacity;
    uint32_t shared_patch_capacity;
    uint32_t system_patch_capacity;
    uint32_t worker_count;
    uint32_t cubin_slots_per_worker;
} OdezzaScoringPipelineCreateInfo;

/* projects/odezza/core/odezza.h:304-311: a coefficient drawn from a shared pool.  distribution 0 =
 * the value `shift`, 1 = uniform pool, 2 = normal pool; pool index = offset + bank * stride; value =
 * clamp(pool[index] * scale + shift, lower, upper), multiply and add rounded separately. */
typedef struct OdezzaSampledParameter {
    uint64_t offset;
    uint32_t stride, distribution;
    float scale, shift, lower, upper;
} OdezzaSampledParameter;

/* projects/odezza/core/odezza.h:313-343.  Constant banks are [system, bank, constant]; times are
 * [concatenated point]; reference data is [state, concatenated point]; MSE output is [system,
 * configuration], configuration = bank * 2^active_toggle_count + permutation.  Trajectories are
 * ragged (trajectory_offsets has trajectory_count + 1 entries); invalid data gives FLT_MAX. */
typedef struct OdezzaScoringLaunch {
    CUdeviceptr constant_banks_device;
    uint32_t constant_bank_count;
    uint32_t active_toggle_count;
    CUdeviceptr trajectory_offsets_device;
    CUdeviceptr trajectory_times_device;
    CUdeviceptr reference_data_device;
    uint32_t trajectory_count;
    uint32_t trajectory_point_count;
    uint32_t steps_per_observation;
    CUdeviceptr mse_output_device;
    CUdeviceptr sampled_parameters_device, uniform_pool_device, normal_pool_device;
    uint64_t rng_pool_size;
    uint32_t allow_missing_observations;
    CUevent input_ready_event;
    uint32_t profile_timing;
} OdezzaScoringLaunch;

/* projects/odezza/core/odezza.h:345-363.  module_count counts the program batches of the run;
 * specialization_seconds is the time spent translating and encoding programs, module_load_seconds
 * their upload; the three gpu_* fields all hold the device time of the scoring kernels when
 * profile_timing is set. */
typedef struct OdezzaScoringRunReport {
    size_t system_count;
    size_t module_count;
    uint64_t configuration_count;
    double total_seconds;
    double queue_wait_seconds, cubin_reset_seconds, specialization_seconds;
    double module_load_seconds, function_lookup_seconds, launch_seconds;
    double completion_wait_seconds, module_unload_seconds;
    double gpu_sum_seconds, gpu_active_seconds, gpu_span_seconds;
    uint64_t profiled_modules;
    uint32_t maximum_register_count, maximum_shared_memory_bytes;
} OdezzaScoringRunReport;

/* projects/odezza/core/odezza.h:370-398.  The CUDA context current at creation must be current for
 * every run and for destruction; the library never creates or sets one.  A failed creation may
 * return a diagnostic handle on which only write_error and destroy may be called.  run is
 * synchronous, validates the launch before touching anything (a rejected launch reports zero
 * modules and configurations), and leaves the handle reusable after a bad program. */
ODEZZA_DEC OdezzaResult odezza_scoring_pipeline_create(const OdezzaScoringPipelineCreateInfo* create_info,
                                                       OdezzaScoringPipeline** pipeline_ret);
ODEZZA_DEC OdezzaResult odezza_scoring_pipeline_destroy(OdezzaScoringPipeline* pipeline);
ODEZZA_DEC OdezzaResult odezza_scoring_pipeline_workspace_requirements(const OdezzaScoringPipeline* pipeline,
                                                                       size_t* workspace_size_ret,
                                                                       size_t* workspace_alignment_ret);
ODEZZA_DEC OdezzaResult odezza_scoring_pipeline_run(OdezzaScoringPipeline* pipeline, const OdezzaScoringSystem* systems,
                                                    size_t system_count, const OdezzaScoringLaunch* launch, void* workspace,
                                                    size_t workspace_size, OdezzaScoringRunReport* report_ret);
ODEZZA_DEC OdezzaResult odezza_scoring_pipeline_write_error(const OdezzaScoringPipeline* pipeline, char* buffer,
                                                            size_t buffer_size, size_t* error_bytes_ret);

/* Counters the reference keeps for its own tests (projects/odezza/core/o_odezza_internal.h:84-103,
 * :209); only the ticket and failure counts are meaningful here (one ticket per program batch). */
typedef struct OdezzaScoringPipelineStats {
    uint64_t submitted_ticket_count;
    uint64_t completed_ticket_count;
    uint64_t cubin_reset_count;
    uint64_t cubin_reset_byte_count;
    uint64_t specialization_failure_count;
    uint64_t cuda_failure_count;
    uint64_t worker_slot_wait_count;
    uint32_t peak_pending_ticket_count;
    uint32_t peak_ready_slot_count;
    uint32_t peak_inflight_module_count;
    double cubin_reset_seconds;
    double specialization_seconds;
    double module_load_seconds;
    double function_lookup_seconds;
    double launch_seconds;
    double completion_wait_seconds;
    double module_unload_seconds;
    double cuda_resource_create_seconds;
} OdezzaScoringPipelineStats;
ODEZZA_DEC OdezzaResult o_scoring_pipeline_stats(const OdezzaScoringPipeline* pipeline, OdezzaScoringPipelineStats* stats_ret);

/* ---- random pools: projects/odezza/core/odezza.h:400-434, projects/odezza/core/o_philox.cu ------- */
#define ODEZZA_RNG_VERSION 1u
#define ODEZZA_RNG_UNIFORM 1u
#define ODEZZA_RNG_NORMAL 2u
typedef struct OdezzaRngPool OdezzaRngPool;
typedef struct OdezzaRngPoolInfo {
    uint64_t seed, stream, sample_base, size; /* size = samples per plane */
    uint32_t distributions;                   /* ODEZZA_RNG_UNIFORM | ODEZZA_RNG_NORMAL */
} OdezzaRngPoolInfo;
typedef struct OdezzaRngPoolView {
    CUdeviceptr uniform_device, normal_device;
    OdezzaRngPoolInfo info;
    double uniform_seconds, normal_seconds;
} OdezzaRngPoolView;
/* Standard Philox4x32-10, on the host. */
ODEZZA_DEC OdezzaResult odezza_philox4x32(const uint32_t counter[4], const uint32_t key[2], uint32_t out[4]);
/* Host replay of one uniform sample: block = sample / 4, key = seed, counter = {block, stream << 1},
 * value = ((bits >> 9) + 0.5) * 2^-23 (open interval). */
ODEZZA_DEC OdezzaResult odezza_rng_uniform(uint64_t seed, uint64_t stream, uint64_t sample, float* out);
/* Fills the requested planes on the device of the current context; the pool owns its allocation.
 * Normal samples are Box-Muller pairs of the uniform samples of the normal domain, in float32. */
ODEZZA_DEC OdezzaResult odezza_rng_pool_create(uint32_t sm, const OdezzaRngPoolInfo* info, OdezzaRngPool** out);
ODEZZA_DEC OdezzaResult odezza_rng_pool_view(const OdezzaRngPool* pool, OdezzaRngPoolView* out);
ODEZZA_DEC OdezzaResult odezza_rng_pool_write_error(const OdezzaRngPool* pool, char* out, size_t capacity);
ODEZZA_DEC OdezzaResult odezza_rng_pool_destroy(OdezzaRngPool* pool);
ODEZZA_DEC OdezzaResult odezza_sampled_parameter_validate(const OdezzaRngPoolInfo* pool, uint32_t bank_count,
                                                          const OdezzaSampledParameter* parameter);

/* ---- score reduction: projects/odezza/core/odezza.h:436-518, projects/odezza/core/o_score_reduce.cu */
typedef struct OdezzaScoreReducer OdezzaScoreReducer;
typedef enum OdezzaScoreGrouping {
    ODEZZA_SCORE_BY_SYSTEM = 0,
    ODEZZA_SCORE_BY_SYSTEM_PERMUTATION = 1,
    ODEZZA_SCORE_GLOBAL = 2
} OdezzaScoreGrouping;
typedef struct OdezzaScoreWinner { /* stable order (mse, score_index); unfilled ranks FLT_MAX, UINT64_MAX */
    float mse;
    uint32_t reserved;
    uint64_t score_index;
} OdezzaScoreWinner;
typedef struct OdezzaScoreCounts {
    uint64_t valid, invalid, negative;
} OdezzaScoreCounts;
typedef struct OdezzaScoreIndex {
    uint64_t system_index, configuration_index, bank_index;
    uint32_t permutation;
} OdezzaScoreIndex;
typedef struct OdezzaScoreReductionSize {
    uint64_t configuration_count, score_count, group_count;
    uint32_t tiles_per_group;
    size_t workspace_bytes, winner_bytes, count_bytes;
} OdezzaScoreReductionSize;
typedef struct OdezzaScoreReductionReport {
    double kernel_seconds;
    uint64_t group_count, score_count;
} OdezzaScoreReductionReport;
/* k in 1..256.  No kernel is compiled at creation here; set_k, run and gather allocate nothing. */
ODEZZA_DEC OdezzaResult odezza_score_reducer_create(uint32_t sm_version, uint32_t k, OdezzaScoreReducer** out);
ODEZZA_DEC OdezzaResult odezza_score_reducer_set_k(OdezzaScoreReducer* r, uint32_t k);
ODEZZA_DEC OdezzaResult odezza_score_reducer_destroy(OdezzaScoreReducer* r);
ODEZZA_DEC OdezzaResult odezza_score_reducer_write_error(const OdezzaScoreReducer* r, char* out, size_t capacity);
/* Layout from the launch and the bulk run's system count; no CUDA needed.  workspace_bytes is what
 * the reference's tiled reducer would need; this library's reducer uses none of it. */
ODEZZA_DEC OdezzaResult odezza_score_reduction_requirements(const OdezzaScoringLaunch* launch, size_t system_count,
                                                            OdezzaScoreGrouping grouping, uint32_t k,
                                                            OdezzaScoreReductionSize* out);
ODEZZA_DEC OdezzaResult odezza_score_decode_index(const OdezzaScoringLaunch* launch, size_t system_count, uint64_t score_index,
                                                  OdezzaScoreIndex* out);
/* Synchronous.  winners [group, k], counts [group]; raw scores are not modified. */
ODEZZA_DEC OdezzaResult odezza_score_reducer_run(OdezzaScoreReducer* r, const OdezzaScoringLaunch* launch, size_t system_count,
                                                 OdezzaScoreGrouping grouping, CUdeviceptr workspace, size_t workspace_bytes,
                                                 CUdeviceptr winners, size_t winner_bytes, CUdeviceptr counts,
                                                 size_t count_bytes, OdezzaScoreReductionReport* report);
/* Gathers the winners' constants from [system, bank, constant] into rows [group, k, constant];
 * unfilled ranks receive NaN. */
ODEZZA_DEC OdezzaResult odezza_score_reducer_gather(OdezzaScoreReducer* r, const OdezzaScoringLaunch* launch, size_t system_count,
                                                    OdezzaScoreGrouping grouping, uint32_t constant_count, CUdeviceptr winners,
                                                    size_t winner_bytes, CUdeviceptr rows, size_t row_bytes);

#ifdef __cplusplus
}
#endif

#endif /* ODEZZA_B200_H */
