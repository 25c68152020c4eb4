/*
 * evaluator.cuh - launch interface of the population evaluator kernels (evaluator.cu).
 */
#ifndef SECANT_B200_EVALUATOR_CUH
#define SECANT_B200_EVALUATOR_CUH

#include "../../include/secant_b200.h"
#include "record.h"

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace sb {
/* adds to the process-wide count reported by secant_b200_kernel_launch_count() */
void note_kernel_launches(unsigned n);

/* Grouped top-k of a [system][configuration] score grid (reduce.cu); scratch may be zero. */
SecantResult grouped_topk(uintptr_t scores, size_t num_systems, size_t num_banks, uint32_t toggle_bits, uint32_t grouping, uint32_t k,
                          uintptr_t winners, uintptr_t counts, uintptr_t scratch, size_t scratch_bytes, cudaStream_t stream);

/* Random pools and winner gathering of the ODE engine interface (pools.cu). */
cudaError_t fill_pool(float* out, unsigned long long size, unsigned long long seed, unsigned long long stream_id,
                      unsigned long long sample_base, bool normal, cudaStream_t stream);
struct GatherProblem {
    const SecantB200Winner* winners;
    const float* banks;                          /* [system][bank][constant], or null when sampled */
    const SecantB200SampledParameter* sampled;   /* [system][constant], or null */
    const float* uniform_pool;
    const float* normal_pool;
    unsigned long long pool_size, entries, configurations, bank_count, score_count;
    unsigned toggle_bits, constants;
    float* rows;                                 /* [entry][constant] */
};
cudaError_t gather_constants(const GatherProblem& problem, cudaStream_t stream);
}

namespace sb {

enum EvalMode : int {
    EVAL_SSE = 0,          /* sum over rows of (prediction - target)^2 per (program, target, configuration) */
    EVAL_MATERIALIZE = 1,  /* prediction per (program, row), one configuration */
    EVAL_AFFINE_STATS = 2  /* sum p, sum p*p, sum p*t per program */
};

/* Device-resident records of one program batch. */
struct DeviceBatch {
    const SbProgram* programs;
    const SbInsn* insns;
    const SbPatch* patches;
    const SbAffine* affines;
    const float* lits;
    uint32_t num_programs;
    uint32_t max_insn;    /* largest instruction count in the batch */
    uint32_t max_extra;   /* largest n_affine + n_lits (rollout records address source constants directly) */
    uint32_t max_slots;   /* largest spill-slot count */
    uint32_t max_hoisted; /* largest number of row-prelude values */
    uint32_t max_cst;     /* largest constant table */
    uint32_t max_btmp;    /* largest number of bank-part temporaries */
    uint32_t uses_scratch; /* some program needs the scratch spill slot */
};

struct EvalProblem {
    int mode;
    const float* input;       /* [column][row] */
    size_t input_ld;
    uint32_t num_inputs;
    const float* targets;     /* [target][row] */
    size_t targets_ld;
    uint32_t num_targets;
    const float* banks;       /* [bank][slot] (+ program * program_bank_stride) */
    size_t bank_stride;
    size_t program_bank_stride;
    size_t first_program;     /* index of the batch's first program within the run */
    uint32_t num_constants;
    uint32_t num_banks;       /* >= 1 */
    uint32_t toggle_bits;
    uint32_t fixed_permutation; /* materialize: the single permutation evaluated */
    uint32_t fast_math;       /* 1: approximate division and transcendental functions (see sbmath.cuh) */
    size_t num_rows;
    float* output;
    size_t out_program_stride; /* elements between consecutive programs */
    size_t out_target_stride;  /* elements between consecutive targets  */
};

/* Launch geometry chosen by plan_launch(). */
struct LaunchPlan {
    int variant;              /* rows x banks per thread: 0: 4x4, 1: 8x2, 2: 16x1 */
    uint32_t warps;           /* per CTA */
    uint32_t tile_rows;       /* rows staged per tile, multiple of the pass size */
    uint32_t tile_buffers;    /* 2 when a CTA walks more than one tile: the next tile is fetched while this one is used */
    uint32_t num_groups;      /* CTAs along the programs; group g owns programs g, g + num_groups, ... */
    uint32_t groups_per_item; /* bank groups of one permutation a warp handles per queue item */
    uint32_t perms_per_item;  /* consecutive permutations one item covers (a power of two; above 1 only when an item holds every bank group) */
    uint32_t row_splits;      /* CTAs sharing one program group, each with a row range */
    size_t rows_per_split;
    size_t smem_bytes;
    size_t partial_elements;  /* floats of per-split partial sums the launch needs (0: materialize) */
    uint32_t grid_x;
    bool ok;
    bool overflow;            /* !ok because a count does not fit the kernel's 32-bit indices */
};

/* Shared-memory layout and loop bounds of one launch, derived from the plan. */
struct Geom {
    uint32_t tile_rows;       /* floats between consecutive columns of a staged tile */
    uint32_t tile_buffers;
    uint32_t tile_bytes;      /* one buffer */
    uint32_t num_groups;
    uint32_t row_splits;
    uint32_t groups_per_item;
    uint32_t perms_per_item;
    uint32_t exec_bytes;      /* per-warp regions, each a multiple of 16 bytes */
    uint32_t table_bytes;
    uint32_t hoist_bytes;
    uint32_t slot_bytes;
    uint32_t psum_bytes;
    uint32_t warp_bytes;
    uint32_t scratch_slot;    /* spill slot reserved for the element-by-element FMA */
    unsigned long long rows_per_split;
};

constexpr int kNumVariants = 3;
constexpr int kVariantRows[kNumVariants] = {4, 8, 16};
constexpr int kVariantBanks[kNumVariants] = {4, 2, 1};

Geom make_geom(const DeviceBatch& batch, const EvalProblem& problem, const LaunchPlan& plan);

/* scratch_limit: most floats of per-split partial sums a launch may use (row splits are reduced to fit). */
LaunchPlan plan_launch(const DeviceBatch& batch, const EvalProblem& problem, int sm_count, size_t smem_limit,
                       size_t scratch_limit);

/* Enqueues the evaluation of one batch on `stream`: the evaluator kernel writes per-split partial
 * sums into `partial` (plan.partial_elements floats, private to the stream until the launch has
 * finished) and a second kernel adds them in a fixed order into the output, so a result does
 * not depend on the order CTAs ran in.  Returns the CUDA status of the launches. */
cudaError_t launch_eval(const DeviceBatch& batch, const EvalProblem& problem, const LaunchPlan& plan, float* partial,
                        cudaStream_t stream, unsigned* launches);

/* Fixed-step RK4 rollout scoring of S-state systems whose right-hand sides are programs. */
struct Rk4Problem {
    uint32_t num_systems, num_states, num_constants, num_banks, toggle_bits;
    const float* banks;            /* [system][bank][slot] */
    size_t bank_stride, system_bank_stride;
    const float* reference;        /* [state][total_points]; a trajectory starts at its first point */
    size_t reference_ld;
    uint32_t num_trajectories, points_per_trajectory, substeps;
    const float* times;            /* [points_per_trajectory], or [total_points] with offsets */
    const uint32_t* offsets;       /* [num_trajectories + 1] partition of total_points, or null */
    uint32_t total_points;         /* concatenated points (both forms) */
    uint32_t allow_missing;        /* NaN reference values after a first point are unobserved */
    int* invalid_flag;             /* device word the validation kernel raises */
    const SecantB200SampledParameter* sampled; /* [system][constant] descriptors, or null: explicit banks */
    const float* uniform_pool;
    const float* normal_pool;
    unsigned long long pool_size;
    float* output;                 /* [system][configuration] */
    size_t output_ld;
    unsigned long long* queue;      /* device counter, zero at launch: the next item to be taken */
    const uint32_t* order;          /* optional [num_systems]: the system whose items are taken k-th (costliest first) */
    unsigned long long* integrated; /* optional device counter: (trajectory, observation interval) pairs integrated */
};
/* batch.programs holds num_systems * num_states records, system-major, encoded with
 * columns_are_slots, 4 * num_states reserved slots and a bank part.  `concurrent` = how many such
 * launches share the device at a time (the launch takes that share of the resident CTAs). */
cudaError_t launch_rk4(const DeviceBatch& batch, const Rk4Problem& problem, size_t smem_limit, unsigned concurrent, cudaStream_t stream);

/* Adds the statistics of the static Gram shape for a batch of cohorts over `rows` rows of
 * materialized predictions [program of the batch][prediction_ld] (gram.cu); statistics points at
 * the batch's first cohort. */
cudaError_t launch_gram(const float* predictions, size_t prediction_ld, uint32_t rows, const float* targets, size_t targets_ld,
                        uint32_t num_targets, uint32_t cohort_size, uint32_t batch_programs, float* statistics, size_t statistics_ld,
                        cudaStream_t stream);

/* One-time per-device kernel attribute setup (dynamic shared memory opt-in). */
cudaError_t configure_kernels();

}  // namespace sb

#endif
