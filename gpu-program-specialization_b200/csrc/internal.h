/*
 * internal.h - host-side types shared by the API shims, the validator and the runner.
 */
#ifndef SECANT_B200_INTERNAL_H
#define SECANT_B200_INTERNAL_H

#include "../../include/secant_b200.h"
#include "encoder.h"

#include <cstddef>
#include <cstdint>

/* The opaque plan lives in caller-owned storage (reference contract, secant.h:1012-1016).
 * It records the validated recipe and the size of the binary the caller compiled; the
 * binary itself is never inspected because no machine code is patched. */
struct SecantCubinPlan {
    uint64_t magic;
    SecantKernelShape shape;
    uint32_t pad;
    size_t cubin_size;
    size_t num_kernels, asts_per_kernel, num_inputs, num_constants, num_targets, tile_rows, threads_per_block,
        patch_capacity_instructions;
};

namespace sb {

constexpr uint64_t kPlanMagic = 0x5342323030504c4eull; /* "SB200PLN" */

/* A run request reduced to what the evaluator needs, after all reference checks. */
struct UnpackedRun {
    SecantAstProgramSet programs{};
    SecantDeviceMatrixF32 input{}, targets{}, output{};
    SecantDeviceConstantBanks banks{};
    size_t rows = 0, num_targets = 0, num_banks = 1, configurations = 1;
    uint32_t toggle_bits = 0;
    size_t program_bank_stride = 0, first_program_index = 0;
    size_t input_span = 0, target_span = 0, bank_span = 0, output_span = 0;
    size_t output_count = 0, output_width = 0; /* cleared region: count vectors of width elements */
};

SecantResult recipe_header_validate(const SecantCubinRecipeHeader* recipe);
SecantResult recipe_validate(const SecantCubinRecipeHeader* recipe);
void plan_fill(SecantCubinPlan* plan, const SecantCubinRecipeHeader* recipe, size_t cubin_size);

/* Restates s_run_unpack (projects/secant/s_cubin_runner.c:33-137). */
SecantResult run_unpack(const SecantCubinPlan& plan, const SecantCubinRunHeader* header, UnpackedRun* out);
/* Restates s_runs_validate (projects/secant/s_cubin_runner.c:195-241): identical program
 * arrays, address ranges, overlap inside and across entries, program preflight. */
SecantResult runs_validate(const SecantCubinPlan& plan, const UnpackedRun* runs, size_t count, ProgramRules* rules_ret,
                           bool skip_preflight = false);

}  // namespace sb

#endif
