/*
 * api.cpp - the entry points of the reference C API that need no GPU: result names,
 * recipe validation, source/plan shims and program validation.
 *
 * The reference generates a CUDA kernel template per recipe, has the caller compile it,
 * inspects the binary into a plan and patches machine code into copies of it
 * (projects/secant/s_cubin_api.c, s_cubin_inspect.c, s_cubin_specialize.c).  This library
 * evaluates programs with resident kernels, so these calls keep their signatures, their
 * validation and their error codes but carry no machine code: the generated source is a
 * stub, the plan records the recipe, and "specialize" validates programs.
 */
#include "internal.h"

#include <cstdio>
#include <cstring>

namespace sb {

namespace {

bool add_ok(size_t a, size_t b, size_t* out) {
    if (b > SIZE_MAX - a) return false;
    *out = a + b;
    return true;
}
bool mul_ok(size_t a, size_t b, size_t* out) {
    if (a && b > SIZE_MAX / a) return false;
    *out = a * b;
    return true;
}

constexpr size_t kMarkerRegisters = 256; /* the reference's per-kernel marker budget */

/* Shared by the static SSE / affine / Gram recipes (s_cubin_generate_sse.c:385-459 and the
 * matching blocks of the affine and Gram generators). */
SecantResult tiled_recipe_validate(size_t kernels, size_t asts, size_t inputs, size_t targets, size_t tile_rows,
                                   size_t threads, size_t patch, size_t per_ast_outputs_base, bool gram) {
    size_t per_ast, outputs, markers, total;
    if (!kernels || !asts || asts > kMarkerRegisters || !inputs || inputs > SECANT_AST_MAX_INPUTS || !targets || !patch)
        return SECANT_ERROR_INVALID_VALUE;
    if (gram) {
        if (asts > 32u) return SECANT_ERROR_INVALID_VALUE;
        if (!add_ok(inputs, asts, &markers) || markers > kMarkerRegisters) return SECANT_ERROR_INVALID_VALUE;
    } else {
        if (!add_ok(per_ast_outputs_base, targets, &per_ast) || !mul_ok(asts, per_ast, &outputs) ||
            !add_ok(inputs, targets, &markers) || !add_ok(markers, outputs, &markers) || markers > kMarkerRegisters)
            return SECANT_ERROR_INVALID_VALUE;
    }
    if (!mul_ok(kernels, markers, &total) || total - 1u > 0x3fffffffu) return SECANT_ERROR_INVALID_VALUE;
    if (!tile_rows || threads < 32u || threads > tile_rows || threads > 512u || threads % 32u)
        return SECANT_ERROR_UNSUPPORTED_SHAPE;
    if (gram) {
        size_t columns, elements;
        if (!add_ok(inputs, asts + 1u, &columns) || !mul_ok(columns, tile_rows, &elements) || elements + 1u > 12288u)
            return SECANT_ERROR_UNSUPPORTED_SHAPE;
    }
    return SECANT_SUCCESS;
}

size_t concrete_size(SecantKernelShape shape) {
    switch (shape) {
    case SECANT_KERNEL_SHAPE_STATIC_MATERIALIZE_F32: return sizeof(SecantCubinMaterializeRecipe);
    case SECANT_KERNEL_SHAPE_STATIC_SSE_F32: return sizeof(SecantCubinSSERecipe);
    case SECANT_KERNEL_SHAPE_STATIC_AFFINE_STATS_F32: return sizeof(SecantCubinAffineStatsRecipe);
    case SECANT_KERNEL_SHAPE_STATIC_GRAM_STATS_F32: return sizeof(SecantCubinGramStatsRecipe);
    case SECANT_KERNEL_SHAPE_TOGGLE_SSE_F32: return sizeof(SecantCubinToggleSSERecipe);
    default: return 0;
    }
}

const char* shape_tag(SecantKernelShape shape) {
    switch (shape) {
    case SECANT_KERNEL_SHAPE_STATIC_MATERIALIZE_F32: return "materialize";
    case SECANT_KERNEL_SHAPE_STATIC_SSE_F32: return "sse";
    case SECANT_KERNEL_SHAPE_STATIC_AFFINE_STATS_F32: return "affine_stats";
    case SECANT_KERNEL_SHAPE_STATIC_GRAM_STATS_F32: return "gram_stats";
    default: return "toggle_sse";
    }
}

/* The stub translation unit handed to the caller's compiler.  It defines one empty kernel
 * per recipe kernel, named like the reference names its kernels, so code that looks the
 * functions up keeps working; nothing in it is ever launched by this library. */
SecantResult stub_source(const SecantCubinPlan& p, char* output, size_t output_size, size_t* required) {
    size_t at = 0;
    bool overflow = false;
    auto put = [&](const char* text) {
        const size_t n = std::strlen(text);
        if (output && !overflow) {
            if (at + n + 1 > output_size) overflow = true;
            else std::memcpy(output + at, text, n);
        }
        at += n;
    };
    char line[256];
    std::snprintf(line, sizeof(line),
                  "// secant-b200 %s: programs are evaluated by the library's resident sm_100a kernels.\n"
                  "// recipe %s kernels=%zu asts_per_kernel=%zu inputs=%zu constants=%zu targets=%zu\n",
                  SECANT_VERSION_STRING, shape_tag(p.shape), p.num_kernels, p.asts_per_kernel, p.num_inputs,
                  p.num_constants, p.num_targets);
    put(line);
    for (size_t k = 0; k < p.num_kernels; ++k) {
        std::snprintf(line, sizeof(line), "extern \"C\" __global__ void secant_cubin_%s_%03zu() {}\n", shape_tag(p.shape), k);
        put(line);
    }
    *required = at + 1;
    if (!output) return SECANT_SUCCESS;
    if (overflow || at + 1 > output_size) return SECANT_ERROR_INSUFFICIENT_BUFFER;
    output[at] = '\0';
    return SECANT_SUCCESS;
}

}  // namespace

SecantResult recipe_header_validate(const SecantCubinRecipeHeader* recipe) {
    if (!recipe || recipe->struct_size < sizeof(*recipe)) return SECANT_ERROR_INVALID_VALUE;
    if (recipe->version != SECANT_CUBIN_RECIPE_VERSION_3) return SECANT_ERROR_UNSUPPORTED_VERSION;
    if (recipe->flags) return SECANT_ERROR_INVALID_VALUE;
    const size_t need = concrete_size(recipe->shape);
    if (!need) return SECANT_ERROR_UNSUPPORTED_SHAPE;
    return recipe->struct_size < need ? SECANT_ERROR_INVALID_VALUE : SECANT_SUCCESS;
}

SecantResult recipe_validate(const SecantCubinRecipeHeader* recipe) {
    const SecantResult header = recipe_header_validate(recipe);
    if (header != SECANT_SUCCESS) return header;
    switch (recipe->shape) {
    case SECANT_KERNEL_SHAPE_STATIC_MATERIALIZE_F32: {
        const auto* r = reinterpret_cast<const SecantCubinMaterializeRecipe*>(recipe);
        size_t markers, total;
        if (!r->num_kernels || !r->asts_per_kernel || r->asts_per_kernel > kMarkerRegisters || !r->num_inputs ||
            r->num_inputs > SECANT_AST_MAX_INPUTS || !r->patch_capacity_instructions ||
            !add_ok(r->num_inputs, r->asts_per_kernel, &markers) || markers > kMarkerRegisters ||
            !mul_ok(r->num_kernels, markers, &total) || total - 1u > 0x3fffffffu)
            return SECANT_ERROR_INVALID_VALUE;
        return SECANT_SUCCESS;
    }
    case SECANT_KERNEL_SHAPE_STATIC_SSE_F32: {
        const auto* r = reinterpret_cast<const SecantCubinSSERecipe*>(recipe);
        return tiled_recipe_validate(r->num_kernels, r->asts_per_kernel, r->num_inputs, r->num_targets, r->tile_rows,
                                     r->threads_per_block, r->patch_capacity_instructions, 0, false);
    }
    case SECANT_KERNEL_SHAPE_STATIC_AFFINE_STATS_F32: {
        const auto* r = reinterpret_cast<const SecantCubinAffineStatsRecipe*>(recipe);
        return tiled_recipe_validate(r->num_kernels, r->asts_per_kernel, r->num_inputs, r->num_targets, r->tile_rows,
                                     r->threads_per_block, r->patch_capacity_instructions, 2, false);
    }
    case SECANT_KERNEL_SHAPE_STATIC_GRAM_STATS_F32: {
        const auto* r = reinterpret_cast<const SecantCubinGramStatsRecipe*>(recipe);
        return tiled_recipe_validate(r->num_kernels, r->asts_per_kernel, r->num_inputs, r->num_targets, r->tile_rows,
                                     r->threads_per_block, r->patch_capacity_instructions, 0, true);
    }
    default: { /* toggle SSE: s_cubin_generate_toggle_sse.c:320-337 */
        const auto* r = reinterpret_cast<const SecantCubinToggleSSERecipe*>(recipe);
        size_t sources, outputs, markers, all, shared;
        if (!r->num_kernels || r->num_kernels > 65535u || !r->asts_per_kernel || r->asts_per_kernel > 32u ||
            r->num_inputs > SECANT_AST_MAX_INPUTS || r->num_constants > SECANT_AST_MAX_INPUTS || !r->num_targets ||
            r->num_targets > 32u || !r->tile_rows || !r->threads_per_block || r->threads_per_block > 1024u ||
            r->threads_per_block % 32u || !r->patch_capacity_instructions ||
            !add_ok(r->num_inputs, r->num_constants, &sources) || sources > SECANT_AST_MAX_INPUTS ||
            !add_ok(sources, r->num_targets, &sources) || !mul_ok(r->asts_per_kernel, r->num_targets, &outputs) ||
            !add_ok(sources, outputs, &markers) || markers > 192u || !mul_ok(markers, r->num_kernels, &all) ||
            all > 0x7fffffffu || !mul_ok(r->num_inputs + r->num_targets, r->tile_rows, &shared) || shared > 12000u)
            return SECANT_ERROR_INVALID_VALUE;
        return SECANT_SUCCESS;
    }
    }
}

void plan_fill(SecantCubinPlan* plan, const SecantCubinRecipeHeader* recipe, size_t cubin_size) {
    std::memset(plan, 0, sizeof(*plan));
    plan->magic = kPlanMagic;
    plan->shape = recipe->shape;
    plan->cubin_size = cubin_size;
    if (recipe->shape == SECANT_KERNEL_SHAPE_STATIC_MATERIALIZE_F32) {
        const auto* r = reinterpret_cast<const SecantCubinMaterializeRecipe*>(recipe);
        plan->num_kernels = r->num_kernels; plan->asts_per_kernel = r->asts_per_kernel; plan->num_inputs = r->num_inputs;
        plan->patch_capacity_instructions = r->patch_capacity_instructions;
    } else if (recipe->shape == SECANT_KERNEL_SHAPE_TOGGLE_SSE_F32) {
        const auto* r = reinterpret_cast<const SecantCubinToggleSSERecipe*>(recipe);
        plan->num_kernels = r->num_kernels; plan->asts_per_kernel = r->asts_per_kernel; plan->num_inputs = r->num_inputs;
        plan->num_constants = r->num_constants; plan->num_targets = r->num_targets; plan->tile_rows = r->tile_rows;
        plan->threads_per_block = r->threads_per_block; plan->patch_capacity_instructions = r->patch_capacity_instructions;
    } else { /* the three tiled static recipes share one layout */
        const auto* r = reinterpret_cast<const SecantCubinSSERecipe*>(recipe);
        plan->num_kernels = r->num_kernels; plan->asts_per_kernel = r->asts_per_kernel; plan->num_inputs = r->num_inputs;
        plan->num_targets = r->num_targets; plan->tile_rows = r->tile_rows; plan->threads_per_block = r->threads_per_block;
        plan->patch_capacity_instructions = r->patch_capacity_instructions;
    }
}

}  // namespace sb

using namespace sb;

extern "C" {

const char* secant_result_to_string(SecantResult result) {
    static const char* const names[SECANT_RESULT_COUNT] = {
        "SECANT_SUCCESS", "SECANT_ERROR_INVALID_VALUE", "SECANT_ERROR_OVERFLOW", "SECANT_ERROR_INSUFFICIENT_BUFFER",
        "SECANT_ERROR_FORMAT", "SECANT_ERROR_ALLOCATION_FAILED", "SECANT_ERROR_COMPILE_FAILED",
        "SECANT_ERROR_PARSE_FAILED", "SECANT_ERROR_SKELETON_NOT_FOUND", "SECANT_ERROR_BAD_PROGRAM",
        "SECANT_ERROR_STACK_OVERFLOW", "SECANT_ERROR_STACK_UNDERFLOW", "SECANT_ERROR_TOO_MANY_ARGS",
        "SECANT_ERROR_UNSUPPORTED_OP", "SECANT_ERROR_ROUTINE_IDX_OUT_OF_BOUNDS",
        "SECANT_ERROR_ROUTINE_ARG_IDX_OUT_OF_BOUNDS", "SECANT_ERROR_ROUTINE_DEPTH_EXCEEDED",
        "SECANT_ERROR_INSUFFICIENT_PATCH_SPACE", "SECANT_ERROR_REGISTER_OVERFLOW",
        "SECANT_ERROR_UNSUPPORTED_ARCHITECTURE", "SECANT_ERROR_INVALID_STATE", "SECANT_ERROR_UNSUPPORTED_SHAPE",
        "SECANT_ERROR_UNEXPECTED_INSTRUCTION", "SECANT_ERROR_BACKEND_UNAVAILABLE", "SECANT_ERROR_BAD_BINARY",
        "SECANT_ERROR_BAD_PATCH_SITE", "SECANT_ERROR_FUNCTION_NOT_FOUND", "SECANT_ERROR_PATCH_SITE_NOT_FOUND",
        "SECANT_ERROR_REGISTER_COUNT_NOT_FOUND", "SECANT_ERROR_THREAD_FAILED", "SECANT_ERROR_DRIVER_FAILED",
        "SECANT_ERROR_EAGER_LOADING_REQUIRED", "SECANT_ERROR_UNSUPPORTED_VERSION", "SECANT_ERROR_COMPLETION_UNKNOWN"};
    return (result >= 0 && result < SECANT_RESULT_COUNT) ? names[result] : "SECANT_ERROR_UNKNOWN";
}

/* Sum and sum of squares of every target column, accumulated atomically into
 * target_stats[target][2]; launch with grid.y = num_targets and a multiple of 32 threads
 * (contract of projects/secant/secant.h:690-716). */
const char* secant_cuda_target_stats_f32_source_get(size_t* source_size_ret) {
    static const char source[] =
        "extern \"C\" __global__ void secant_cuda_target_stats_f32(\n"
        "    const float* targets, size_t targets_leading_dimension, size_t num_rows, size_t num_targets,\n"
        "    float* target_stats, size_t target_stats_leading_dimension) {\n"
        "    const size_t target = blockIdx.y;\n"
        "    if (target >= num_targets) return;\n"
        "    const float* column = targets + target * targets_leading_dimension;\n"
        "    float sum = 0.0f, squares = 0.0f;\n"
        "    for (size_t row = (size_t)blockIdx.x * blockDim.x + threadIdx.x; row < num_rows;\n"
        "         row += (size_t)gridDim.x * blockDim.x) {\n"
        "        const float value = column[row];\n"
        "        sum += value;\n"
        "        squares = fmaf(value, value, squares);\n"
        "    }\n"
        "    for (int offset = 16; offset > 0; offset >>= 1) {\n"
        "        sum += __shfl_down_sync(0xffffffffu, sum, offset);\n"
        "        squares += __shfl_down_sync(0xffffffffu, squares, offset);\n"
        "    }\n"
        "    if ((threadIdx.x & 31u) == 0u) {\n"
        "        atomicAdd(target_stats + target * target_stats_leading_dimension, sum);\n"
        "        atomicAdd(target_stats + target * target_stats_leading_dimension + 1, squares);\n"
        "    }\n"
        "}\n";
    if (source_size_ret) *source_size_ret = sizeof(source);
    return source;
}

SecantResult secant_cubin_recipe_validate(const SecantCubinRecipeHeader* recipe) { return recipe_validate(recipe); }

SecantResult secant_cubin_source_size(const SecantCubinRecipeHeader* recipe, size_t* required_size_ret) {
    if (!required_size_ret) return SECANT_ERROR_INVALID_VALUE;
    *required_size_ret = 0;
    const SecantResult r = recipe_validate(recipe);
    if (r != SECANT_SUCCESS) return r;
    SecantCubinPlan plan;
    plan_fill(&plan, recipe, 0);
    return stub_source(plan, nullptr, 0, required_size_ret);
}

SecantResult secant_cubin_source_write(const SecantCubinRecipeHeader* recipe, char* output, size_t output_size) {
    if (!output || !output_size) return SECANT_ERROR_INVALID_VALUE;
    const SecantResult r = recipe_validate(recipe);
    if (r != SECANT_SUCCESS) return r;
    SecantCubinPlan plan;
    size_t required;
    plan_fill(&plan, recipe, 0);
    return stub_source(plan, output, output_size, &required);
}

SecantResult secant_cubin_plan_storage_size(const SecantCubinRecipeHeader* recipe, const void* cubin, size_t cubin_size,
                                            size_t* required_storage_size_ret) {
    if (!required_storage_size_ret) return SECANT_ERROR_INVALID_VALUE;
    *required_storage_size_ret = 0;
    const SecantResult r = recipe_validate(recipe);
    if (r != SECANT_SUCCESS) return r;
    if (!cubin || !cubin_size) return SECANT_ERROR_INVALID_VALUE;
    *required_storage_size_ret = sizeof(SecantCubinPlan) + alignof(SecantCubinPlan); /* room to align any pointer */
    return SECANT_SUCCESS;
}

SecantResult secant_cubin_plan_init(const SecantCubinRecipeHeader* recipe, const void* cubin, size_t cubin_size,
                                    void* plan_storage, size_t plan_storage_size, SecantCubinPlan** plan_ret) {
    if (!plan_ret) return SECANT_ERROR_INVALID_VALUE;
    *plan_ret = nullptr;
    const SecantResult r = recipe_validate(recipe);
    if (r != SECANT_SUCCESS) return r;
    if (!cubin || !cubin_size || !plan_storage) return SECANT_ERROR_INVALID_VALUE;
    uintptr_t at = reinterpret_cast<uintptr_t>(plan_storage);
    const uintptr_t aligned = (at + alignof(SecantCubinPlan) - 1) / alignof(SecantCubinPlan) * alignof(SecantCubinPlan);
    if (plan_storage_size < (aligned - at) + sizeof(SecantCubinPlan)) return SECANT_ERROR_INSUFFICIENT_BUFFER;
    auto* plan = reinterpret_cast<SecantCubinPlan*>(aligned);
    plan_fill(plan, recipe, cubin_size);
    *plan_ret = plan;
    return SECANT_SUCCESS;
}

SecantResult secant_cubin_plan_info_get(const SecantCubinPlan* plan, SecantCubinPlanInfo* info_ret) {
    if (!plan || plan->magic != kPlanMagic || !info_ret || info_ret->struct_size < sizeof(*info_ret)) return SECANT_ERROR_INVALID_VALUE;
    if (info_ret->version != SECANT_CUBIN_PLAN_INFO_VERSION_1) return SECANT_ERROR_UNSUPPORTED_VERSION;
    if (info_ret->flags) return SECANT_ERROR_INVALID_VALUE;
    info_ret->shape = plan->shape;
    info_ret->cubin_size = plan->cubin_size;
    return SECANT_SUCCESS;
}

SecantResult secant_cubin_plan_recipe_get(const SecantCubinPlan* plan, SecantCubinRecipeHeader* recipe_ret) {
    if (!plan || plan->magic != kPlanMagic) return SECANT_ERROR_INVALID_VALUE;
    const SecantResult r = recipe_header_validate(recipe_ret);
    if (r != SECANT_SUCCESS) return r;
    if (recipe_ret->shape != plan->shape) return SECANT_ERROR_UNSUPPORTED_SHAPE;
    if (plan->shape == SECANT_KERNEL_SHAPE_STATIC_MATERIALIZE_F32) {
        auto* out = reinterpret_cast<SecantCubinMaterializeRecipe*>(recipe_ret);
        out->num_kernels = plan->num_kernels; out->asts_per_kernel = plan->asts_per_kernel; out->num_inputs = plan->num_inputs;
        out->patch_capacity_instructions = plan->patch_capacity_instructions;
    } else if (plan->shape == SECANT_KERNEL_SHAPE_TOGGLE_SSE_F32) {
        auto* out = reinterpret_cast<SecantCubinToggleSSERecipe*>(recipe_ret);
        out->num_kernels = plan->num_kernels; out->asts_per_kernel = plan->asts_per_kernel; out->num_inputs = plan->num_inputs;
        out->num_constants = plan->num_constants; out->num_targets = plan->num_targets; out->tile_rows = plan->tile_rows;
        out->threads_per_block = plan->threads_per_block; out->patch_capacity_instructions = plan->patch_capacity_instructions;
    } else {
        auto* out = reinterpret_cast<SecantCubinSSERecipe*>(recipe_ret);
        out->num_kernels = plan->num_kernels; out->asts_per_kernel = plan->asts_per_kernel; out->num_inputs = plan->num_inputs;
        out->num_targets = plan->num_targets; out->tile_rows = plan->tile_rows; out->threads_per_block = plan->threads_per_block;
        out->patch_capacity_instructions = plan->patch_capacity_instructions;
    }
    return SECANT_SUCCESS;
}

/* Validates the programs the way the reference's single-pass specializer would reject them
 * (s_cubin_specialize.c:1791-1860, 1990-2017); the binary is not modified. */
SecantResult secant_cubin_specialize_into(const SecantCubinPlan* plan, const SecantAstProgramSet* programs, void* cubin,
                                          size_t cubin_size) {
    size_t capacity;
    if (!plan || plan->magic != kPlanMagic || !programs || !cubin || !programs->asts.items || !programs->asts.count ||
        (programs->routines.count && !programs->routines.items) || programs->routines.count > SECANT_AST_MAX_ROUTINES ||
        !mul_ok(plan->num_kernels, plan->asts_per_kernel, &capacity) || programs->asts.count > capacity)
        return SECANT_ERROR_INVALID_VALUE;
    if (cubin_size != plan->cubin_size)
        return cubin_size < plan->cubin_size ? SECANT_ERROR_INSUFFICIENT_BUFFER : SECANT_ERROR_INVALID_VALUE;
    uint8_t arity[SECANT_AST_MAX_ROUTINES];
    SecantResult r = routine_arities(programs->routines, arity);
    if (r != SECANT_SUCCESS) return r;
    ProgramRules rules;
    rules.num_columns = plan->num_inputs;
    rules.num_constants = plan->num_constants;
    rules.banks_allowed = plan->shape == SECANT_KERNEL_SHAPE_TOGGLE_SSE_F32;
    rules.toggle_bits = 32; /* the specializer itself only bounds toggle bits by 32 */
    EncodedBatch scratch;
    for (size_t i = 0; i < programs->asts.count; ++i) {
        scratch.clear();
        r = encode_program(programs->asts.items[i], programs->routines, arity, rules, scratch);
        if (r != SECANT_SUCCESS) return r;
    }
    return SECANT_SUCCESS;
}

/* No host evaluator is shipped: a valid request is answered with BACKEND_UNAVAILABLE
 * after the same header checks the reference performs (s_cpu.c:919-957). */
SecantResult secant_cpu_run(const SecantCpuRunHeader* run) {
    if (!run || run->struct_size < sizeof(*run)) return SECANT_ERROR_INVALID_VALUE;
    if (run->version != SECANT_CPU_RUN_VERSION_3) return SECANT_ERROR_UNSUPPORTED_VERSION;
    if (run->flags) return SECANT_ERROR_INVALID_VALUE;
    size_t need;
    switch (run->shape) {
    case SECANT_KERNEL_SHAPE_STATIC_MATERIALIZE_F32: need = sizeof(SecantCpuMaterializeRun); break;
    case SECANT_KERNEL_SHAPE_STATIC_SSE_F32: need = sizeof(SecantCpuSSERun); break;
    case SECANT_KERNEL_SHAPE_STATIC_AFFINE_STATS_F32: need = sizeof(SecantCpuAffineStatsRun); break;
    case SECANT_KERNEL_SHAPE_STATIC_GRAM_STATS_F32: need = sizeof(SecantCpuGramStatsRun); break;
    case SECANT_KERNEL_SHAPE_TOGGLE_SSE_F32: need = sizeof(SecantCpuToggleSSERun); break;
    default: return SECANT_ERROR_UNSUPPORTED_SHAPE;
    }
    if (run->struct_size < need) return SECANT_ERROR_INVALID_VALUE;
    return SECANT_ERROR_BACKEND_UNAVAILABLE;
}

}  // extern "C"
