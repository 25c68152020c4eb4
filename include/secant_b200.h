/*
 * secant_b200.h - C ABI of the B200-native Secant population evaluator.
 *
 * Every type, constant and exported function in the first part of this header is
 * layout- and value-compatible with the reference engine's public header
 * (projects/secant/secant.h and projects/secant/secant_instructions.h, version 0.3.1),
 * so a caller built against that header can link this library unchanged.  Each block
 * cites the reference lines it mirrors.  The second part ("B200 extensions") adds entry
 * points the reference has no counterpart for; they are all prefixed secant_b200_.
 *
 * Conventions shared by all descriptors (reference secant.h:42-56): descriptors start
 * with {struct_size, version, shape, flags}; an unknown version gives
 * SECANT_ERROR_UNSUPPORTED_VERSION, an unknown shape SECANT_ERROR_UNSUPPORTED_SHAPE,
 * non-zero flags or a short struct_size SECANT_ERROR_INVALID_VALUE; a larger
 * struct_size is accepted and trailing bytes are ignored.  Sizes and strides count
 * elements, not bytes.  All matrices are f32, column-major [column][row].
 */
#ifndef SECANT_B200_H_INCLUDED
#define SECANT_B200_H_INCLUDED

#include <stddef.h>
#include <stdint.h>
#include <string.h>

#if defined(__GNUC__) || defined(__clang__)
#define SECANT_B200_VISIBLE __attribute__((visibility("default")))
#else
#define SECANT_B200_VISIBLE
#endif
#ifdef __cplusplus
#define SECANT_DEC extern "C" SECANT_B200_VISIBLE
#define SECANT_B200_ZERO_INIT(T, v) T v = T()
#else
#define SECANT_DEC extern SECANT_B200_VISIBLE
#define SECANT_B200_ZERO_INIT(T, v) T v = {0}
#endif

#define SECANT_VERSION_MAJOR 0u
#define SECANT_VERSION_MINOR 3u
#define SECANT_VERSION_PATCH 1u
#define SECANT_VERSION_STRING "0.3.1"

/* ---- result codes (secant.h:92-131) -------------------------------------------- */
typedef int32_t SecantResult;
enum {
    SECANT_SUCCESS = 0, SECANT_ERROR_INVALID_VALUE, SECANT_ERROR_OVERFLOW,
    SECANT_ERROR_INSUFFICIENT_BUFFER, SECANT_ERROR_FORMAT, SECANT_ERROR_ALLOCATION_FAILED,
    SECANT_ERROR_COMPILE_FAILED, SECANT_ERROR_PARSE_FAILED, SECANT_ERROR_SKELETON_NOT_FOUND,
    SECANT_ERROR_BAD_PROGRAM, SECANT_ERROR_STACK_OVERFLOW, SECANT_ERROR_STACK_UNDERFLOW,
    SECANT_ERROR_TOO_MANY_ARGS, SECANT_ERROR_UNSUPPORTED_OP,
    SECANT_ERROR_ROUTINE_IDX_OUT_OF_BOUNDS, SECANT_ERROR_ROUTINE_ARG_IDX_OUT_OF_BOUNDS,
    SECANT_ERROR_ROUTINE_DEPTH_EXCEEDED, SECANT_ERROR_INSUFFICIENT_PATCH_SPACE,
    SECANT_ERROR_REGISTER_OVERFLOW, SECANT_ERROR_UNSUPPORTED_ARCHITECTURE,
    SECANT_ERROR_INVALID_STATE, SECANT_ERROR_UNSUPPORTED_SHAPE,
    SECANT_ERROR_UNEXPECTED_INSTRUCTION, SECANT_ERROR_BACKEND_UNAVAILABLE,
    SECANT_ERROR_BAD_BINARY, SECANT_ERROR_BAD_PATCH_SITE, SECANT_ERROR_FUNCTION_NOT_FOUND,
    SECANT_ERROR_PATCH_SITE_NOT_FOUND, SECANT_ERROR_REGISTER_COUNT_NOT_FOUND,
    SECANT_ERROR_THREAD_FAILED, SECANT_ERROR_DRIVER_FAILED,
    SECANT_ERROR_EAGER_LOADING_REQUIRED, SECANT_ERROR_UNSUPPORTED_VERSION,
    SECANT_ERROR_COMPLETION_UNKNOWN, SECANT_RESULT_COUNT,
    SECANT_RESULT_NUM_ENUMS = SECANT_RESULT_COUNT
};

/* ---- program bytecode (secant.h:133-207, secant_instructions.h:41-48) ---------- */
typedef uint8_t SecantAstInstruction;
typedef uint8_t SecantAstIdx;
typedef uint8_t SecantAstInstructionType;

/* Opcode bytes.  The s32/u32 ranges 0x96-0xb5 are reserved: decodable, never evaluated. */
#define SECANT_B200_OP(name, value) SECANT_AST_INSTRUCTION_TYPE_##name = value
enum {
    SECANT_B200_OP(NONE, 0x80), SECANT_B200_OP(CONSTANT_BITS_F32, 0x81),
    SECANT_B200_OP(ROUTINE_F32, 0x82), SECANT_B200_OP(RETURN_F32, 0x83),
    SECANT_B200_OP(ROUTINE_ARG_F32, 0x84), SECANT_B200_OP(ADD_F32, 0x85),
    SECANT_B200_OP(SUB_F32, 0x86), SECANT_B200_OP(MUL_F32, 0x87), SECANT_B200_OP(DIV_F32, 0x88),
    SECANT_B200_OP(NEG_F32, 0x89), SECANT_B200_OP(SQRT_F32, 0x8a), SECANT_B200_OP(RCP_F32, 0x8b),
    SECANT_B200_OP(ABS_F32, 0x8c), SECANT_B200_OP(MIN_F32, 0x8d), SECANT_B200_OP(MAX_F32, 0x8e),
    SECANT_B200_OP(FMA_F32, 0x8f), SECANT_B200_OP(SIN_F32, 0x90), SECANT_B200_OP(COS_F32, 0x91),
    SECANT_B200_OP(EX2_F32, 0x92), SECANT_B200_OP(LG2_F32, 0x93), SECANT_B200_OP(RSQRT_F32, 0x94),
    SECANT_B200_OP(TANH_F32, 0x95),
    SECANT_B200_OP(INPUT_S32, 0x96), SECANT_B200_OP(CONSTANT_S32, 0x97),
    SECANT_B200_OP(ROUTINE_S32, 0x98), SECANT_B200_OP(RETURN_S32, 0x99),
    SECANT_B200_OP(ROUTINE_ARG_S32, 0x9a), SECANT_B200_OP(ADD_S32, 0x9b),
    SECANT_B200_OP(SUB_S32, 0x9c), SECANT_B200_OP(MUL_S32, 0x9d), SECANT_B200_OP(DIV_S32, 0x9e),
    SECANT_B200_OP(NEG_S32, 0x9f), SECANT_B200_OP(ABS_S32, 0xa0), SECANT_B200_OP(MIN_S32, 0xa1),
    SECANT_B200_OP(MAX_S32, 0xa2), SECANT_B200_OP(FMA_S32, 0xa3),
    SECANT_B200_OP(INPUT_U32, 0xa4), SECANT_B200_OP(CONSTANT_U32, 0xa5),
    SECANT_B200_OP(ROUTINE_U32, 0xa6), SECANT_B200_OP(RETURN_U32, 0xa7),
    SECANT_B200_OP(ROUTINE_ARG_U32, 0xa8), SECANT_B200_OP(ADD_U32, 0xa9),
    SECANT_B200_OP(SUB_U32, 0xaa), SECANT_B200_OP(MUL_U32, 0xab), SECANT_B200_OP(DIV_U32, 0xac),
    SECANT_B200_OP(MIN_U32, 0xad), SECANT_B200_OP(MAX_U32, 0xae), SECANT_B200_OP(FMA_U32, 0xaf),
    SECANT_B200_OP(AND_U32, 0xb0), SECANT_B200_OP(OR_U32, 0xb1), SECANT_B200_OP(XOR_U32, 0xb2),
    SECANT_B200_OP(NOT_U32, 0xb3), SECANT_B200_OP(SHL_U32, 0xb4), SECANT_B200_OP(SHR_U32, 0xb5),
    SECANT_B200_OP(COLUMN_F32, 0xb6),            /* 0xb7-0xb9 are retired and invalid */
    SECANT_B200_OP(EXP_F32, 0xba), SECANT_B200_OP(LOG_F32, 0xbb),
    SECANT_B200_OP(BANK_CONSTANT_F32, 0xbc), SECANT_B200_OP(TOGGLE2_F32, 0xbd),
    SECANT_B200_OP(TOGGLE4_F32, 0xbe), SECANT_B200_OP(AFFINE_BANK_F32, 0xbf),
    SECANT_B200_OP(ONE_PAST_LAST, 0xc0),
    SECANT_AST_INSTRUCTION_TYPE_NUM_ENUMS = SECANT_AST_INSTRUCTION_TYPE_ONE_PAST_LAST
};

#define SECANT_AST_MAX_PROGRAM_INSTRUCTIONS 1024u
#define SECANT_AST_MAX_INSTRUCTION_BYTES 10u
#define SECANT_AST_MAX_PROGRAM_BYTES (SECANT_AST_MAX_PROGRAM_INSTRUCTIONS * SECANT_AST_MAX_INSTRUCTION_BYTES)
#define SECANT_AST_MAX_STACK_DEPTH 128u
#define SECANT_AST_MAX_INSTRUCTION_ARGS 4u
#define SECANT_AST_MAX_INPUTS 128u
#define SECANT_AST_MAX_TOGGLE_BITS 32u
#define SECANT_AST_MAX_ROUTINES 255u

/* Bit patterns of a few f32 literals (secant_instructions.h:50-63). */
#define SECANT_F32_BITS_POSITIVE_ZERO 0x00000000u
#define SECANT_F32_BITS_NEGATIVE_ZERO 0x80000000u
#define SECANT_F32_BITS_ONE_MILLIONTH 0x358637bdu
#define SECANT_F32_BITS_ONE_HUNDREDTH 0x3c23d70au
#define SECANT_F32_BITS_QUARTER 0x3e800000u
#define SECANT_F32_BITS_HALF 0x3f000000u
#define SECANT_F32_BITS_ONE 0x3f800000u
#define SECANT_F32_BITS_ONE_AND_HALF 0x3fc00000u
#define SECANT_F32_BITS_TWO 0x40000000u
#define SECANT_F32_BITS_TWO_AND_HALF 0x40200000u
#define SECANT_F32_BITS_NEGATIVE_ONE 0xbf800000u
#define SECANT_F32_BITS_PI 0x40490fdbu
#define SECANT_F32_BITS_LN_TWO 0x3f317218u
#define SECANT_F32_BITS_LOG2_E 0x3fb8aa3bu

/* Encoded width of the instruction starting at p, 0 for an invalid opcode
 * (secant_instructions.h:86-120): affine-bank leaf 10 bytes, scalar literal 5,
 * indexed tokens 2, four-way toggle 3, everything else 1. */
static inline size_t secant_ast_instruction_size_get(const SecantAstInstruction* p) {
    const unsigned op = p[0];
    if (op == SECANT_AST_INSTRUCTION_TYPE_AFFINE_BANK_F32) return 10u;
    if (op == SECANT_AST_INSTRUCTION_TYPE_CONSTANT_BITS_F32 || op == SECANT_AST_INSTRUCTION_TYPE_CONSTANT_S32 ||
        op == SECANT_AST_INSTRUCTION_TYPE_CONSTANT_U32) return 5u;
    if (op == SECANT_AST_INSTRUCTION_TYPE_TOGGLE4_F32) return 3u;
    if (op == SECANT_AST_INSTRUCTION_TYPE_ROUTINE_F32 || op == SECANT_AST_INSTRUCTION_TYPE_ROUTINE_ARG_F32 ||
        op == SECANT_AST_INSTRUCTION_TYPE_BANK_CONSTANT_F32 || op == SECANT_AST_INSTRUCTION_TYPE_TOGGLE2_F32 ||
        op == SECANT_AST_INSTRUCTION_TYPE_COLUMN_F32 || op == SECANT_AST_INSTRUCTION_TYPE_INPUT_S32 ||
        op == SECANT_AST_INSTRUCTION_TYPE_ROUTINE_S32 || op == SECANT_AST_INSTRUCTION_TYPE_ROUTINE_ARG_S32 ||
        op == SECANT_AST_INSTRUCTION_TYPE_INPUT_U32 || op == SECANT_AST_INSTRUCTION_TYPE_ROUTINE_U32 ||
        op == SECANT_AST_INSTRUCTION_TYPE_ROUTINE_ARG_U32) return 2u;
    if (op >= 0xb7u && op <= 0xb9u) return 0u;
    return (op > SECANT_AST_INSTRUCTION_TYPE_NONE && op < SECANT_AST_INSTRUCTION_TYPE_ONE_PAST_LAST) ? 1u : 0u;
}
static inline SecantAstInstructionType secant_ast_instruction_type_get(const SecantAstInstruction* p) { return p[0]; }
static inline SecantAstIdx secant_ast_index_get(const SecantAstInstruction* p) { return p[1]; }
/* Little-endian 32-bit payload following the opcode byte (secant_instructions.h:145-152). */
static inline uint32_t secant_ast_constant_bits_get(const SecantAstInstruction* p) {
    return (uint32_t)p[1] | ((uint32_t)p[2] << 8) | ((uint32_t)p[3] << 16) | ((uint32_t)p[4] << 24);
}
static inline float secant_b200_bits_to_f32(uint32_t bits) { float f; memcpy(&f, &bits, 4); return f; }
static inline float secant_ast_constant_f32_get(const SecantAstInstruction* p) {
    return secant_b200_bits_to_f32(secant_ast_constant_bits_get(p));
}
/* Affine bank leaf = opcode, slot, scale bits, offset bits (secant_instructions.h:154-177). */
static inline float secant_ast_affine_bank_scale_get(const uint8_t* p) { return secant_b200_bits_to_f32(secant_ast_constant_bits_get(p + 1)); }
static inline float secant_ast_affine_bank_offset_get(const uint8_t* p) { return secant_b200_bits_to_f32(secant_ast_constant_bits_get(p + 5)); }
static inline void secant_ast_affine_bank_write(uint8_t* p, uint8_t slot, float scale, float offset) {
    uint32_t s, o; int i;
    memcpy(&s, &scale, 4); memcpy(&o, &offset, 4);
    p[0] = SECANT_AST_INSTRUCTION_TYPE_AFFINE_BANK_F32; p[1] = slot;
    for (i = 0; i < 4; ++i) { p[2 + i] = (uint8_t)(s >> (8 * i)); p[6 + i] = (uint8_t)(o >> (8 * i)); }
}

/* Initializer-list encoders (secant_instructions.h:253-322). */
#define SECANT_AST_ENCODE_U8(type_, value_) ((uint8_t)(type_)), ((uint8_t)(value_))
#define SECANT_AST_ENCODE_U32(type_, value_) ((uint8_t)(type_)), ((uint8_t)((uint32_t)(value_))), \
    ((uint8_t)((uint32_t)(value_) >> 8)), ((uint8_t)((uint32_t)(value_) >> 16)), ((uint8_t)((uint32_t)(value_) >> 24))
#define secant_ast_encode_column_f32(i) SECANT_AST_ENCODE_U8(SECANT_AST_INSTRUCTION_TYPE_COLUMN_F32, i)
#define secant_ast_encode_constant_f32_bits(b) SECANT_AST_ENCODE_U32(SECANT_AST_INSTRUCTION_TYPE_CONSTANT_BITS_F32, b)
#define secant_ast_encode_routine_f32(i) SECANT_AST_ENCODE_U8(SECANT_AST_INSTRUCTION_TYPE_ROUTINE_F32, i)
#define secant_ast_encode_routine_arg_f32(i) SECANT_AST_ENCODE_U8(SECANT_AST_INSTRUCTION_TYPE_ROUTINE_ARG_F32, i)
#define secant_ast_encode_bank_constant_f32(i) SECANT_AST_ENCODE_U8(SECANT_AST_INSTRUCTION_TYPE_BANK_CONSTANT_F32, i)
#define secant_ast_encode_toggle2_f32(bit) SECANT_AST_ENCODE_U8(SECANT_AST_INSTRUCTION_TYPE_TOGGLE2_F32, bit)
#define secant_ast_encode_toggle4_f32(b0, b1) ((uint8_t)SECANT_AST_INSTRUCTION_TYPE_TOGGLE4_F32), ((uint8_t)(b0)), ((uint8_t)(b1))
#define SECANT_B200_ENC1(lower, UPPER) ((uint8_t)SECANT_AST_INSTRUCTION_TYPE_##UPPER)
#define secant_ast_encode_add_f32 SECANT_B200_ENC1(add, ADD_F32)
#define secant_ast_encode_sub_f32 SECANT_B200_ENC1(sub, SUB_F32)
#define secant_ast_encode_mul_f32 SECANT_B200_ENC1(mul, MUL_F32)
#define secant_ast_encode_div_f32 SECANT_B200_ENC1(div, DIV_F32)
#define secant_ast_encode_neg_f32 SECANT_B200_ENC1(neg, NEG_F32)
#define secant_ast_encode_sqrt_f32 SECANT_B200_ENC1(sqrt, SQRT_F32)
#define secant_ast_encode_rcp_f32 SECANT_B200_ENC1(rcp, RCP_F32)
#define secant_ast_encode_abs_f32 SECANT_B200_ENC1(abs, ABS_F32)
#define secant_ast_encode_min_f32 SECANT_B200_ENC1(min, MIN_F32)
#define secant_ast_encode_max_f32 SECANT_B200_ENC1(max, MAX_F32)
#define secant_ast_encode_fma_f32 SECANT_B200_ENC1(fma, FMA_F32)
#define secant_ast_encode_sin_f32 SECANT_B200_ENC1(sin, SIN_F32)
#define secant_ast_encode_cos_f32 SECANT_B200_ENC1(cos, COS_F32)
#define secant_ast_encode_ex2_f32 SECANT_B200_ENC1(ex2, EX2_F32)
#define secant_ast_encode_lg2_f32 SECANT_B200_ENC1(lg2, LG2_F32)
#define secant_ast_encode_rsqrt_f32 SECANT_B200_ENC1(rsqrt, RSQRT_F32)
#define secant_ast_encode_tanh_f32 SECANT_B200_ENC1(tanh, TANH_F32)
#define secant_ast_encode_exp_f32 SECANT_B200_ENC1(exp, EXP_F32)
#define secant_ast_encode_log_f32 SECANT_B200_ENC1(log, LOG_F32)
#define secant_ast_encode_return_f32 SECANT_B200_ENC1(ret, RETURN_F32)

/* ---- shapes and descriptor versions (secant.h:209-243) -------------------------- */
typedef uint32_t SecantKernelShape;
enum {
    SECANT_KERNEL_SHAPE_NONE = 0u,
    SECANT_KERNEL_SHAPE_STATIC_MATERIALIZE_F32 = 1u,
    SECANT_KERNEL_SHAPE_STATIC_SSE_F32 = 2u,
    SECANT_KERNEL_SHAPE_STATIC_AFFINE_STATS_F32 = 5u,
    SECANT_KERNEL_SHAPE_STATIC_GRAM_STATS_F32 = 6u,
    SECANT_KERNEL_SHAPE_TOGGLE_SSE_F32 = 10u
};
enum { SECANT_AFFINE_AST_STAT_SUM_PREDICTION_F32 = 0u, SECANT_AFFINE_AST_STAT_SUM_PREDICTION_SQUARED_F32 = 1u,
       SECANT_AFFINE_AST_STAT_PREDICTION_TARGET_BASE_F32 = 2u };
enum { SECANT_AFFINE_TARGET_STAT_SUM_F32 = 0u, SECANT_AFFINE_TARGET_STAT_SUM_SQUARED_F32 = 1u,
       SECANT_AFFINE_TARGET_STAT_COUNT_F32 = 2u };
enum { SECANT_CUBIN_RECIPE_VERSION_3 = 3u, SECANT_CUBIN_RUN_VERSION_3 = 3u, SECANT_CPU_RUN_VERSION_3 = 3u,
       SECANT_CUBIN_RUNNER_OPTIONS_VERSION_1 = 1u, SECANT_CUBIN_PLAN_INFO_VERSION_1 = 1u,
       SECANT_RUNNER_STATS_VERSION_1 = 1u };

/* ---- borrowed views (secant.h:245-281, 506-520) --------------------------------- */
typedef struct SecantAstProgramList { const SecantAstInstruction* const* items; size_t count; } SecantAstProgramList;
typedef struct SecantAstProgramSet { SecantAstProgramList routines; SecantAstProgramList asts; } SecantAstProgramSet;
typedef struct SecantDeviceMatrixF32 { uintptr_t address; size_t num_elements; size_t leading_dimension; } SecantDeviceMatrixF32;
typedef struct SecantConstHostMatrixF32 { const float* data; size_t num_elements; size_t leading_dimension; } SecantConstHostMatrixF32;
typedef struct SecantHostMatrixF32 { float* data; size_t num_elements; size_t leading_dimension; } SecantHostMatrixF32;
/* Coefficient banks are [bank][slot] with bank_stride >= slots, shared by every program of a run. */
typedef struct SecantDeviceConstantBanks { uintptr_t address; size_t num_elements; size_t bank_stride; } SecantDeviceConstantBanks;
typedef struct SecantConstHostConstantBanks { const float* data; size_t num_elements; size_t bank_stride; } SecantConstHostConstantBanks;

/* ---- recipes (secant.h:283-394) ------------------------------------------------- */
typedef struct SecantCubinRecipeHeader { uint32_t struct_size, version; SecantKernelShape shape; uint32_t flags; } SecantCubinRecipeHeader;
typedef struct SecantCubinMaterializeRecipe {
    SecantCubinRecipeHeader header;
    size_t num_kernels, asts_per_kernel, num_inputs, patch_capacity_instructions;
} SecantCubinMaterializeRecipe;
#define SECANT_B200_TILED_RECIPE_FIELDS \
    SecantCubinRecipeHeader header; \
    size_t num_kernels, asts_per_kernel, num_inputs, num_targets, tile_rows, threads_per_block, patch_capacity_instructions
typedef struct SecantCubinSSERecipe { SECANT_B200_TILED_RECIPE_FIELDS; } SecantCubinSSERecipe;
typedef struct SecantCubinAffineStatsRecipe { SECANT_B200_TILED_RECIPE_FIELDS; } SecantCubinAffineStatsRecipe;
typedef struct SecantCubinGramStatsRecipe { SECANT_B200_TILED_RECIPE_FIELDS; } SecantCubinGramStatsRecipe;
typedef struct SecantCubinToggleSSERecipe {
    SecantCubinRecipeHeader header;
    size_t num_kernels, asts_per_kernel, num_inputs, num_constants, num_targets, tile_rows, threads_per_block,
        patch_capacity_instructions;
} SecantCubinToggleSSERecipe;

/* ---- device run requests (secant.h:396-540) ------------------------------------- */
typedef struct SecantCubinRunHeader { uint32_t struct_size, version; SecantKernelShape shape; uint32_t flags; } SecantCubinRunHeader;
/* Predictions [ast][row]; written, not accumulated. */
typedef struct SecantCubinMaterializeRun {
    SecantCubinRunHeader header; SecantAstProgramSet programs; SecantDeviceMatrixF32 input; size_t num_rows;
    SecantDeviceMatrixF32 output; size_t output_module_stride;
} SecantCubinMaterializeRun;
/* Sum of squared errors [ast][target]; the active range is cleared, then written. */
typedef struct SecantCubinSSERun {
    SecantCubinRunHeader header; SecantAstProgramSet programs; SecantDeviceMatrixF32 input, targets;
    size_t num_rows, num_targets; SecantDeviceMatrixF32 output;
} SecantCubinSSERun;
/* [ast][2 + target]: sum p, sum p*p, sum p*t per target. */
typedef struct SecantCubinAffineStatsRun {
    SecantCubinRunHeader header; SecantAstProgramSet programs; SecantDeviceMatrixF32 input, targets;
    size_t num_rows, num_targets; SecantDeviceMatrixF32 ast_stats;
} SecantCubinAffineStatsRun;
typedef struct SecantCubinGramStatsRun {
    SecantCubinRunHeader header; SecantAstProgramSet programs; SecantDeviceMatrixF32 input, targets;
    size_t num_rows, num_targets; SecantDeviceMatrixF32 statistics;
} SecantCubinGramStatsRun;
/* Raw SSE [ast][target][configuration], configuration = bank * 2^toggle_bits + permutation;
 * output.leading_dimension spans configurations and padding beyond them is preserved. */
typedef struct SecantCubinToggleSSERun {
    SecantCubinRunHeader header; SecantAstProgramSet programs; SecantDeviceMatrixF32 input, targets;
    SecantDeviceConstantBanks constants; size_t num_rows, num_targets, num_banks; uint32_t toggle_bits;
    SecantDeviceMatrixF32 output;
} SecantCubinToggleSSERun;

/* ---- host run requests (secant.h:542-633) --------------------------------------- */
typedef struct SecantCpuRunHeader { uint32_t struct_size, version; SecantKernelShape shape; uint32_t flags; } SecantCpuRunHeader;
typedef struct SecantCpuMaterializeRun {
    SecantCpuRunHeader header; SecantAstProgramSet programs; size_t num_inputs; SecantConstHostMatrixF32 input;
    size_t num_rows; SecantHostMatrixF32 output;
} SecantCpuMaterializeRun;
#define SECANT_B200_CPU_STATIC_FIELDS(out_name) \
    SecantCpuRunHeader header; SecantAstProgramSet programs; size_t num_inputs, num_targets; \
    SecantConstHostMatrixF32 input, targets; size_t num_rows; SecantHostMatrixF32 out_name
typedef struct SecantCpuSSERun { SECANT_B200_CPU_STATIC_FIELDS(output); } SecantCpuSSERun;
typedef struct SecantCpuAffineStatsRun { SECANT_B200_CPU_STATIC_FIELDS(ast_stats); } SecantCpuAffineStatsRun;
typedef struct SecantCpuGramStatsRun {
    SecantCpuRunHeader header; SecantAstProgramSet programs; size_t asts_per_cohort, num_inputs, num_targets;
    SecantConstHostMatrixF32 input, targets; size_t num_rows; SecantHostMatrixF32 statistics;
} SecantCpuGramStatsRun;
typedef struct SecantCpuToggleSSERun {
    SecantCpuRunHeader header; SecantAstProgramSet programs; size_t num_inputs, num_constants;
    SecantConstHostMatrixF32 input, targets; SecantConstHostConstantBanks constants;
    size_t num_rows, num_targets, num_banks; uint32_t toggle_bits; SecantHostMatrixF32 output;
} SecantCpuToggleSSERun;

/* ---- runner options, plan info, statistics (secant.h:635-685) ------------------- */
typedef struct SecantCubinRunnerOptions { uint32_t struct_size, version, flags, reserved; size_t num_workers, num_streams; } SecantCubinRunnerOptions;
typedef struct SecantCubinPlanInfo { uint32_t struct_size, version; SecantKernelShape shape; uint32_t flags; size_t cubin_size; } SecantCubinPlanInfo;
/* In this library "compile" seconds are program-encoding time, "module load" seconds are
 * record upload (host to device) time and "module unload" stays zero. */
typedef struct SecantRunnerStats {
    uint32_t struct_size, version, flags, reserved;
    size_t num_modules, num_asts, modules_loaded;
    double compile_window_seconds, compile_critical_seconds, compile_work_seconds, module_load_seconds,
        completion_wait_seconds, module_unload_seconds, runtime_seconds, total_seconds;
} SecantRunnerStats;
typedef struct SecantCubinPlan SecantCubinPlan;
typedef struct SecantCubinRunnerImpl* SecantCubinRunner;

/* ---- default initialisers (secant.h:718-949) ------------------------------------ */
#define SECANT_B200_INIT_HEADERED(fn, T, ver, shp) \
    static inline T fn(void) { SECANT_B200_ZERO_INIT(T, v); v.header.struct_size = (uint32_t)sizeof(v); \
        v.header.version = (ver); v.header.shape = (shp); return v; }
SECANT_B200_INIT_HEADERED(secant_cubin_materialize_recipe_init, SecantCubinMaterializeRecipe, SECANT_CUBIN_RECIPE_VERSION_3, SECANT_KERNEL_SHAPE_STATIC_MATERIALIZE_F32)
SECANT_B200_INIT_HEADERED(secant_cubin_sse_recipe_init, SecantCubinSSERecipe, SECANT_CUBIN_RECIPE_VERSION_3, SECANT_KERNEL_SHAPE_STATIC_SSE_F32)
SECANT_B200_INIT_HEADERED(secant_cubin_affine_stats_recipe_init, SecantCubinAffineStatsRecipe, SECANT_CUBIN_RECIPE_VERSION_3, SECANT_KERNEL_SHAPE_STATIC_AFFINE_STATS_F32)
SECANT_B200_INIT_HEADERED(secant_cubin_gram_stats_recipe_init, SecantCubinGramStatsRecipe, SECANT_CUBIN_RECIPE_VERSION_3, SECANT_KERNEL_SHAPE_STATIC_GRAM_STATS_F32)
SECANT_B200_INIT_HEADERED(secant_cubin_materialize_run_init, SecantCubinMaterializeRun, SECANT_CUBIN_RUN_VERSION_3, SECANT_KERNEL_SHAPE_STATIC_MATERIALIZE_F32)
SECANT_B200_INIT_HEADERED(secant_cubin_sse_run_init, SecantCubinSSERun, SECANT_CUBIN_RUN_VERSION_3, SECANT_KERNEL_SHAPE_STATIC_SSE_F32)
SECANT_B200_INIT_HEADERED(secant_cubin_affine_stats_run_init, SecantCubinAffineStatsRun, SECANT_CUBIN_RUN_VERSION_3, SECANT_KERNEL_SHAPE_STATIC_AFFINE_STATS_F32)
SECANT_B200_INIT_HEADERED(secant_cubin_gram_stats_run_init, SecantCubinGramStatsRun, SECANT_CUBIN_RUN_VERSION_3, SECANT_KERNEL_SHAPE_STATIC_GRAM_STATS_F32)
SECANT_B200_INIT_HEADERED(secant_cubin_toggle_sse_run_init, SecantCubinToggleSSERun, SECANT_CUBIN_RUN_VERSION_3, SECANT_KERNEL_SHAPE_TOGGLE_SSE_F32)
SECANT_B200_INIT_HEADERED(secant_cpu_materialize_run_init, SecantCpuMaterializeRun, SECANT_CPU_RUN_VERSION_3, SECANT_KERNEL_SHAPE_STATIC_MATERIALIZE_F32)
SECANT_B200_INIT_HEADERED(secant_cpu_sse_run_init, SecantCpuSSERun, SECANT_CPU_RUN_VERSION_3, SECANT_KERNEL_SHAPE_STATIC_SSE_F32)
SECANT_B200_INIT_HEADERED(secant_cpu_affine_stats_run_init, SecantCpuAffineStatsRun, SECANT_CPU_RUN_VERSION_3, SECANT_KERNEL_SHAPE_STATIC_AFFINE_STATS_F32)
SECANT_B200_INIT_HEADERED(secant_cpu_gram_stats_run_init, SecantCpuGramStatsRun, SECANT_CPU_RUN_VERSION_3, SECANT_KERNEL_SHAPE_STATIC_GRAM_STATS_F32)
SECANT_B200_INIT_HEADERED(secant_cpu_toggle_sse_run_init, SecantCpuToggleSSERun, SECANT_CPU_RUN_VERSION_3, SECANT_KERNEL_SHAPE_TOGGLE_SSE_F32)
/* The toggle recipe defaults to one program per kernel (secant.h:874-885). */
static inline SecantCubinToggleSSERecipe secant_cubin_toggle_sse_recipe_init(void) {
    SECANT_B200_ZERO_INIT(SecantCubinToggleSSERecipe, v);
    v.header.struct_size = (uint32_t)sizeof(v); v.header.version = SECANT_CUBIN_RECIPE_VERSION_3;
    v.header.shape = SECANT_KERNEL_SHAPE_TOGGLE_SSE_F32; v.asts_per_kernel = 1u; return v;
}
static inline SecantCubinRunnerOptions secant_cubin_runner_options_init(void) {
    SECANT_B200_ZERO_INIT(SecantCubinRunnerOptions, v);
    v.struct_size = (uint32_t)sizeof(v); v.version = SECANT_CUBIN_RUNNER_OPTIONS_VERSION_1;
    v.num_workers = 1u; v.num_streams = 1u; return v;
}
static inline SecantCubinPlanInfo secant_cubin_plan_info_init(void) {
    SECANT_B200_ZERO_INIT(SecantCubinPlanInfo, v);
    v.struct_size = (uint32_t)sizeof(v); v.version = SECANT_CUBIN_PLAN_INFO_VERSION_1; return v;
}
static inline SecantRunnerStats secant_runner_stats_init(void) {
    SECANT_B200_ZERO_INIT(SecantRunnerStats, v);
    v.struct_size = (uint32_t)sizeof(v); v.version = SECANT_RUNNER_STATS_VERSION_1; return v;
}

/* ---- exported functions --------------------------------------------------------- */

/* Symbolic name of a result code; replaces secant.h:688. */
SECANT_DEC const char* secant_result_to_string(SecantResult result);
/* CUDA source text of the dataset-level target-moment kernel
 * secant_cuda_target_stats_f32(targets, ld, rows, num_targets, stats, stats_ld); replaces secant.h:716. */
SECANT_DEC const char* secant_cuda_target_stats_f32_source_get(size_t* source_size_ret);
/* Full validation of a concrete recipe; replaces secant.h:957. */
SECANT_DEC SecantResult secant_cubin_recipe_validate(const SecantCubinRecipeHeader* recipe);
/* Size (with NUL) and text of a CUDA translation unit for the recipe; replace secant.h:966,984.
 * This library evaluates programs with its own resident kernels, so the text is a small
 * stub that compiles with NVRTC or nvcc and only carries the recipe tag. */
SECANT_DEC SecantResult secant_cubin_source_size(const SecantCubinRecipeHeader* recipe, size_t* required_size_ret);
SECANT_DEC SecantResult secant_cubin_source_write(const SecantCubinRecipeHeader* recipe, char* output, size_t output_size);
/* Plan storage measurement and initialisation; replace secant.h:1004,1030.  The binary the
 * caller compiled is not parsed: the plan records the recipe and cubin_size. */
SECANT_DEC SecantResult secant_cubin_plan_storage_size(const SecantCubinRecipeHeader* recipe, const void* cubin,
                                                       size_t cubin_size, size_t* required_storage_size_ret);
SECANT_DEC SecantResult secant_cubin_plan_init(const SecantCubinRecipeHeader* recipe, const void* cubin, size_t cubin_size,
                                               void* plan_storage, size_t plan_storage_size, SecantCubinPlan** plan_ret);
/* Plan queries; replace secant.h:1046,1062. */
SECANT_DEC SecantResult secant_cubin_plan_info_get(const SecantCubinPlan* plan, SecantCubinPlanInfo* info_ret);
SECANT_DEC SecantResult secant_cubin_plan_recipe_get(const SecantCubinPlan* plan, SecantCubinRecipeHeader* recipe_ret);
/* Structural validation of up to num_kernels * asts_per_kernel programs with the reference's
 * error codes; the binary is left untouched.  Replaces secant.h:1076. */
SECANT_DEC SecantResult secant_cubin_specialize_into(const SecantCubinPlan* plan, const SecantAstProgramSet* programs,
                                                     void* cubin, size_t cubin_size);
/* Runner lifecycle and the blocking hot entry; replace secant.h:1105,1126,1166,1187. */
SECANT_DEC SecantResult secant_cubin_runner_create(const SecantCubinPlan* plan, const void* cubin, size_t cubin_size,
                                                   const SecantCubinRunnerOptions* options, SecantCubinRunner* runner_ret);
SECANT_DEC SecantResult secant_cubin_runner_run_batch(SecantCubinRunner runner, const SecantCubinRunHeader* const* runs,
                                                      size_t num_runs, SecantRunnerStats* stats_ret);
SECANT_DEC SecantResult secant_cubin_runner_run(SecantCubinRunner runner, const SecantCubinRunHeader* run,
                                                SecantRunnerStats* stats_ret);
SECANT_DEC SecantResult secant_cubin_runner_destroy(SecantCubinRunner runner);
/* Host evaluation entry; replaces secant.h:1201.  This library has no host evaluator:
 * after header validation it returns SECANT_ERROR_BACKEND_UNAVAILABLE. */
SECANT_DEC SecantResult secant_cpu_run(const SecantCpuRunHeader* run);

/* Typed wrappers (secant.h:1203-1273). */
#define SECANT_B200_TYPED_RUN(fn, T) \
    static inline SecantResult fn(SecantCubinRunner r, const T* run, SecantRunnerStats* s) { \
        return run == NULL ? SECANT_ERROR_INVALID_VALUE : secant_cubin_runner_run(r, &run->header, s); }
SECANT_B200_TYPED_RUN(secant_cubin_runner_run_materialize, SecantCubinMaterializeRun)
SECANT_B200_TYPED_RUN(secant_cubin_runner_run_sse, SecantCubinSSERun)
SECANT_B200_TYPED_RUN(secant_cubin_runner_run_affine_stats, SecantCubinAffineStatsRun)
SECANT_B200_TYPED_RUN(secant_cubin_runner_run_gram_stats, SecantCubinGramStatsRun)
static inline SecantResult secant_cubin_runner_run_toggle_sse(SecantCubinRunner r, const SecantCubinToggleSSERun* run,
                                                              SecantRunnerStats* s) {
    return secant_cubin_runner_run(r, run ? &run->header : NULL, s);
}
#define SECANT_B200_TYPED_CPU(fn, T) \
    static inline SecantResult fn(const T* run) { return run == NULL ? SECANT_ERROR_INVALID_VALUE : secant_cpu_run(&run->header); }
SECANT_B200_TYPED_CPU(secant_cpu_run_materialize, SecantCpuMaterializeRun)
SECANT_B200_TYPED_CPU(secant_cpu_run_sse, SecantCpuSSERun)
SECANT_B200_TYPED_CPU(secant_cpu_run_affine_stats, SecantCpuAffineStatsRun)
SECANT_B200_TYPED_CPU(secant_cpu_run_gram_stats, SecantCpuGramStatsRun)
static inline SecantResult secant_cpu_run_toggle_sse(const SecantCpuToggleSSERun* run) { return secant_cpu_run(run ? &run->header : NULL); }

#include "secant_b200_ext.h"

#endif /* SECANT_B200_H_INCLUDED */
