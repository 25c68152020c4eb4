/*
 * secant_oracle.c - CPU restatement of the reference host evaluator.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker used by the test-suite, by the smoke test and by the CPU
 * baseline leg of the benchmark.  Nothing the shipped library does may call into it.
 *
 * It restates, in independent code, the algorithm of the reference's host evaluator:
 *   - one program on one row for one (bank, permutation):   projects/secant/s_cpu.c:193-414
 *   - routine arity discovery:                              projects/secant/s_cpu.c:129-191
 *   - static materialize / static SSE loops:                projects/secant/s_cpu.c:455-619
 *   - toggle SSE layout, validation order and loops:        projects/secant/s_cpu.c:851-917,
 *                                                           projects/secant/s_toggle_internal.h:44-71
 *   - affine statistics loop:                               projects/secant/s_cpu.c:683-720
 *   - best-configuration rule per program:                  projects/secant-sr/toggle/src/cpu.c:45-67
 *   - score ordering for top-k:                             projects/odezza/core/o_score_reduce.cu:36-39
 *   - fixed-step RK4 rollout scoring:                       projects/odezza/core/o_generate_scoring_cuda.c:494-588
 *
 * Parity pin: the functions below are checked against the reference's own fixtures
 * (tests/toggle_fixture.h closed forms, tests/toggle_test.c exact affine values and error
 * cases, tests/cpu_test.c closed forms) and, where the reference tree is available, against
 * the reference's s_cpu.c compiled unmodified (oracle/_ref/libsecant_ref.so).  The RK4
 * scorer has no general reference implementation to run; it is pinned on the reference's own
 * launch test data, closed-form value and invalid-data matrix
 * (projects/odezza/tests/o_scoring_cuda_test.c:97-186), parity otherwise unpinned.
 *
 * Arithmetic contract: IEEE binary32, libm for transcendental functions, no contraction
 * of a*b+c except where the program says FMA.  Compile with -ffp-contract=off.
 */
#include "../include/secant_b200.h"

#include <float.h>
#include <math.h>
#include <stdlib.h>

#define SO_EXPORT __attribute__((visibility("default")))
#define SO_ROUTINE_DEPTH 8u

typedef struct {
    const uint8_t* const* routines;
    size_t num_routines;
    const uint8_t* arity; /* per routine, number of arguments */
    size_t num_columns;
    size_t num_constants;
    const float* input;
    size_t input_ld;
    const float* constants; /* one bank vector, or NULL */
    uint32_t toggle_bits;
    uint32_t permutation;
    size_t row;
} SoEnv;

static int so_is_f32_op(unsigned op) {
    return op == 0xbf || op == 0xb6 || op == 0xbc || op == 0xbd || op == 0xbe || (op >= 0x81 && op <= 0x95) ||
           op == 0xba || op == 0xbb;
}

/* Number of operands an arithmetic opcode consumes, 0 if it is not arithmetic. */
static unsigned so_arity(unsigned op) {
    switch (op) {
    case SECANT_AST_INSTRUCTION_TYPE_ADD_F32: case SECANT_AST_INSTRUCTION_TYPE_SUB_F32:
    case SECANT_AST_INSTRUCTION_TYPE_MUL_F32: case SECANT_AST_INSTRUCTION_TYPE_DIV_F32:
    case SECANT_AST_INSTRUCTION_TYPE_MIN_F32: case SECANT_AST_INSTRUCTION_TYPE_MAX_F32:
        return 2;
    case SECANT_AST_INSTRUCTION_TYPE_FMA_F32:
        return 3;
    case SECANT_AST_INSTRUCTION_TYPE_NEG_F32: case SECANT_AST_INSTRUCTION_TYPE_SQRT_F32:
    case SECANT_AST_INSTRUCTION_TYPE_RCP_F32: case SECANT_AST_INSTRUCTION_TYPE_ABS_F32:
    case SECANT_AST_INSTRUCTION_TYPE_SIN_F32: case SECANT_AST_INSTRUCTION_TYPE_COS_F32:
    case SECANT_AST_INSTRUCTION_TYPE_EX2_F32: case SECANT_AST_INSTRUCTION_TYPE_LG2_F32:
    case SECANT_AST_INSTRUCTION_TYPE_RSQRT_F32: case SECANT_AST_INSTRUCTION_TYPE_TANH_F32:
    case SECANT_AST_INSTRUCTION_TYPE_EXP_F32: case SECANT_AST_INSTRUCTION_TYPE_LOG_F32:
        return 1;
    default:
        return 0;
    }
}

/* Test knob: when non-zero, every transcendental result (sin, cos, exp2, log2, tanh, exp,
 * log) is moved by that many units in the last place before it is used.  Evaluating a
 * program with the knob at +k and -k shows how far its value moves when the math library
 * differs by k ulp, i.e. how well-conditioned the comparison against another
 * implementation is.  The IEEE operations are never perturbed. */
static int so_ulp_shift = 0;
SO_EXPORT void so_set_ulp_shift(int ulps) { so_ulp_shift = ulps; }

static float so_shifted(float v) {
    int k = so_ulp_shift;
    if (!k || !isfinite(v)) return v;
    for (; k > 0; --k) v = nextafterf(v, INFINITY);
    for (; k < 0; ++k) v = nextafterf(v, -INFINITY);
    return v;
}

static float so_apply(unsigned op, const float* a) {
    switch (op) {
    case SECANT_AST_INSTRUCTION_TYPE_ADD_F32: return a[0] + a[1];
    case SECANT_AST_INSTRUCTION_TYPE_SUB_F32: return a[0] - a[1];
    case SECANT_AST_INSTRUCTION_TYPE_MUL_F32: return a[0] * a[1];
    case SECANT_AST_INSTRUCTION_TYPE_DIV_F32: return a[0] / a[1];
    case SECANT_AST_INSTRUCTION_TYPE_MIN_F32: return fminf(a[0], a[1]);
    case SECANT_AST_INSTRUCTION_TYPE_MAX_F32: return fmaxf(a[0], a[1]);
    case SECANT_AST_INSTRUCTION_TYPE_FMA_F32: return fmaf(a[0], a[1], a[2]);
    case SECANT_AST_INSTRUCTION_TYPE_NEG_F32: return -a[0];
    case SECANT_AST_INSTRUCTION_TYPE_SQRT_F32: return sqrtf(a[0]);
    case SECANT_AST_INSTRUCTION_TYPE_RCP_F32: return 1.0f / a[0];
    case SECANT_AST_INSTRUCTION_TYPE_ABS_F32: return fabsf(a[0]);
    case SECANT_AST_INSTRUCTION_TYPE_SIN_F32: return so_shifted(sinf(a[0]));
    case SECANT_AST_INSTRUCTION_TYPE_COS_F32: return so_shifted(cosf(a[0]));
    case SECANT_AST_INSTRUCTION_TYPE_EX2_F32: return so_shifted(exp2f(a[0]));
    case SECANT_AST_INSTRUCTION_TYPE_LG2_F32: return so_shifted(log2f(a[0]));
    case SECANT_AST_INSTRUCTION_TYPE_RSQRT_F32: return 1.0f / sqrtf(a[0]);
    case SECANT_AST_INSTRUCTION_TYPE_TANH_F32: return so_shifted(tanhf(a[0]));
    case SECANT_AST_INSTRUCTION_TYPE_EXP_F32: return so_shifted(expf(a[0]));
    default: return so_shifted(logf(a[0]));
    }
}

/* Highest ROUTINE_ARG index + 1 used by a routine body (s_cpu.c:129-165). */
static SecantResult so_routine_arity(const uint8_t* body, uint8_t* arity_ret) {
    size_t n, at = 0;
    unsigned arity = 0;
    if (!body) return SECANT_ERROR_INVALID_VALUE;
    for (n = 0; n < SECANT_AST_MAX_PROGRAM_INSTRUCTIONS; ++n) {
        const uint8_t* ins = body + at;
        size_t width = secant_ast_instruction_size_get(ins);
        if (!width) return SECANT_ERROR_BAD_PROGRAM;
        if (ins[0] == SECANT_AST_INSTRUCTION_TYPE_ROUTINE_ARG_F32) {
            if (ins[1] >= SECANT_AST_MAX_INSTRUCTION_ARGS) return SECANT_ERROR_TOO_MANY_ARGS;
            if (ins[1] + 1u > arity) arity = ins[1] + 1u;
        }
        if (ins[0] == SECANT_AST_INSTRUCTION_TYPE_RETURN_F32) {
            *arity_ret = (uint8_t)arity;
            return SECANT_SUCCESS;
        }
        at += width;
    }
    return SECANT_ERROR_BAD_PROGRAM;
}

static SecantResult so_arity_table(const uint8_t* const* routines, size_t count, uint8_t* table) {
    size_t i;
    if (count && !routines) return SECANT_ERROR_INVALID_VALUE;
    for (i = 0; i < count; ++i) {
        SecantResult r;
        if (!routines[i]) return SECANT_ERROR_ROUTINE_IDX_OUT_OF_BOUNDS;
        r = so_routine_arity(routines[i], table + i);
        if (r != SECANT_SUCCESS) return r;
    }
    return SECANT_SUCCESS;
}

/* One frame of the stack interpreter (s_cpu.c:193-414).  Every frame owns a private
 * 128-entry value stack; routine calls recurse with the caller's top values as arguments. */
static SecantResult so_frame(const SoEnv* env, const uint8_t* code, const float* args, size_t num_args,
                             size_t depth, float* value_ret) {
    float stack[SECANT_AST_MAX_STACK_DEPTH];
    size_t top = 0, direct_run = 0, n, at = 0;
    if (!code || !value_ret || env->toggle_bits > 32u) return SECANT_ERROR_INVALID_VALUE;
    for (n = 0; n < SECANT_AST_MAX_PROGRAM_INSTRUCTIONS; ++n) {
        const uint8_t* ins = code + at;
        const unsigned op = ins[0];
        const size_t width = secant_ast_instruction_size_get(ins);
        int is_direct = 0;
        if (!width) return SECANT_ERROR_BAD_PROGRAM;
        if (!so_is_f32_op(op)) return SECANT_ERROR_UNSUPPORTED_OP;
        if (op == SECANT_AST_INSTRUCTION_TYPE_COLUMN_F32) {
            if (ins[1] >= env->num_columns || !env->input) return SECANT_ERROR_INVALID_VALUE;
            if (top == SECANT_AST_MAX_STACK_DEPTH) return SECANT_ERROR_STACK_OVERFLOW;
            stack[top++] = env->input[(size_t)ins[1] * env->input_ld + env->row];
            is_direct = 1;
        } else if (op == SECANT_AST_INSTRUCTION_TYPE_BANK_CONSTANT_F32 || op == SECANT_AST_INSTRUCTION_TYPE_AFFINE_BANK_F32) {
            if (ins[1] >= env->num_constants || !env->constants) return SECANT_ERROR_BAD_PROGRAM;
            if (top == SECANT_AST_MAX_STACK_DEPTH) return SECANT_ERROR_STACK_OVERFLOW;
            if (op == SECANT_AST_INSTRUCTION_TYPE_AFFINE_BANK_F32) {
                const float scale = secant_ast_affine_bank_scale_get(ins);
                const float offset = secant_ast_affine_bank_offset_get(ins);
                volatile float scaled; /* force the product to round before the add */
                if (!isfinite(scale) || !isfinite(offset)) return SECANT_ERROR_BAD_PROGRAM;
                scaled = env->constants[ins[1]] * scale;
                stack[top++] = scaled + offset;
            } else {
                stack[top++] = env->constants[ins[1]];
            }
            is_direct = 1;
        } else if (op == SECANT_AST_INSTRUCTION_TYPE_CONSTANT_BITS_F32) {
            if (top == SECANT_AST_MAX_STACK_DEPTH) return SECANT_ERROR_STACK_OVERFLOW;
            stack[top++] = secant_ast_constant_f32_get(ins);
            is_direct = 1;
        } else if (op == SECANT_AST_INSTRUCTION_TYPE_TOGGLE2_F32 || op == SECANT_AST_INSTRUCTION_TYPE_TOGGLE4_F32) {
            const size_t ways = op == SECANT_AST_INSTRUCTION_TYPE_TOGGLE2_F32 ? 2u : 4u;
            unsigned pick;
            if (ins[1] >= env->toggle_bits || direct_run < ways || top < ways) return SECANT_ERROR_BAD_PROGRAM;
            pick = (env->permutation >> ins[1]) & 1u;
            if (ways == 4u) {
                if (ins[2] >= env->toggle_bits || ins[2] == ins[1]) return SECANT_ERROR_BAD_PROGRAM;
                pick |= ((env->permutation >> ins[2]) & 1u) << 1;
            }
            stack[top - ways] = stack[top - ways + pick];
            top -= ways - 1u;
        } else if (op == SECANT_AST_INSTRUCTION_TYPE_ROUTINE_ARG_F32) {
            if (!args || ins[1] >= num_args) return SECANT_ERROR_ROUTINE_ARG_IDX_OUT_OF_BOUNDS;
            if (top == SECANT_AST_MAX_STACK_DEPTH) return SECANT_ERROR_STACK_OVERFLOW;
            stack[top++] = args[ins[1]];
        } else if (op == SECANT_AST_INSTRUCTION_TYPE_ROUTINE_F32) {
            size_t want;
            float result;
            SecantResult r;
            if (ins[1] >= env->num_routines || !env->routines[ins[1]]) return SECANT_ERROR_ROUTINE_IDX_OUT_OF_BOUNDS;
            if (depth >= SO_ROUTINE_DEPTH) return SECANT_ERROR_ROUTINE_DEPTH_EXCEEDED;
            want = env->arity[ins[1]];
            if (top < want) return SECANT_ERROR_STACK_UNDERFLOW;
            r = so_frame(env, env->routines[ins[1]], stack + (top - want), want, depth + 1u, &result);
            if (r != SECANT_SUCCESS) return r;
            top -= want;
            stack[top++] = result;
        } else if (op == SECANT_AST_INSTRUCTION_TYPE_RETURN_F32) {
            if (top != 1u) return SECANT_ERROR_BAD_PROGRAM;
            *value_ret = stack[0];
            return SECANT_SUCCESS;
        } else {
            const unsigned want = so_arity(op);
            float result;
            if (!want) return SECANT_ERROR_BAD_PROGRAM; /* NONE and anything non-evaluable */
            if (top < want) return SECANT_ERROR_STACK_UNDERFLOW;
            result = so_apply(op, stack + (top - want));
            top -= want;
            stack[top++] = result;
        }
        direct_run = is_direct ? direct_run + 1u : 0u;
        at += width;
    }
    return SECANT_ERROR_BAD_PROGRAM;
}

/* ---- small helpers shared by the run functions ---------------------------------- */

static int so_mul(size_t a, size_t b, size_t* out) {
    if (a && b > SIZE_MAX / a) return 0;
    *out = a * b;
    return 1;
}
/* Elements spanned by `count` vectors of `width` elements, `stride` apart; 0 when empty. */
static int so_span(size_t count, size_t stride, size_t width, size_t* out) {
    size_t lead;
    if (!count || !width) { *out = 0; return 1; }
    if (stride < width || !so_mul(count - 1, stride, &lead) || width > SIZE_MAX - lead) return 0;
    *out = lead + width;
    return 1;
}
static SecantResult so_disjoint(const void* const* ptr, const size_t* elements, size_t count) {
    uintptr_t lo[8], hi[8];
    size_t i, j, bytes;
    for (i = 0; i < count; ++i) {
        if (!ptr[i] || !so_mul(elements[i], 4u, &bytes)) return SECANT_ERROR_OVERFLOW;
        lo[i] = (uintptr_t)ptr[i];
        if (bytes > UINTPTR_MAX - lo[i]) return SECANT_ERROR_OVERFLOW;
        hi[i] = lo[i] + bytes;
    }
    for (i = 0; i < count; ++i)
        for (j = i + 1; j < count; ++j)
            if (lo[i] < hi[j] && lo[j] < hi[i]) return SECANT_ERROR_INVALID_VALUE;
    return SECANT_SUCCESS;
}

typedef struct {
    const uint8_t** routines;
    const uint8_t** asts;
    uint8_t arity[SECANT_AST_MAX_ROUTINES];
} SoPrograms;

/* Programs arrive as one byte blob plus start offsets (friendly to ctypes callers). */
static SecantResult so_programs_open(SoPrograms* p, const uint8_t* routine_blob, const uint64_t* routine_off,
                                     size_t num_routines, const uint8_t* ast_blob, const uint64_t* ast_off,
                                     size_t num_asts) {
    size_t i;
    p->routines = NULL;
    p->asts = NULL;
    if (num_routines > SECANT_AST_MAX_ROUTINES || !num_asts || !ast_blob || !ast_off) return SECANT_ERROR_INVALID_VALUE;
    p->routines = (const uint8_t**)calloc(num_routines ? num_routines : 1, sizeof(*p->routines));
    p->asts = (const uint8_t**)calloc(num_asts, sizeof(*p->asts));
    if (!p->routines || !p->asts) return SECANT_ERROR_ALLOCATION_FAILED;
    for (i = 0; i < num_routines; ++i) p->routines[i] = routine_blob + routine_off[i];
    for (i = 0; i < num_asts; ++i) p->asts[i] = ast_blob + ast_off[i];
    return so_arity_table(p->routines, num_routines, p->arity);
}
static void so_programs_close(SoPrograms* p) {
    free((void*)p->routines);
    free((void*)p->asts);
}

/* ---- static materialize: predictions [ast][row] (s_cpu.c:455-522) ---------------- */
SO_EXPORT SecantResult so_materialize(const uint8_t* routine_blob, const uint64_t* routine_off, size_t num_routines,
                                      const uint8_t* ast_blob, const uint64_t* ast_off, size_t num_asts,
                                      size_t num_inputs, const float* input, size_t input_ld, size_t num_rows,
                                      float* output, size_t output_ld) {
    SoPrograms p;
    SoEnv env;
    size_t a, row;
    SecantResult r;
    if (!num_inputs || num_inputs > SECANT_AST_MAX_INPUTS || !input || !output || !num_rows || input_ld < num_rows ||
        output_ld < num_rows)
        return SECANT_ERROR_INVALID_VALUE;
    r = so_programs_open(&p, routine_blob, routine_off, num_routines, ast_blob, ast_off, num_asts);
    memset(&env, 0, sizeof(env));
    env.routines = p.routines; env.num_routines = num_routines; env.arity = p.arity;
    env.num_columns = num_inputs; env.input = input; env.input_ld = input_ld;
    for (a = 0; r == SECANT_SUCCESS && a < num_asts; ++a)
        for (row = 0; r == SECANT_SUCCESS && row < num_rows; ++row) {
            env.row = row;
            r = so_frame(&env, p.asts[a], NULL, 0, 0, output + a * output_ld + row);
        }
    so_programs_close(&p);
    return r;
}

/* ---- static SSE (s_cpu.c:524-619): rows outer, programs inner, ACCUMULATES into output.
 * output64, when given, receives the same sums accumulated in binary64 (each squared
 * error is still computed in binary32). */
SO_EXPORT SecantResult so_sse(const uint8_t* routine_blob, const uint64_t* routine_off, size_t num_routines,
                              const uint8_t* ast_blob, const uint64_t* ast_off, size_t num_asts, size_t num_inputs,
                              size_t num_targets, const float* input, size_t input_ld, const float* targets,
                              size_t targets_ld, size_t num_rows, float* output, size_t output_ld, double* output64) {
    SoPrograms p;
    SoEnv env;
    size_t a, t, row;
    SecantResult r;
    if (!num_inputs || num_inputs > SECANT_AST_MAX_INPUTS || !num_targets || !input || !targets || !output ||
        !num_rows || input_ld < num_rows || targets_ld < num_rows || output_ld < num_targets)
        return SECANT_ERROR_INVALID_VALUE;
    r = so_programs_open(&p, routine_blob, routine_off, num_routines, ast_blob, ast_off, num_asts);
    memset(&env, 0, sizeof(env));
    env.routines = p.routines; env.num_routines = num_routines; env.arity = p.arity;
    env.num_columns = num_inputs; env.input = input; env.input_ld = input_ld;
    for (row = 0; r == SECANT_SUCCESS && row < num_rows; ++row)
        for (a = 0; r == SECANT_SUCCESS && a < num_asts; ++a) {
            float value;
            env.row = row;
            r = so_frame(&env, p.asts[a], NULL, 0, 0, &value);
            if (r != SECANT_SUCCESS) break;
            for (t = 0; t < num_targets; ++t) {
                const float err = value - targets[t * targets_ld + row];
                const float sq = err * err;
                output[a * output_ld + t] += sq;
                if (output64) output64[a * output_ld + t] += (double)sq;
            }
        }
    so_programs_close(&p);
    return r;
}

/* ---- affine statistics (s_cpu.c:683-720): [ast][2+target] += {p, p*p, p*t...} ---- */
SO_EXPORT SecantResult so_affine_stats(const uint8_t* routine_blob, const uint64_t* routine_off, size_t num_routines,
                                       const uint8_t* ast_blob, const uint64_t* ast_off, size_t num_asts,
                                       size_t num_inputs, size_t num_targets, const float* input, size_t input_ld,
                                       const float* targets, size_t targets_ld, size_t num_rows, float* stats,
                                       size_t stats_ld, double* stats64) {
    SoPrograms p;
    SoEnv env;
    size_t a, t, row;
    SecantResult r;
    if (!num_inputs || num_inputs > SECANT_AST_MAX_INPUTS || !num_targets || !input || !targets || !stats ||
        !num_rows || input_ld < num_rows || targets_ld < num_rows || stats_ld < 2 + num_targets)
        return SECANT_ERROR_INVALID_VALUE;
    r = so_programs_open(&p, routine_blob, routine_off, num_routines, ast_blob, ast_off, num_asts);
    memset(&env, 0, sizeof(env));
    env.routines = p.routines; env.num_routines = num_routines; env.arity = p.arity;
    env.num_columns = num_inputs; env.input = input; env.input_ld = input_ld;
    for (row = 0; r == SECANT_SUCCESS && row < num_rows; ++row)
        for (a = 0; r == SECANT_SUCCESS && a < num_asts; ++a) {
            float value, sq;
            env.row = row;
            r = so_frame(&env, p.asts[a], NULL, 0, 0, &value);
            if (r != SECANT_SUCCESS) break;
            sq = value * value;
            stats[a * stats_ld + 0] += value;
            stats[a * stats_ld + 1] += sq;
            if (stats64) { stats64[a * stats_ld + 0] += value; stats64[a * stats_ld + 1] += sq; }
            for (t = 0; t < num_targets; ++t) {
                const float cross = value * targets[t * targets_ld + row];
                stats[a * stats_ld + 2 + t] += cross;
                if (stats64) stats64[a * stats_ld + 2 + t] += cross;
            }
        }
    so_programs_close(&p);
    return r;
}

/* ---- Gram statistics (s_cpu.c:724-848): programs in consecutive cohorts of `cohort`; per cohort
 * [0, A) sums, [A, A + A*A) row-major Gram matrix, then [feature][target] cross sums, all added
 * to the caller's values row after row in float32 (products rounded first) ---- */
SO_EXPORT SecantResult so_gram_stats(const uint8_t* routine_blob, const uint64_t* routine_off, size_t num_routines,
                                     const uint8_t* ast_blob, const uint64_t* ast_off, size_t num_asts, size_t cohort,
                                     size_t num_inputs, size_t num_targets, const float* input, size_t input_ld,
                                     const float* targets, size_t targets_ld, size_t num_rows, float* stats,
                                     size_t stats_ld, double* stats64) {
    SoPrograms p;
    SoEnv env;
    float features[32];
    size_t c, i, j, t, row;
    SecantResult r;
    if (!cohort || cohort > 32 || !num_inputs || num_inputs > SECANT_AST_MAX_INPUTS || !num_targets || !num_asts || !input ||
        !targets || !stats || !num_rows || input_ld < num_rows || targets_ld < num_rows ||
        stats_ld < cohort * (1 + cohort + num_targets))
        return SECANT_ERROR_INVALID_VALUE;
    r = so_programs_open(&p, routine_blob, routine_off, num_routines, ast_blob, ast_off, num_asts);
    memset(&env, 0, sizeof(env));
    env.routines = p.routines; env.num_routines = num_routines; env.arity = p.arity;
    env.num_columns = num_inputs; env.input = input; env.input_ld = input_ld;
    for (c = 0; r == SECANT_SUCCESS && c * cohort < num_asts; ++c) {
        const size_t first = c * cohort, active = num_asts - first < cohort ? num_asts - first : cohort;
        float* out = stats + c * stats_ld;
        double* out64 = stats64 ? stats64 + c * stats_ld : NULL;
        for (row = 0; r == SECANT_SUCCESS && row < num_rows; ++row) {
            env.row = row;
            for (i = 0; i < active && r == SECANT_SUCCESS; ++i) {
                r = so_frame(&env, p.asts[first + i], NULL, 0, 0, &features[i]);
                if (r != SECANT_SUCCESS) break;
                out[i] += features[i];
                if (out64) out64[i] += features[i];
            }
            if (r != SECANT_SUCCESS) break;
            for (i = 0; i < active; ++i) {
                for (j = 0; j < active; ++j) {
                    const float product = features[i] * features[j];
                    out[cohort + i * cohort + j] += product;
                    if (out64) out64[cohort + i * cohort + j] += product;
                }
                for (t = 0; t < num_targets; ++t) {
                    const float cross = features[i] * targets[t * targets_ld + row];
                    out[cohort + cohort * cohort + i * num_targets + t] += cross;
                    if (out64) out64[cohort + cohort * cohort + i * num_targets + t] += cross;
                }
            }
        }
    }
    so_programs_close(&p);
    return r;
}

/* ---- toggle SSE (s_cpu.c:851-917) ------------------------------------------------
 * Output [ast][target][configuration], configuration = bank * 2^bits + permutation.
 * Order of checks: null/zero arguments -> layout -> leading dimensions -> span overflow ->
 * buffer sizes -> overlap -> routine table -> dry evaluation of every program on
 * (bank 0, permutation 0, row 0) -> only then clear active bins and accumulate.
 * program_bank_stride (elements) is an addition for per-program coefficient banks:
 * program a reads its banks from constants + a * program_bank_stride; 0 gives the
 * reference behaviour of one table shared by every program. */
SO_EXPORT SecantResult so_toggle_sse(const uint8_t* routine_blob, const uint64_t* routine_off, size_t num_routines,
                                     const uint8_t* ast_blob, const uint64_t* ast_off, size_t num_asts,
                                     size_t num_inputs, size_t num_constants, const float* input,
                                     size_t input_elements, size_t input_ld, const float* targets,
                                     size_t target_elements, size_t targets_ld, const float* constants,
                                     size_t constant_elements, size_t bank_stride, size_t program_bank_stride,
                                     size_t num_rows, size_t num_targets, size_t num_banks, uint32_t toggle_bits,
                                     float* output, size_t output_elements, size_t output_ld, double* output64) {
    SoPrograms p;
    SoEnv env;
    size_t configs, perms, bank_span = 0, input_span, target_span, output_span, pairs, a, b, q, t, row, nranges = 0;
    const void* ranges[4];
    size_t range_elements[4];
    SecantResult r;
    if (!ast_blob || !num_asts || !num_rows || !num_targets || num_inputs > SECANT_AST_MAX_INPUTS ||
        num_routines > SECANT_AST_MAX_ROUTINES)
        return SECANT_ERROR_INVALID_VALUE;
    if (!num_banks || toggle_bits > 32 || num_constants > SECANT_AST_MAX_INPUTS) return SECANT_ERROR_INVALID_VALUE;
    perms = (size_t)1 << toggle_bits;
    if (!so_mul(num_banks, perms, &configs)) return SECANT_ERROR_OVERFLOW;
    if (!num_constants) {
        if (bank_stride) return SECANT_ERROR_INVALID_VALUE;
    } else {
        if (bank_stride < num_constants) return SECANT_ERROR_INVALID_VALUE;
        if (!so_span(num_banks, bank_stride, num_constants, &bank_span)) return SECANT_ERROR_OVERFLOW;
        if (program_bank_stride) {
            size_t lead;
            if (!so_mul(num_asts - 1, program_bank_stride, &lead) || bank_span > SIZE_MAX - lead) return SECANT_ERROR_OVERFLOW;
            bank_span += lead;
        }
    }
    if ((num_inputs && input_ld < num_rows) || targets_ld < num_rows || output_ld < configs) return SECANT_ERROR_INVALID_VALUE;
    if (!so_span(num_inputs, input_ld, num_rows, &input_span) || !so_span(num_targets, targets_ld, num_rows, &target_span) ||
        !so_mul(num_asts, num_targets, &pairs) || !so_span(pairs, output_ld, configs, &output_span))
        return SECANT_ERROR_OVERFLOW;
    if (input_elements < input_span || target_elements < target_span || constant_elements < bank_span ||
        output_elements < output_span)
        return SECANT_ERROR_INSUFFICIENT_BUFFER;
#define SO_RANGE(ptr, span) do { if (span) { if (!(ptr)) return SECANT_ERROR_INVALID_VALUE; \
        ranges[nranges] = (ptr); range_elements[nranges++] = (span); } } while (0)
    SO_RANGE(input, input_span);
    SO_RANGE(constants, bank_span);
    SO_RANGE(targets, target_span);
    SO_RANGE(output, output_span);
#undef SO_RANGE
    r = so_disjoint(ranges, range_elements, nranges);
    if (r != SECANT_SUCCESS) return r;
    r = so_programs_open(&p, routine_blob, routine_off, num_routines, ast_blob, ast_off, num_asts);
    memset(&env, 0, sizeof(env));
    env.routines = p.routines; env.num_routines = num_routines; env.arity = p.arity;
    env.num_columns = num_inputs; env.num_constants = num_constants; env.input = input; env.input_ld = input_ld;
    env.toggle_bits = toggle_bits;
    for (a = 0; r == SECANT_SUCCESS && a < num_asts; ++a) { /* dry run before anything is cleared */
        float unused;
        env.constants = num_constants ? constants + a * program_bank_stride : NULL;
        env.permutation = 0; env.row = 0;
        r = so_frame(&env, p.asts[a], NULL, 0, 0, &unused);
    }
    for (a = 0; r == SECANT_SUCCESS && a < num_asts; ++a) {
        for (t = 0; t < num_targets; ++t) {
            memset(output + (a * num_targets + t) * output_ld, 0, configs * sizeof(float));
            if (output64) memset(output64 + (a * num_targets + t) * output_ld, 0, configs * sizeof(double));
        }
        for (b = 0; r == SECANT_SUCCESS && b < num_banks; ++b) {
            env.constants = num_constants ? constants + a * program_bank_stride + b * bank_stride : NULL;
            for (q = 0; r == SECANT_SUCCESS && q < perms; ++q) {
                const size_t cfg = (b << toggle_bits) + q;
                env.permutation = (uint32_t)q;
                for (row = 0; row < num_rows; ++row) {
                    float value;
                    env.row = row;
                    r = so_frame(&env, p.asts[a], NULL, 0, 0, &value);
                    if (r != SECANT_SUCCESS) break;
                    for (t = 0; t < num_targets; ++t) {
                        const float err = value - targets[t * targets_ld + row];
                        const float sq = err * err;
                        output[(a * num_targets + t) * output_ld + cfg] += sq;
                        if (output64) output64[(a * num_targets + t) * output_ld + cfg] += (double)sq;
                    }
                }
            }
        }
    }
    so_programs_close(&p);
    return r;
}

/* Per-row predictions of ONE configuration of every program, [ast][row].  The reference
 * has no such entry (its materialize shape takes no banks); this is so_frame applied
 * row by row and exists so tests can compare per-row values of bank/toggle programs. */
SO_EXPORT SecantResult so_toggle_materialize(const uint8_t* routine_blob, const uint64_t* routine_off, size_t num_routines,
                                             const uint8_t* ast_blob, const uint64_t* ast_off, size_t num_asts,
                                             size_t num_inputs, size_t num_constants, const float* input, size_t input_ld,
                                             const float* constants, size_t bank_stride, size_t program_bank_stride,
                                             uint32_t toggle_bits, size_t configuration, size_t num_rows, float* output,
                                             size_t output_ld) {
    SoPrograms p;
    SoEnv env;
    size_t a, row;
    SecantResult r = so_programs_open(&p, routine_blob, routine_off, num_routines, ast_blob, ast_off, num_asts);
    memset(&env, 0, sizeof(env));
    env.routines = p.routines; env.num_routines = num_routines; env.arity = p.arity;
    env.num_columns = num_inputs; env.num_constants = num_constants; env.input = input; env.input_ld = input_ld;
    env.toggle_bits = toggle_bits;
    env.permutation = (uint32_t)(configuration & (((uint64_t)1 << toggle_bits) - 1u));
    for (a = 0; r == SECANT_SUCCESS && a < num_asts; ++a) {
        env.constants = num_constants ? constants + a * program_bank_stride + (configuration >> toggle_bits) * bank_stride : NULL;
        for (row = 0; r == SECANT_SUCCESS && row < num_rows; ++row) {
            env.row = row;
            r = so_frame(&env, p.asts[a], NULL, 0, 0, output + a * output_ld + row);
        }
    }
    so_programs_close(&p);
    return r;
}

/* ---- best configuration per program (projects/secant-sr/toggle/src/cpu.c:45-67) ---
 * A score is valid when it is finite and >= 0.  The winner is the smallest valid score,
 * the lowest configuration index on ties.  No valid score: {+inf, UINT64_MAX, 0}. */
SO_EXPORT void so_best_config(const float* scores, size_t num_asts, size_t num_configs, size_t ld, float* best_score,
                              uint64_t* best_config, uint64_t* num_valid) {
    size_t a, c;
    for (a = 0; a < num_asts; ++a) {
        float best = INFINITY;
        uint64_t arg = UINT64_MAX, valid = 0;
        for (c = 0; c < num_configs; ++c) {
            const float s = scores[a * ld + c];
            if (!isfinite(s) || s < 0.0f) continue;
            ++valid;
            if (arg == UINT64_MAX || s < best) { best = s; arg = c; }
        }
        best_score[a] = best; best_config[a] = arg; num_valid[a] = valid;
    }
}

/* ---- global top-k (ordering rule of projects/odezza/core/o_score_reduce.cu:36-39) --
 * Order: valid before invalid, then score ascending, then index ascending.  Writes
 * min(k, count) indices.  O(count * k) selection, fine for test sizes. */
static int so_better(float sa, uint64_t ia, float sb, uint64_t ib) {
    const int va = isfinite(sa) && sa >= 0.0f, vb = isfinite(sb) && sb >= 0.0f;
    if (va != vb) return va;
    if (va && sa != sb) return sa < sb;
    return ia < ib;
}
SO_EXPORT size_t so_topk(const float* scores, size_t count, size_t k, uint64_t* indices_out) {
    size_t filled = 0, i, j;
    if (k > count) k = count;
    for (i = 0; i < count; ++i) {
        j = filled;
        if (filled == k) {
            if (!so_better(scores[i], i, scores[indices_out[k - 1]], indices_out[k - 1])) continue;
            j = k - 1;
        } else {
            ++filled;
        }
        while (j > 0 && so_better(scores[i], i, scores[indices_out[j - 1]], indices_out[j - 1])) {
            indices_out[j] = indices_out[j - 1];
            --j;
        }
        indices_out[j] = i;
    }
    return filled;
}

/* ---- fixed-step RK4 rollout scoring ------------------------------------------------
 * Restates the integration loop of the reference's generated scoring kernel
 * (projects/odezza/core/o_generate_scoring_cuda.c:494-588) for an S-state autonomous
 * system whose right-hand sides are Secant programs (state s is COLUMN s, the system's
 * coefficients are BANK_CONSTANT slots).  Data layout follows the reference kernel:
 *   reference[state * total_points + point], trajectories stored back to back, each with
 *   points_per_trajectory points; a trajectory starts from its first reference point;
 *   times[k] (k < points_per_trajectory) is shared by all trajectories.
 * Per observation interval: interval = times[k] - times[k-1]; h = interval / substeps;
 * per substep: base = stage = state, sum = 0; four stages with
 *     sum   = fmaf(w, rhs(stage), sum)       w = 1, 2, 2, 1
 *     stage = fmaf(h/2 (stages 0,1) or h (stage 2), rhs, base)
 *   then state = fmaf(h/6, sum, base).
 * After each interval every state must be finite and err = state - reference feeds
 * sq = fmaf(err, err, sq).  Score = sq / residual_count when everything stayed finite and
 * intervals are positive, else FLT_MAX (3.402823466e+38F), never NaN.
 * Residuals are accumulated trajectory by trajectory in one binary32 accumulator, like
 * the reference thread does; with ~2e5 residuals that sum alone is only good to ~1e-4
 * relative (small terms fall below the accumulator's ulp), so scores64 optionally returns the
 * same residuals accumulated in binary64.
 * Transcendental opcodes are evaluated with libm here; a device implementation that
 * wants bit-identical chaotic rollouts must restrict right-hand sides to exactly
 * rounded operations (add, sub, mul, div, fma, sqrt, rcp, neg, abs, min, max).
 * Parity: unpinned beyond the reference's closed-form value and invalid-data matrix in the
 * test-suite (the reference has no general fp32 host scorer to run). */
/* Checker-only switch.  The reference's one host-side rollout scorer takes every observation
 * interval to be the constant 0.05f (projects/odezza/research/ast_tools/o_ast_engine_benchmark.c:376)
 * instead of a difference of time stamps, and no float32 time axis has eight consecutive differences
 * that all equal 0.05f.  With a positive value set here the integrator below uses it as the interval
 * of every observation, which makes the two scorers comparable bit for bit; 0 restores the time axis. */
static float so_fixed_interval = 0.0f;
SO_EXPORT void so_rk4_set_fixed_interval(float value) { so_fixed_interval = value; }

/* General form.  offsets == NULL: every trajectory has points_per_trajectory points and
 * times[points_per_trajectory] is shared.  offsets != NULL: the reference engine's launch layout
 * (projects/odezza/core/odezza.h:275-289, checks and loop of
 * projects/odezza/core/o_generate_scoring_cuda.c:494-588): offsets[num_trajectories + 1]
 * partition total_points concatenated points, times is per point, and with allow_missing a NaN
 * reference value after a trajectory's first point is an unobserved value: it is skipped and the
 * mean divides by the residuals that were observed. */
static SecantResult so_rk4_general(const uint8_t* routine_blob, const uint64_t* routine_off, size_t num_routines,
                                   const uint8_t* rhs_blob, const uint64_t* rhs_off, size_t num_systems, size_t num_states,
                                   size_t num_constants, const float* constants, size_t system_constant_stride,
                                   const float* reference, size_t num_trajectories, size_t points_per_trajectory,
                                   const uint32_t* offsets, size_t total_points, int allow_missing, const float* times,
                                   size_t substeps, uint32_t toggle_bits, uint32_t permutation, float* scores, double* scores64) {
    SoPrograms p;
    SoEnv env;
    size_t sys, tr, point, sub, stage, s;
    float state[8], base[8], work[8], sum[8], rhs[8];
    SecantResult r;
    if (!num_states || num_states > 8 || !num_systems || !num_trajectories || (!offsets && points_per_trajectory < 2) || !substeps ||
        !reference || !times || !scores)
        return SECANT_ERROR_INVALID_VALUE;
    if (!offsets) total_points = num_trajectories * points_per_trajectory;
    {   /* the reference kernel stages every time and reference value first and gives up on all
         * scores when one of them is not finite (o_generate_scoring_cuda.c:457-477) */
        int invalid_data = 0;
        const size_t num_times = offsets ? total_points : points_per_trajectory;
        for (s = 0; s < num_states; ++s)
            for (point = 0; point < total_points; ++point) {
                const float v = reference[s * total_points + point];
                invalid_data |= !isfinite(v) && !(allow_missing && isnan(v));
            }
        for (point = 0; point < num_times; ++point) invalid_data |= !isfinite(times[point]);
        if (invalid_data) {
            for (sys = 0; sys < num_systems; ++sys) { scores[sys] = FLT_MAX; if (scores64) scores64[sys] = (double)FLT_MAX; }
            return SECANT_SUCCESS;
        }
    }
    r = so_programs_open(&p, routine_blob, routine_off, num_routines, rhs_blob, rhs_off, num_systems * num_states);
    memset(&env, 0, sizeof(env));
    env.routines = p.routines; env.num_routines = num_routines; env.arity = p.arity;
    env.num_columns = num_states; env.num_constants = num_constants; env.input_ld = 1; env.row = 0;
    env.toggle_bits = toggle_bits; env.permutation = permutation;
    for (sys = 0; r == SECANT_SUCCESS && sys < num_systems; ++sys) {
        float sq = 0.0f;
        double sq64 = 0.0; /* same residuals accumulated in binary64, free of summation-order error */
        size_t residuals = 0, scored_points = 0, expected = 0;
        int valid = 1;
        env.constants = num_constants ? constants + sys * system_constant_stride : NULL;
        for (tr = 0; r == SECANT_SUCCESS && tr < num_trajectories; ++tr) {
            const size_t begin = offsets ? offsets[tr] : tr * points_per_trajectory;
            const size_t end = offsets ? offsets[tr + 1] : begin + points_per_trajectory;
            if (offsets) {
                if (begin != expected || end <= begin || end > total_points) { valid = 0; break; }
                expected = end;
            }
            for (s = 0; s < num_states; ++s) {
                state[s] = reference[s * total_points + begin];
                valid = valid && isfinite(state[s]);
            }
            for (point = begin + 1; r == SECANT_SUCCESS && point < end; ++point) {
                const float stamped = offsets ? times[point] - times[point - 1] : times[point - begin] - times[point - begin - 1];
                const float interval = so_fixed_interval > 0.0f ? so_fixed_interval : stamped;
                const float h = interval / (float)substeps;
                const float half = 0.5f * h, sixth = h / 6.0f;
                valid = valid && isfinite(interval) && interval > 0.0f && h > 0.0f;
                for (sub = 0; r == SECANT_SUCCESS && sub < substeps; ++sub) {
                    for (s = 0; s < num_states; ++s) { base[s] = work[s] = state[s]; sum[s] = 0.0f; }
                    for (stage = 0; r == SECANT_SUCCESS && stage < 4; ++stage) {
                        const float weight = (stage == 0 || stage == 3) ? 1.0f : 2.0f;
                        env.input = work;
                        for (s = 0; r == SECANT_SUCCESS && s < num_states; ++s)
                            r = so_frame(&env, p.asts[sys * num_states + s], NULL, 0, 0, rhs + s);
                        for (s = 0; s < num_states; ++s) sum[s] = fmaf(weight, rhs[s], sum[s]);
                        if (stage != 3)
                            for (s = 0; s < num_states; ++s) work[s] = fmaf(stage == 2 ? h : half, rhs[s], base[s]);
                    }
                    for (s = 0; s < num_states; ++s) state[s] = fmaf(sixth, sum[s], base[s]);
                }
                for (s = 0; s < num_states; ++s) valid = valid && isfinite(state[s]);
                ++scored_points;
                for (s = 0; s < num_states; ++s) {
                    const float ref = reference[s * total_points + point];
                    if (allow_missing && isnan(ref)) continue;
                    {
                        const float err = state[s] - ref;
                        sq = fmaf(err, err, sq);
                        sq64 += (double)err * (double)err;
                        ++residuals;
                    }
                }
            }
        }
        if (r != SECANT_SUCCESS) break;
        valid = valid && (!offsets || expected == total_points) && scored_points && residuals;
        scores[sys] = (valid && isfinite(sq)) ? sq / (float)residuals : FLT_MAX;
        if (scores64) scores64[sys] = (valid && isfinite(sq)) ? sq64 / (double)residuals : (double)FLT_MAX;
    }
    so_programs_close(&p);
    return r;
}

SO_EXPORT SecantResult so_rk4_score(const uint8_t* routine_blob, const uint64_t* routine_off, size_t num_routines,
                                    const uint8_t* rhs_blob, const uint64_t* rhs_off, size_t num_systems,
                                    size_t num_states, size_t num_constants, const float* constants,
                                    size_t system_constant_stride, const float* reference, size_t num_trajectories,
                                    size_t points_per_trajectory, const float* times, size_t substeps, uint32_t toggle_bits,
                                    uint32_t permutation, float* scores, double* scores64) {
    return so_rk4_general(routine_blob, routine_off, num_routines, rhs_blob, rhs_off, num_systems, num_states, num_constants,
                          constants, system_constant_stride, reference, num_trajectories, points_per_trajectory, NULL, 0, 0,
                          times, substeps, toggle_bits, permutation, scores, scores64);
}

/* Ragged trajectories, per-point times, optional missing observations. */
SO_EXPORT SecantResult so_rk4_score_ragged(const uint8_t* routine_blob, const uint64_t* routine_off, size_t num_routines,
                                           const uint8_t* rhs_blob, const uint64_t* rhs_off, size_t num_systems,
                                           size_t num_states, size_t num_constants, const float* constants,
                                           size_t system_constant_stride, const float* reference, size_t num_trajectories,
                                           const uint32_t* offsets, size_t total_points, int allow_missing, const float* times,
                                           size_t substeps, uint32_t toggle_bits, uint32_t permutation, float* scores,
                                           double* scores64) {
    if (!offsets) return SECANT_ERROR_INVALID_VALUE;
    return so_rk4_general(routine_blob, routine_off, num_routines, rhs_blob, rhs_off, num_systems, num_states, num_constants,
                          constants, system_constant_stride, reference, num_trajectories, 0, offsets, total_points,
                          allow_missing, times, substeps, toggle_bits, permutation, scores, scores64);
}

/* Grouped top-k of a [system][configuration] score grid: rules of the reference engine's reducer
 * (projects/odezza/core/o_score_reduce.cu:36-62): valid when 0 <= score < FLT_MAX, -0 orders as
 * +0, winners by (score, flat index), unfilled ranks {FLT_MAX, UINT64_MAX}, counts of valid,
 * invalid and finite-negative scores.  grouping 0: per system, 1: per (system, permutation) over
 * banks, 2: global.  winners_mse / winners_index are [group][k], counts is [group][3]. */
SO_EXPORT SecantResult so_grouped_topk(const float* scores, size_t num_systems, size_t num_banks, uint32_t toggle_bits,
                                       uint32_t grouping, size_t k, float* winners_mse, uint64_t* winners_index, uint64_t* counts) {
    const uint64_t perms = (uint64_t)1 << toggle_bits, configs = (uint64_t)num_banks << toggle_bits;
    const uint64_t groups = grouping == 0 ? num_systems : grouping == 1 ? num_systems * perms : 1;
    const uint64_t elements = grouping == 0 ? configs : grouping == 1 ? num_banks : configs * num_systems;
    uint64_t g, e, r;
    if (!scores || !k || grouping > 2 || !winners_mse || !winners_index || !counts) return SECANT_ERROR_INVALID_VALUE;
    for (g = 0; g < groups; ++g) {
        uint64_t valid = 0, invalid = 0, negative = 0;
        for (r = 0; r < k; ++r) { winners_mse[g * k + r] = FLT_MAX; winners_index[g * k + r] = UINT64_MAX; }
        for (e = 0; e < elements; ++e) {
            const uint64_t index = grouping == 2 ? e : grouping == 0 ? g * configs + e : (g / perms) * configs + e * perms + g % perms;
            const float f = scores[index];
            uint64_t at;
            if (!(f >= 0 && f < FLT_MAX)) { ++invalid; negative += isfinite(f) && f < 0; continue; }
            ++valid;
            /* insertion into the sorted prefix; elements arrive in flat-index order, so a strict
             * comparison keeps the lower index first on ties */
            for (at = k; at > 0; --at) {
                const float w = winners_mse[g * k + at - 1];
                if (winners_index[g * k + at - 1] != UINT64_MAX && !((f == 0 ? 0.f : f) < (w == 0 ? 0.f : w))) break;
            }
            if (at == k) continue;
            for (r = k - 1; r > at; --r) { winners_mse[g * k + r] = winners_mse[g * k + r - 1]; winners_index[g * k + r] = winners_index[g * k + r - 1]; }
            winners_mse[g * k + at] = f;
            winners_index[g * k + at] = index;
        }
        counts[g * 3] = valid; counts[g * 3 + 1] = invalid; counts[g * 3 + 2] = negative;
    }
    return SECANT_SUCCESS;
}

/* Evaluate one program once; the smallest building block, used by unit tests. */
SO_EXPORT SecantResult so_eval(const uint8_t* routine_blob, const uint64_t* routine_off, size_t num_routines,
                               const uint8_t* program, size_t num_columns, size_t num_constants, const float* input,
                               size_t input_ld, const float* constants, uint32_t toggle_bits, uint32_t permutation,
                               size_t row, float* value_ret) {
    SoPrograms p;
    SoEnv env;
    const uint64_t zero = 0;
    SecantResult r = so_programs_open(&p, routine_blob, routine_off, num_routines, program, &zero, 1);
    memset(&env, 0, sizeof(env));
    env.routines = p.routines; env.num_routines = num_routines; env.arity = p.arity;
    env.num_columns = num_columns; env.num_constants = num_constants; env.input = input; env.input_ld = input_ld;
    env.constants = constants; env.toggle_bits = toggle_bits; env.permutation = permutation; env.row = row;
    if (r == SECANT_SUCCESS) r = so_frame(&env, program, NULL, 0, 0, value_ret);
    so_programs_close(&p);
    return r;
}
