/*
 * testhooks.cpp - host-only helpers for the CPU test-suite (built as a separate library,
 * never linked into libsecant_b200.so).
 *
 * sbt_encode() runs the production encoder on a set of programs; sbt_eval() executes one
 * encoded record with plain scalar C arithmetic, instruction by instruction, the way one
 * lane of the device evaluator does for one (row, bank).  Comparing that with the CPU
 * oracle checks the encoder (operand order, spill slots, toggle patches, affine entries)
 * on machines without a GPU.  This interpreter is test infrastructure, not a fallback.
 */
#include "encoder.h"

#include <cmath>
#include <cstring>
#include <new>
#include <vector>

using namespace sb;

struct SbtBatch {
    EncodedBatch enc;
    ProgramRules rules;
};

#define SBT_EXPORT extern "C" __attribute__((visibility("default")))

SBT_EXPORT int sbt_encode(const uint8_t* routine_blob, const uint64_t* routine_off, size_t num_routines,
                          const uint8_t* ast_blob, const uint64_t* ast_off, size_t num_asts, size_t num_columns,
                          size_t num_constants, int banks_allowed, unsigned toggle_bits, int run_preflight,
                          SbtBatch** out) {
    const bool hoist = (run_preflight & 2) != 0; /* bit 1 of the flag word asks for the prelude split */
    run_preflight &= 1;
    std::vector<const SecantAstInstruction*> routines(num_routines), asts(num_asts);
    for (size_t i = 0; i < num_routines; ++i) routines[i] = routine_blob + routine_off[i];
    for (size_t i = 0; i < num_asts; ++i) asts[i] = ast_blob + ast_off[i];
    SecantAstProgramList rl{routines.data(), num_routines};
    uint8_t arity[SECANT_AST_MAX_ROUTINES];
    *out = nullptr;
    SbtBatch* b = new (std::nothrow) SbtBatch();
    if (!b) return SECANT_ERROR_ALLOCATION_FAILED;
    b->rules.num_columns = num_columns;
    b->rules.num_constants = num_constants;
    b->rules.banks_allowed = banks_allowed != 0;
    b->rules.toggle_bits = toggle_bits;
    b->rules.hoist_invariants = hoist;
    SecantResult r = SECANT_SUCCESS;
    if (run_preflight) {
        for (size_t i = 0; i < num_routines && r == SECANT_SUCCESS; ++i) r = preflight(routines[i], b->rules);
        for (size_t i = 0; i < num_asts && r == SECANT_SUCCESS; ++i) r = preflight(asts[i], b->rules);
    }
    if (r == SECANT_SUCCESS) r = routine_arities(rl, arity);
    for (size_t i = 0; i < num_asts && r == SECANT_SUCCESS; ++i) r = encode_program(asts[i], rl, arity, b->rules, b->enc);
    if (r != SECANT_SUCCESS) { delete b; return r; }
    *out = b;
    return SECANT_SUCCESS;
}

SBT_EXPORT void sbt_free(SbtBatch* b) { delete b; }

SBT_EXPORT void sbt_info(const SbtBatch* b, size_t program, uint32_t* n_insn, uint32_t* n_slots, uint32_t* n_ops,
                         uint32_t* n_patch, uint32_t* n_affine, uint32_t* n_lits) {
    /* with the prelude split requested, n_patch / n_affine report main_off / n_hoisted instead */
    const SbProgram& p = b->enc.programs[program];
    *n_insn = p.n_insn; *n_slots = p.n_slots; *n_ops = p.n_ops; *n_lits = p.n_lits;
    *n_patch = b->rules.hoist_invariants ? p.main_off : p.n_patch;
    *n_affine = b->rules.hoist_invariants ? p.n_hoisted : p.n_affine;
}

/* Instruction counts by case id over all programs: prelude[SB_NUM_CASES] for the
 * bank-independent part, main[SB_NUM_CASES] for the part repeated per bank group. */
SBT_EXPORT unsigned sbt_case_histogram(const SbtBatch* b, uint64_t* prelude, uint64_t* main_part) {
    for (unsigned c = 0; c < SB_NUM_CASES; ++c) prelude[c] = main_part[c] = 0;
    for (const SbProgram& p : b->enc.programs)
        for (unsigned i = 0; i < p.n_insn; ++i) {
            const unsigned c = b->enc.insns[p.insn_off + i].w0 & 0xffu;
            if (c < SB_NUM_CASES) (i < p.main_off ? prelude : main_part)[c]++;
        }
    return SB_NUM_CASES;
}

static float apply_bin(unsigned op, float a, float x) {
    switch (op) {
    case SB_BIN_ADD: return a + x;
    case SB_BIN_SUB: return a - x;
    case SB_BIN_RSUB: return x - a;
    case SB_BIN_MUL: return a * x;
    case SB_BIN_DIV: return a / x;
    case SB_BIN_RDIV: return x / a;
    case SB_BIN_MIN: return fminf(a, x);
    default: return fmaxf(a, x);
    }
}
static float apply_un(unsigned op, float a) {
    switch (op) {
    case SB_UN_NEG: return -a;
    case SB_UN_SQRT: return sqrtf(a);
    case SB_UN_RCP: return 1.0f / a;
    case SB_UN_ABS: return fabsf(a);
    case SB_UN_SIN: return sinf(a);
    case SB_UN_COS: return cosf(a);
    case SB_UN_EX2: return exp2f(a);
    case SB_UN_LG2: return log2f(a);
    case SB_UN_RSQRT: return 1.0f / sqrtf(a);
    case SB_UN_TANH: return tanhf(a);
    case SB_UN_EXP: return expf(a);
    default: return logf(a);
    }
}

/* Value of program `program` on `row` for one bank vector and one permutation. */
SBT_EXPORT int sbt_eval(const SbtBatch* b, size_t program, const float* input, size_t input_ld, size_t row,
                        const float* bank, uint64_t permutation, float* value) {
    const EncodedBatch& e = b->enc;
    const SbProgram& p = e.programs[program];
    const size_t K = b->rules.num_constants;
    std::vector<SbInsn> code(e.insns.begin() + p.insn_off, e.insns.begin() + p.insn_off + p.n_insn);
    for (unsigned i = 0; i < p.n_patch; ++i) {
        const SbPatch& s = e.patches[p.patch_off + i];
        unsigned choice = (unsigned)(permutation >> s.bit0) & 1u;
        if (s.bit1 != 0xff) choice |= ((unsigned)(permutation >> s.bit1) & 1u) << 1;
        code[s.insn] = s.alt[choice];
    }
    std::vector<float> cst(K + p.n_affine + p.n_lits, 0.0f);
    for (size_t k = 0; k < K; ++k) cst[k] = bank ? bank[k] : 0.0f;
    for (unsigned j = 0; j < p.n_affine; ++j) {
        const SbAffine& a = e.affines[p.affine_off + j];
        volatile float scaled = bank[a.slot] * a.scale;
        cst[K + j] = scaled + a.offset;
    }
    for (unsigned j = 0; j < p.n_lits; ++j) cst[K + p.n_affine + j] = e.lits[p.lit_off + j];
    std::vector<float> slots(p.n_slots ? p.n_slots : 1, 0.0f);
    std::vector<float> hoisted(p.n_hoisted ? p.n_hoisted : 1, 0.0f);
    float acc = 0.0f;
    bool second_round = false;
    auto operand = [&](unsigned kind, unsigned index, uint32_t imm) -> float {
        switch (kind) {
        case SB_KIND_ROW: return (index & SB_ROW_HOISTED) ? hoisted[index & 0x7f] : input[(size_t)index * input_ld + row];
        case SB_KIND_CST: return cst[index];
        default: (void)imm; return slots[index];
        }
    };
    for (size_t pc = 0; pc < code.size(); ++pc) {
        const SbInsn ins = code[pc];
        const unsigned cs = ins.w0 & 0xffu, index = ins.w0 >> 16;
        if (cs == SB_CASE_END) {
            if (pc + 1 <= p.main_off) continue; /* end of the prelude: fall through into the main part */
            if (p.main_off && !second_round) {
                /* The device runs the main part once per bank group after ONE prelude: do it a
                 * second time with every spill slot poisoned, so a main part that relied on a
                 * slot written by the prelude or by its own previous run is caught. */
                second_round = true;
                for (auto& v : slots) v = std::nanf("");
                acc = std::nanf("");
                pc = (size_t)p.main_off - 1;
                continue;
            }
            *value = acc;
            return SECANT_SUCCESS;
        }
        if (cs >= SB_CASE_LOAD && cs < SB_CASE_LOAD + SB_NUM_KINDS) acc = operand(cs - SB_CASE_LOAD, index, ins.w1);
        else if (cs == SB_CASE_STORE) slots[index] = acc;
        else if (cs == SB_CASE_STOREH) hoisted[index] = acc;
        else if (cs >= SB_CASE_BIN && cs < SB_CASE_UN) {
            const unsigned rel = cs - SB_CASE_BIN;
            acc = apply_bin(rel / SB_NUM_KINDS, acc, operand(rel % SB_NUM_KINDS, index, ins.w1));
        } else if (cs >= SB_CASE_UN && cs < SB_CASE_FMA) acc = apply_un(cs - SB_CASE_UN, acc);
        else if (cs == SB_CASE_FMA) {
            const unsigned kinds = (ins.w0 >> 8) & 0x3fu;
            float v[3];
            for (int i = 0; i < 3; ++i) {
                const unsigned kind = (kinds >> (2 * i)) & 3u, idx = (ins.w1 >> (10 * i)) & 1023u;
                v[i] = kind == SB_FMA_ACC ? acc : operand(kind, idx, 0);
            }
            acc = fmaf(v[0], v[1], v[2]);
        } else return SECANT_ERROR_UNEXPECTED_INSTRUCTION;
    }
    return SECANT_ERROR_UNEXPECTED_INSTRUCTION;
}

/* Runs the request validation the runner performs before it clears or launches anything
 * (header, extents, overlap, program preflight) against a plan built from `recipe`. */
#include "internal.h"
SBT_EXPORT int sbt_validate_runs(const SecantCubinRecipeHeader* recipe, const SecantCubinRunHeader* const* headers,
                                 size_t count) {
    SecantResult r = recipe_validate(recipe);
    if (r != SECANT_SUCCESS) return r;
    SecantCubinPlan plan;
    plan_fill(&plan, recipe, 0);
    if (!headers || !count) return SECANT_ERROR_INVALID_VALUE;
    std::vector<UnpackedRun> runs(count);
    for (size_t i = 0; i < count; ++i) {
        r = run_unpack(plan, headers[i], &runs[i]);
        if (r != SECANT_SUCCESS) return r;
    }
    ProgramRules rules;
    return runs_validate(plan, runs.data(), count, &rules);
}
