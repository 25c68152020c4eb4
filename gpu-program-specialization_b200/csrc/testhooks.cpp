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

#include <algorithm>
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
                          size_t num_constants, int banks_allowed, unsigned toggle_bits, int flags,
                          SbtBatch** out) {
    /* flags: bit 0 run the preflight scan first; bit 1 hoist bank-only and row-only sub-expressions; bit 3 only
     * row-only sub-expressions that no toggle reaches;
     * bit 2 one-part records with direct constant addressing (the rollout kernel's form);
     * bit 4 the rollout kernel's split form: columns are the first spill slots (four vectors of them are
     * reserved for the integrator), bank-only sub-expressions move to the bank part, nothing else is hoisted;
     * bits 8..15 cap on hoisted row values (0 = default) */
    const bool run_preflight = (flags & 1) != 0, hoist = (flags & 2) != 0, flat = (flags & 4) != 0;
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
    b->rules.split_parts = !flat;
    b->rules.hoist_bank = hoist && !flat;
    b->rules.hoist_row = hoist && !flat;
    b->rules.hoist_toggled = !(flags & 8u);
    if (flags & 16u) {
        b->rules.columns_are_slots = true;
        b->rules.reserved_slots = (unsigned)(4 * num_columns);
        b->rules.split_parts = true;
        b->rules.hoist_bank = true;
        b->rules.hoist_row = false;
        b->rules.fuse_store_load = true;
    }
    if ((flags >> 8) & 0xff) b->rules.max_hoisted = (unsigned)((flags >> 8) & 0xff);
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

/* info[0..9] = n_insn, n_slots, n_ops, n_patch, n_affine, n_lits, pre_off, main_off, n_hoisted, n_cst;
 * info[10] = n_btmp, info[11] = flags, info[12] = mid_off */
SBT_EXPORT void sbt_info(const SbtBatch* b, size_t program, uint32_t* info) {
    const SbProgram& p = b->enc.programs[program];
    const uint32_t v[13] = {p.n_insn, p.n_slots, p.n_ops, p.n_patch, p.n_affine, p.n_lits,
                            p.pre_off, p.main_off, p.n_hoisted, p.n_cst, p.n_btmp, p.flags, p.mid_off};
    for (int i = 0; i < 13; ++i) info[i] = v[i];
}

/* Instruction counts by case id over all programs, per part:
 * hist[0][..] bank part, hist[1][..] row prelude, hist[2][..] main part. */
SBT_EXPORT unsigned sbt_case_histogram(const SbtBatch* b, uint64_t* hist) {
    for (unsigned c = 0; c < 3 * SB_NUM_CASES; ++c) hist[c] = 0;
    for (const SbProgram& p : b->enc.programs)
        for (unsigned i = 0; i < p.n_insn; ++i) {
            const unsigned c = b->enc.insns[p.insn_off + i].w0 & 0xffu;
            const unsigned part = i < p.pre_off ? 0u : i < p.main_off ? 1u : 2u;
            if (c < SB_NUM_CASES) hist[part * SB_NUM_CASES + c]++;
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

/* Value of program `program` on `row` for one bank vector and one permutation: the bank part
 * once (filling the constant table), the two row preludes once, then the main part twice with every
 * spill slot poisoned in between, as the device runs the main part once per bank group after
 * one prelude: a main part that relied on a slot written by the prelude or by its own previous
 * run is caught. */
SBT_EXPORT int sbt_eval(const SbtBatch* b, size_t program, const float* input, size_t input_ld, size_t row,
                        const float* bank, uint64_t permutation, float* value) {
    const EncodedBatch& e = b->enc;
    const SbProgram& p = e.programs[program];
    const size_t K = b->rules.num_constants;
    std::vector<SbInsn> code(e.insns.begin() + p.insn_off, e.insns.begin() + p.insn_off + p.n_insn);
    auto patch_for = [&](uint64_t perm) -> bool {
        for (unsigned i = 0; i < p.n_patch; ++i) {
            const SbPatch& s = e.patches[p.patch_off + i];
            unsigned choice = (unsigned)(perm >> s.bit0) & 1u;
            if (s.bit1 != 0xff) choice |= ((unsigned)(perm >> s.bit1) & 1u) << 1;
            if (s.insn >= code.size()) return false;
            code[s.insn] = s.alt[choice];
        }
        return true;
    };
    std::vector<float> source(K + p.n_affine + p.n_lits, 0.0f);
    for (size_t k = 0; k < K; ++k) source[k] = bank ? bank[k] : 0.0f;
    for (unsigned j = 0; j < p.n_affine; ++j) {
        const SbAffine& a = e.affines[p.affine_off + j];
        volatile float scaled = bank[a.slot] * a.scale;
        source[K + j] = scaled + a.offset;
    }
    for (unsigned j = 0; j < p.n_lits; ++j) source[K + p.n_affine + j] = e.lits[p.lit_off + j];
    const bool split = b->rules.split_parts;
    std::vector<float> table(p.n_cst ? p.n_cst : 1, std::nanf(""));
    std::vector<float> slots(std::max<unsigned>(1, std::max(p.n_slots, p.n_btmp)), std::nanf(""));
    std::vector<float> hoisted(p.n_hoisted ? p.n_hoisted : 1, std::nanf(""));
    float acc = std::nanf("");
    uint64_t bank_permutation = permutation; /* the permutation the bank part's lanes select by */
    int part = 0; /* 0 bank, 1 prelude, 2 main */
    bool failed = false;
    auto operand = [&](unsigned kind, unsigned index, bool fma) -> float {
        const unsigned hflag = fma ? (unsigned)SB_FMA_ROW_HOISTED : (unsigned)SB_ROW_HOISTED;
        switch (kind) {
        case SB_KIND_ROW:
            if (part == 0) { if (index >= table.size()) { failed = true; return 0; } return table[index]; }
            if (index & hflag) { const unsigned h = index & (hflag - 1); if (h >= hoisted.size()) { failed = true; return 0; } return hoisted[h]; }
            return input[(size_t)index * input_ld + row];
        case SB_KIND_CST:
            if (!split || part == 0) { if (index >= source.size()) { failed = true; return 0; } return source[index]; }
            if (index >= p.n_cst) { failed = true; return 0; }
            return table[index];
        default:
            if (index >= slots.size()) { failed = true; return 0; }
            return slots[index];
        }
    };
    auto run_part = [&](size_t begin, int which) -> bool {
        part = which;
        for (size_t pc = begin; pc < code.size(); ++pc) {
            SbInsn ins = code[pc];
            if (which == 0 && ins.w1 && (ins.w0 & 0xffu) != SB_CASE_FMA) { /* a toggle site of the bank part picks its own alternative */
                if (ins.w1 > p.n_patch) return false;
                const SbPatch& site = e.patches[p.patch_off + ins.w1 - 1];
                unsigned choice = (unsigned)(bank_permutation >> site.bit0) & 1u;
                if (site.bit1 != 0xff) choice |= ((unsigned)(bank_permutation >> site.bit1) & 1u) << 1;
                if (site.insn != pc || (site.alt[choice].w0 & 0xffu) == SB_CASE_END) return false;
                ins.w0 = site.alt[choice].w0;
            }
            const unsigned cs = ins.w0 & 0xffu, index = ins.w0 >> 16;
            if (cs == SB_CASE_END) return !failed;
            if (cs >= SB_CASE_LOAD && cs < SB_CASE_LOAD + SB_NUM_KINDS) acc = operand(cs - SB_CASE_LOAD, index, false);
            else if (cs == SB_CASE_STORE) {
                if (index >= slots.size()) return false;
                slots[index] = acc;
                if (ins.w1 & SB_STORE_THEN_LOAD) { /* the rollout records' fused form: then acc = X */
                    if (which == 0) return false;
                    acc = operand((ins.w1 >> 16) & 3u, ins.w1 & 0xffffu, false);
                }
            }
            else if (cs == SB_CASE_STOREH) {
                std::vector<float>& dst = which == 0 ? table : hoisted;
                if (which == 2 || index >= dst.size()) return false;
                dst[index] = acc;
            } else if (cs >= SB_CASE_BIN && cs < SB_CASE_UN) {
                const unsigned rel = cs - SB_CASE_BIN;
                acc = apply_bin(rel / SB_NUM_KINDS, acc, operand(rel % SB_NUM_KINDS, index, false));
            } else if (cs >= SB_CASE_UN && cs < SB_CASE_FMA) acc = apply_un(cs - SB_CASE_UN, acc);
            else if (cs == SB_CASE_FMA) {
                const unsigned kinds = (ins.w0 >> 8) & 0x3fu;
                float v[3];
                for (int i = 0; i < 3; ++i) {
                    const unsigned kind = (kinds >> (2 * i)) & 3u, idx = (ins.w1 >> (10 * i)) & 1023u;
                    v[i] = kind == SB_FMA_ACC ? acc : operand(kind, idx, true);
                }
                acc = fmaf(v[0], v[1], v[2]);
            } else return false;
        }
        return false;
    };
    /* the shared prelude runs once for all permutations of an item, with the program patched for
     * whichever of them came last and the table of the item's first one: here under the
     * complementary permutation, which differs in every toggle */
    if (p.mid_off > p.pre_off) {
        if (!patch_for(~permutation)) return SECANT_ERROR_UNEXPECTED_INSTRUCTION;
        bank_permutation = ~permutation;
        if (p.pre_off && !run_part(0, 0)) return SECANT_ERROR_UNEXPECTED_INSTRUCTION;
        for (auto& v : slots) v = std::nanf("");
        if (!run_part(p.pre_off, 1)) return SECANT_ERROR_UNEXPECTED_INSTRUCTION;
        for (auto& v : table) v = std::nanf("");
    }
    /* the bank part selects by itself: run it on a copy patched for yet another permutation */
    if (!patch_for(permutation ^ 0x5555555555555555ull)) return SECANT_ERROR_UNEXPECTED_INSTRUCTION;
    bank_permutation = permutation;
    if (p.pre_off && !run_part(0, 0)) return SECANT_ERROR_UNEXPECTED_INSTRUCTION;
    if (!patch_for(permutation)) return SECANT_ERROR_UNEXPECTED_INSTRUCTION;
    if (p.main_off > p.mid_off) {
        for (auto& v : slots) v = std::nanf("");
        if (!run_part(p.mid_off, 1)) return SECANT_ERROR_UNEXPECTED_INSTRUCTION;
    }
    for (int round = 0; round < 2; ++round) {
        for (auto& v : slots) v = std::nanf("");
        if (b->rules.columns_are_slots) /* the integrator keeps state i in slot i */
            for (size_t c = 0; c < b->rules.num_columns && c < slots.size(); ++c) slots[c] = input[c * input_ld + row];
        acc = std::nanf("");
        if (!run_part(p.main_off, 2)) return SECANT_ERROR_UNEXPECTED_INSTRUCTION;
    }
    *value = acc;
    return SECANT_SUCCESS;
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

/* Launch geometry the runner would pick for a batch with the given maxima (planner.cpp), so its
 * bounds can be checked without a device.  Returns 1 when a plan exists, 0 when the batch does not
 * fit shared memory, -1 when a count does not fit the kernel's 32-bit indices.
 * out[0..13] = variant, warps, tile_rows, tile_buffers, num_groups, groups_per_item, row_splits,
 * rows_per_split, smem_bytes, partial_elements, grid_x, warp_bytes, items per CTA and tile, perms_per_item. */
#include "evaluator.cuh"
SBT_EXPORT int sbt_plan(uint32_t num_programs, uint32_t max_insn, uint32_t max_slots, uint32_t max_hoisted, uint32_t max_cst,
                        uint32_t max_btmp, int mode, uint32_t num_inputs, uint32_t num_targets, uint32_t num_banks,
                        uint32_t toggle_bits, uint64_t rows, int sm_count, uint64_t smem_limit, uint64_t scratch_floats, uint64_t* out) {
    DeviceBatch db;
    std::memset(&db, 0, sizeof(db));
    db.num_programs = num_programs; db.max_insn = max_insn; db.max_slots = max_slots; db.max_hoisted = max_hoisted;
    db.max_cst = max_cst; db.max_btmp = max_btmp;
    EvalProblem p;
    std::memset(&p, 0, sizeof(p));
    p.mode = mode; p.num_inputs = num_inputs; p.num_targets = num_targets; p.num_banks = num_banks; p.toggle_bits = toggle_bits;
    p.num_rows = rows;
    const LaunchPlan plan = plan_launch(db, p, sm_count, smem_limit, scratch_floats);
    if (!plan.ok) return plan.overflow ? -1 : 0;
    const Geom g = make_geom(db, p, plan);
    const uint64_t rc = (uint64_t)kVariantBanks[plan.variant];
    const uint64_t bank_groups = mode == EVAL_MATERIALIZE ? 1 : (num_banks + rc - 1) / rc;
    const uint64_t items_per_program = mode == EVAL_MATERIALIZE ? 1 : ((bank_groups / plan.groups_per_item) << toggle_bits) / plan.perms_per_item;
    const uint64_t per_cta = (num_programs + plan.num_groups - 1) / plan.num_groups;
    const uint64_t v[14] = {(uint64_t)plan.variant, plan.warps, plan.tile_rows, plan.tile_buffers, plan.num_groups, plan.groups_per_item,
                            plan.row_splits, plan.rows_per_split, plan.smem_bytes, plan.partial_elements, plan.grid_x, g.warp_bytes,
                            per_cta * items_per_program, plan.perms_per_item};
    for (int i = 0; i < 14; ++i) out[i] = v[i];
    return 1;
}

/* Copies the instruction words of one record (w0, w1 pairs); returns the instruction count. */
SBT_EXPORT size_t sbt_instructions(const SbtBatch* b, size_t program, uint32_t* words, size_t capacity_insns) {
    const SbProgram& p = b->enc.programs[program];
    for (size_t i = 0; i < p.n_insn && i < capacity_insns; ++i) {
        words[2 * i] = b->enc.insns[p.insn_off + i].w0;
        words[2 * i + 1] = b->enc.insns[p.insn_off + i].w1;
    }
    return p.n_insn;
}
