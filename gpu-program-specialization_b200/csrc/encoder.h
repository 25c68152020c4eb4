/*
 * encoder.h - host-side program encoder: postfix bytecode -> accumulator-machine records.
 *
 * Plays the role of the reference specializer (projects/secant/s_cubin_specialize.c):
 * same linear traversal with routine inlining and the same structural error codes, but
 * the output is a compact record per program (record.h) instead of machine code.
 */
#ifndef SECANT_B200_ENCODER_H
#define SECANT_B200_ENCODER_H

#include "../../include/secant_b200.h"
#include "record.h"

#include <cstddef>
#include <vector>

namespace sb {

constexpr unsigned kMaxSlots = 48;       /* spill slots one program may need */
constexpr unsigned kRoutineDepth = 8;    /* nested routine frames, as in the reference */

struct ProgramRules {
    size_t num_columns = 0;     /* COLUMN indices must be below this */
    size_t num_constants = 0;   /* BANK / AFFINE_BANK slots must be below this */
    bool banks_allowed = false; /* only the toggle shape has banks and toggles */
    unsigned toggle_bits = 0;   /* toggle bit indices must be below this */
    /* Rollout scoring: COLUMN i is not a dataset column but state i of the trajectory being
     * integrated, which the kernel keeps in spill slot i; the first `reserved_slots` slots
     * belong to the integrator and program temporaries start after them. */
    bool columns_are_slots = false;
    unsigned reserved_slots = 0;
    /* main part: "STORE slot; LOAD x" becomes one instruction (record.h, SB_STORE_THEN_LOAD); only the
     * rollout kernel understands it */
    bool fuse_store_load = false;
    /* Records for the population evaluator are split into a bank part, a row prelude and a main
     * part (record.h, SbProgram) and address constants through a per-program table the bank part
     * fills.  Without split_parts (the rollout kernel) a record is one main part that addresses
     * source constants directly. */
    bool split_parts = false;
    /* hoist_bank: sub-expressions that depend on the coefficient bank only (or on nothing) are
     * computed in the bank part, once per bank.  hoist_row: sub-expressions that depend on the row
     * only are computed in the row prelude, once per row; at most max_hoisted values are kept, the
     * costliest first.  Values and rounding are unchanged: the same operations run on the same
     * operands, only less often. */
    bool hoist_bank = false;
    bool hoist_row = false;
    /* hoist_toggled: row-only sub-expressions that a toggle reaches get a prelude value as well (one
     * per permutation: worth it when a permutation is evaluated for several bank groups); without
     * it only what no toggle reaches is hoisted, which an item shares among its permutations. */
    bool hoist_toggled = true;
    unsigned max_hoisted = 4;
};

/* Encoded records of a contiguous group of programs, ready to upload as five arrays. */
struct EncodedBatch {
    std::vector<SbProgram> programs;
    std::vector<SbInsn> insns;
    std::vector<SbPatch> patches;
    std::vector<SbAffine> affines;
    std::vector<float> lits;
    unsigned max_insn = 1;      /* largest n_insn */
    unsigned max_extra = 0;     /* largest n_affine + n_lits */
    unsigned max_slots = 0;     /* largest n_slots */
    unsigned max_patch = 0;
    unsigned max_hoisted = 0;   /* largest n_hoisted */
    unsigned max_cst = 0;       /* largest n_cst */
    unsigned max_btmp = 0;      /* largest n_btmp */
    bool uses_scratch = false;  /* some program runs an FMA over the scratch slot */
    void clear();
};

/* Leaf-range / opcode scan of one program without inlining; mirrors the runner preflight
 * (projects/secant/s_cubin_runner.c:138-181).  Runs before any output is cleared. */
SecantResult preflight(const SecantAstInstruction* program, const ProgramRules& rules);

/* Number of ROUTINE_ARG slots each routine uses (projects/secant/s_cpu.c:129-191). */
SecantResult routine_arities(const SecantAstProgramList& routines, uint8_t* arity /* [255] */);

/* Appends the record of one program to `out`.  On error `out` may hold a partial record. */
SecantResult encode_program(const SecantAstInstruction* program, const SecantAstProgramList& routines,
                            const uint8_t* routine_arity, const ProgramRules& rules, EncodedBatch& out);

}  // namespace sb

#endif
