/*
 * record.h - the compact program record shared by the host encoder and the device
 * evaluator.
 *
 * The reference turns every postfix program into machine code patched into a compiled
 * kernel template (projects/secant/s_cubin_specialize.c:1203-1368).  Here the same
 * traversal produces a short list of 8-byte instructions for an accumulator machine
 * that one warp interprets:
 *
 *   - every thread owns a register tile acc[rows][banks];
 *   - an instruction combines acc with ONE operand X (a per-row value, an entry of the
 *     per-warp constant area, or a spill slot),
 *     or applies a unary function to acc, or stores acc into a spill slot;
 *   - spill slots and the order of evaluation are fixed by the encoder, so the device
 *     never manipulates a stack.
 *
 * Instruction word 0:  bits 0..7 case id (SB_CASE_*), bits 8..15 aux, bits 16..31 operand index.
 * Instruction word 1:  packed FMA operand indices.  In records made for the rollout kernel a STORE
 *                      may carry SB_STORE_THEN_LOAD | kind << 16 | index there: "slot = acc, then
 *                      acc = X" (a parked value is nearly always followed by the load that starts
 *                      the next sub-expression; one dispatch instead of two).  Zero otherwise.
 */
#ifndef SECANT_B200_RECORD_H
#define SECANT_B200_RECORD_H

#include <stdint.h>

/* Operand kinds.  Few kinds means few interpreter cases, and the interpreter's hot code has to
 * stay small enough for the instruction caches:
 *   ROW   one float per row: a dataset column (index < SB_ROW_HOISTED) or a bank-independent
 *         value left by the program's row prelude (index = SB_ROW_HOISTED | n)
 *   CST   one float per bank: entry `index` of the program's constant table
 *   SLOT  one float per (row, bank): a spill slot
 * Inside the bank part of a program (see SbProgram) the same three codes address the scalar
 * machine that runs once per coefficient bank: ROW = an entry of the constant table written
 * earlier in the bank part, CST = a source constant (bank slot k for k < K, then the program's
 * affine entries, then its literals), SLOT = a scalar temporary. */
enum { SB_KIND_ROW = 0, SB_KIND_CST = 1, SB_KIND_SLOT = 2, SB_NUM_KINDS = 3 };
enum { SB_ROW_HOISTED = 0x8000 };
/* FMA operand descriptors: kind 3 means "the accumulator"; 10-bit indices, bit 9 = hoisted row value. */
enum { SB_FMA_ACC = 3, SB_FMA_ROW_HOISTED = 0x200 };
enum { SB_STORE_THEN_LOAD = 0x80000000u };

/* Binary operations; R* = operand on the left, accumulator on the right. */
enum { SB_BIN_ADD = 0, SB_BIN_SUB, SB_BIN_RSUB, SB_BIN_MUL, SB_BIN_DIV, SB_BIN_RDIV, SB_BIN_MIN, SB_BIN_MAX, SB_NUM_BIN };
/* Unary operations, in the order of the reference opcodes they implement. */
enum { SB_UN_NEG = 0, SB_UN_SQRT, SB_UN_RCP, SB_UN_ABS, SB_UN_SIN, SB_UN_COS, SB_UN_EX2, SB_UN_LG2, SB_UN_RSQRT,
       SB_UN_TANH, SB_UN_EXP, SB_UN_LOG, SB_NUM_UN };

enum {
    SB_CASE_END = 0,
    SB_CASE_LOAD = 1,                                  /* + kind           : acc = X            */
    SB_CASE_STORE = SB_CASE_LOAD + SB_NUM_KINDS,       /* slot[index] = acc                     */
    SB_CASE_STOREH = SB_CASE_STORE + 1,                /* row prelude: hoisted[index] = acc; bank part: table[index] = acc */
    SB_CASE_BIN = SB_CASE_STOREH + 1,                  /* + op * 3 + kind  : acc = acc (op) X   */
    SB_CASE_UN = SB_CASE_BIN + SB_NUM_BIN * SB_NUM_KINDS, /* + op          : acc = f(acc)       */
    SB_CASE_FMA = SB_CASE_UN + SB_NUM_UN,              /* acc = fma(A, B, C), generic operands  */
    SB_NUM_CASES
};

typedef struct SbInsn {
    uint32_t w0;
    uint32_t w1;
} SbInsn;

static inline uint32_t sb_w0(unsigned case_id, unsigned aux, unsigned index) {
    return (uint32_t)case_id | ((uint32_t)aux << 8) | ((uint32_t)index << 16);
}
/* FMA: aux = kindA | kindB << 2 | kindC << 4 ; w1 = idxA | idxB << 10 | idxC << 20. */

/* One toggle site: instruction `insn` is replaced by alt[choice] for every permutation,
 * choice = bit(bit0) + 2 * bit(bit1); bit1 == 0xff marks a two-way toggle. */
typedef struct SbPatch {
    uint16_t insn;
    uint8_t bit0;
    uint8_t bit1;
    uint32_t pad;
    SbInsn alt[4];
} SbPatch;

/* A derived source constant: bank[slot] * scale + offset, both operations rounded. */
typedef struct SbAffine {
    uint32_t slot;
    float scale;
    float offset;
} SbAffine;

enum {
    SB_PROG_BANK_INDEPENDENT = 1, /* the value does not depend on the coefficient bank: every bank scores alike */
    SB_PROG_USES_SCRATCH = 2      /* an FMA runs over the scratch spill slot */
};

/* Per-program header; offsets index the pools of the batch the program belongs to.
 *
 * A program is up to four instruction runs, each closed by END:
 *   [0, pre_off)         bank part: everything that depends on the coefficient bank but not on
 *                        the row (and every constant the other parts read) is computed once per
 *                        bank by a scalar machine and left in the program's constant table of
 *                        n_cst entries per bank (STOREH);
 *   [pre_off, mid_off)   shared row prelude: sub-expressions that depend on the row but neither on
 *                        the bank nor on any toggle, evaluated once per row for all permutations
 *                        an item covers and kept as per-row values (STOREH), which later runs read
 *                        as ROW operands with SB_ROW_HOISTED set;
 *   [mid_off, main_off)  row prelude: the same for row-only sub-expressions a toggle reaches,
 *                        evaluated once per (row, permutation);
 *   [main_off, n_insn)   main part, run once per (row tile, permutation, bank group).
 * Values and rounding are those of the plain postfix evaluation: the same operations run on the
 * same operands, only less often.  Records made for the rollout kernel have a main part only
 * (pre_off = main_off = 0) and address source constants directly. */
typedef struct SbProgram {
    uint32_t insn_off;
    uint32_t patch_off;
    uint32_t affine_off;
    uint32_t lit_off;
    uint16_t n_insn; /* all parts, including their END instructions */
    uint16_t n_patch;
    uint16_t n_affine;
    uint16_t n_lits;
    uint16_t n_slots;
    uint16_t n_ops; /* arithmetic nodes after routine inlining, for work accounting */
    uint16_t pre_off;
    uint16_t main_off;
    uint16_t n_hoisted; /* per-row values the prelude leaves */
    uint16_t n_cst;     /* constant-table entries per bank */
    uint16_t n_btmp;    /* scalar temporaries of the bank part */
    uint16_t flags;     /* SB_PROG_* */
    uint32_t index;     /* position of the program in the run (output row, bank table) */
    uint32_t cost;      /* scheduling weight: bits 0..15 main part per bank group, bits 16..31 row prelude */
    uint16_t mid_off;
    uint16_t reserved;
} SbProgram;

#endif
