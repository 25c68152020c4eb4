/*
 * encoder.cpp - postfix bytecode -> accumulator-machine record.
 *
 * Stage 1 (parse) walks the byte stream with the per-token checks of the reference evaluator
 * and specializer (projects/secant/s_cpu.c:193-414, s_cubin_specialize.c:1203-1368), in their
 * order, expanding routine calls in place with their arguments bound once.  It builds an
 * expression DAG (a routine argument used several times becomes a shared node).
 * Stage 2 (classify) labels every node by what its value depends on: nothing (literals), the
 * coefficient bank, the row, or both.
 * Stage 3 (emit) linearises the DAG for a machine with one accumulator: a binary node whose
 * other operand is a leaf costs one instruction, a node with two computed operands spills the
 * first through a slot.  The deeper operand is evaluated first (Sethi-Ullman order), which only
 * changes the order pure sub-expressions are computed in, never how values are rounded or
 * associated.  For the population evaluator the instructions go to up to four runs (record.h):
 * bank-only sub-expressions to the bank part, row-only ones to the shared row prelude (no toggle
 * reaches them) or the row prelude, the rest to the main part.
 */
#include "encoder.h"

#include <algorithm>
#include <cmath>
#include <cstring>

namespace sb {

void EncodedBatch::clear() {
    programs.clear(); insns.clear(); patches.clear(); affines.clear(); lits.clear();
    max_insn = 1; max_extra = 0; max_slots = 0; max_patch = 0; max_hoisted = 0; max_cst = 0; max_btmp = 0;
    uses_scratch = false;
}

namespace {

/* ---- tokens ---------------------------------------------------------------------------- */

enum TokenKind : uint8_t { TK_COLUMN, TK_BANK, TK_AFFINE, TK_LITERAL, TK_TOGGLE, TK_ARG, TK_CALL, TK_RETURN, TK_OPERATION };

struct Token {
    TokenKind kind;
    uint8_t ways;   /* toggles: 2 or 4 */
    uint8_t arity;  /* operations */
    uint8_t node;   /* operations: 1 unary, 2 binary, 3 fma */
    uint8_t op;     /* SB_UN_* or SB_BIN_* */
    size_t width;
};

/* operations by opcode: {opcode, arity, SB_* code} */
struct OperationRow { uint8_t opcode, arity, code; };
const OperationRow kOperations[] = {
    {SECANT_AST_INSTRUCTION_TYPE_ADD_F32, 2, SB_BIN_ADD},   {SECANT_AST_INSTRUCTION_TYPE_SUB_F32, 2, SB_BIN_SUB},
    {SECANT_AST_INSTRUCTION_TYPE_MUL_F32, 2, SB_BIN_MUL},   {SECANT_AST_INSTRUCTION_TYPE_DIV_F32, 2, SB_BIN_DIV},
    {SECANT_AST_INSTRUCTION_TYPE_MIN_F32, 2, SB_BIN_MIN},   {SECANT_AST_INSTRUCTION_TYPE_MAX_F32, 2, SB_BIN_MAX},
    {SECANT_AST_INSTRUCTION_TYPE_FMA_F32, 3, 0},
    {SECANT_AST_INSTRUCTION_TYPE_NEG_F32, 1, SB_UN_NEG},    {SECANT_AST_INSTRUCTION_TYPE_SQRT_F32, 1, SB_UN_SQRT},
    {SECANT_AST_INSTRUCTION_TYPE_RCP_F32, 1, SB_UN_RCP},    {SECANT_AST_INSTRUCTION_TYPE_ABS_F32, 1, SB_UN_ABS},
    {SECANT_AST_INSTRUCTION_TYPE_SIN_F32, 1, SB_UN_SIN},    {SECANT_AST_INSTRUCTION_TYPE_COS_F32, 1, SB_UN_COS},
    {SECANT_AST_INSTRUCTION_TYPE_EX2_F32, 1, SB_UN_EX2},    {SECANT_AST_INSTRUCTION_TYPE_LG2_F32, 1, SB_UN_LG2},
    {SECANT_AST_INSTRUCTION_TYPE_RSQRT_F32, 1, SB_UN_RSQRT}, {SECANT_AST_INSTRUCTION_TYPE_TANH_F32, 1, SB_UN_TANH},
    {SECANT_AST_INSTRUCTION_TYPE_EXP_F32, 1, SB_UN_EXP},    {SECANT_AST_INSTRUCTION_TYPE_LOG_F32, 1, SB_UN_LOG},
};

/* The float32 opcodes the evaluators accept (projects/secant/s_ast_internal.h:103-117). */
bool evaluable_opcode(unsigned op) {
    switch (op) {
    case SECANT_AST_INSTRUCTION_TYPE_AFFINE_BANK_F32: case SECANT_AST_INSTRUCTION_TYPE_COLUMN_F32:
    case SECANT_AST_INSTRUCTION_TYPE_BANK_CONSTANT_F32: case SECANT_AST_INSTRUCTION_TYPE_TOGGLE2_F32:
    case SECANT_AST_INSTRUCTION_TYPE_TOGGLE4_F32: case SECANT_AST_INSTRUCTION_TYPE_EXP_F32:
    case SECANT_AST_INSTRUCTION_TYPE_LOG_F32:
        return true;
    default:
        return op >= SECANT_AST_INSTRUCTION_TYPE_CONSTANT_BITS_F32 && op <= SECANT_AST_INSTRUCTION_TYPE_TANH_F32;
    }
}

/* Decodes one token and applies every check that needs no evaluation state: byte width, opcode
 * class, leaf index ranges, toggle bit ranges, finite affine payloads.  Both the runner's
 * preflight (projects/secant/s_cubin_runner.c:138-181) and the parser below start from it, so
 * the two cannot disagree on what a well-formed token is. */
SecantResult read_token(const SecantAstInstruction* ins, const ProgramRules& rules, Token* t) {
    const unsigned op = ins[0];
    t->width = secant_ast_instruction_size_get(ins);
    t->ways = t->arity = t->node = t->op = 0;
    if (!t->width) return SECANT_ERROR_BAD_PROGRAM;
    if (!evaluable_opcode(op)) return SECANT_ERROR_UNSUPPORTED_OP;
    switch (op) {
    case SECANT_AST_INSTRUCTION_TYPE_COLUMN_F32:
        t->kind = TK_COLUMN;
        return ins[1] < rules.num_columns ? SECANT_SUCCESS : SECANT_ERROR_BAD_PROGRAM;
    case SECANT_AST_INSTRUCTION_TYPE_BANK_CONSTANT_F32:
        t->kind = TK_BANK;
        return rules.banks_allowed && ins[1] < rules.num_constants ? SECANT_SUCCESS : SECANT_ERROR_BAD_PROGRAM;
    case SECANT_AST_INSTRUCTION_TYPE_AFFINE_BANK_F32:
        t->kind = TK_AFFINE;
        if (!rules.banks_allowed || ins[1] >= rules.num_constants) return SECANT_ERROR_BAD_PROGRAM;
        return std::isfinite(secant_ast_affine_bank_scale_get(ins)) && std::isfinite(secant_ast_affine_bank_offset_get(ins))
                   ? SECANT_SUCCESS : SECANT_ERROR_BAD_PROGRAM;
    case SECANT_AST_INSTRUCTION_TYPE_CONSTANT_BITS_F32:
        t->kind = TK_LITERAL;
        return SECANT_SUCCESS;
    case SECANT_AST_INSTRUCTION_TYPE_TOGGLE2_F32:
    case SECANT_AST_INSTRUCTION_TYPE_TOGGLE4_F32:
        t->kind = TK_TOGGLE;
        t->ways = op == SECANT_AST_INSTRUCTION_TYPE_TOGGLE2_F32 ? 2 : 4;
        if (!rules.banks_allowed || ins[1] >= rules.toggle_bits) return SECANT_ERROR_BAD_PROGRAM;
        if (t->ways == 4 && (ins[2] >= rules.toggle_bits || ins[2] == ins[1])) return SECANT_ERROR_BAD_PROGRAM;
        return SECANT_SUCCESS;
    case SECANT_AST_INSTRUCTION_TYPE_ROUTINE_ARG_F32: t->kind = TK_ARG; return SECANT_SUCCESS;
    case SECANT_AST_INSTRUCTION_TYPE_ROUTINE_F32: t->kind = TK_CALL; return SECANT_SUCCESS;
    case SECANT_AST_INSTRUCTION_TYPE_RETURN_F32: t->kind = TK_RETURN; return SECANT_SUCCESS;
    default: break;
    }
    t->kind = TK_OPERATION;
    for (const OperationRow& row : kOperations)
        if (row.opcode == op) {
            t->arity = row.arity;
            t->node = row.arity;
            t->op = row.code;
            return SECANT_SUCCESS;
        }
    return SECANT_SUCCESS; /* NONE: decodable, rejected when evaluated (arity 0) */
}

bool direct_leaf(TokenKind k) { return k == TK_COLUMN || k == TK_BANK || k == TK_AFFINE || k == TK_LITERAL; }

/* ---- expression DAG -------------------------------------------------------------------- */

enum NodeType : uint8_t { N_COL, N_BANK, N_AFFINE, N_LIT, N_TOGGLE, N_UN, N_BIN, N_FMA };
/* What a value depends on.  Joining two classes: a literal adopts the other class, bank and row
 * together make a mixed value. */
enum ValueClass : int8_t { VC_UNKNOWN = -1, VC_LITERAL = 0, VC_BANK = 1, VC_ROW = 2, VC_MIXED = 3 };

ValueClass join(ValueClass a, ValueClass b) {
    if (a == b || b == VC_LITERAL) return a;
    if (a == VC_LITERAL) return b;
    return VC_MIXED;
}

struct Node {
    NodeType type;
    uint8_t op = 0;       /* SB_UN_* for N_UN, SB_BIN_{ADD,SUB,MUL,DIV,MIN,MAX} for N_BIN */
    uint8_t ways = 0;     /* toggle: 2 or 4 */
    uint8_t bit0 = 0, bit1 = 0xff;
    int32_t child[4] = {-1, -1, -1, -1};
    uint32_t index = 0;   /* column / bank slot / affine entry */
    uint32_t bits = 0;    /* literal */
    int32_t uses = 0;     /* parents inside the run being emitted */
    int32_t pending = 0;  /* uses not yet emitted */
    int32_t slot = -1;    /* spill slot holding the value, once computed */
    int32_t su = 0;       /* slots needed to compute the node into the accumulator */
    ValueClass cls = VC_UNKNOWN;
    int32_t hoisted = -1; /* per-row value the prelude left */
    int32_t entry = -1;   /* constant-table entry the bank part left */
    int32_t weight = 0;   /* rough instruction cost of the sub-expression */
};

unsigned arity_of(const Node& n) { return n.type == N_UN ? 1 : n.type == N_BIN ? 2 : n.type == N_FMA ? 3 : 0; }

struct Parser {
    const SecantAstProgramList& routines;
    const uint8_t* arity;
    const ProgramRules& rules;
    std::vector<Node>& nodes;
    std::vector<SbAffine>& affines; /* of this program */
    unsigned n_ops = 0;

    int add(const Node& n) { nodes.push_back(n); return (int)nodes.size() - 1; }

    int affine_entry(uint32_t slot, float scale, float offset) {
        for (size_t i = 0; i < affines.size(); ++i)
            if (affines[i].slot == slot && !std::memcmp(&affines[i].scale, &scale, 4) &&
                !std::memcmp(&affines[i].offset, &offset, 4))
                return (int)i;
        affines.push_back(SbAffine{slot, scale, offset});
        return (int)affines.size() - 1;
    }

    /* One frame of the evaluator: its own value stack, arguments bound to nodes of the caller. */
    SecantResult frame(const SecantAstInstruction* code, const int* args, size_t num_args, unsigned depth, int* result) {
        int stack[SECANT_AST_MAX_STACK_DEPTH];
        size_t top = 0, leaves_in_a_row = 0, at = 0;
        if (!code) return SECANT_ERROR_BAD_PROGRAM;
        for (size_t n = 0; n < SECANT_AST_MAX_PROGRAM_INSTRUCTIONS; ++n) {
            const SecantAstInstruction* ins = code + at;
            Token t;
            const SecantResult token_status = read_token(ins, rules, &t);
            if (token_status != SECANT_SUCCESS) return token_status;
            const bool pushes = direct_leaf(t.kind) || t.kind == TK_ARG;
            if (t.kind == TK_ARG && (!args || ins[1] >= num_args)) return SECANT_ERROR_ROUTINE_ARG_IDX_OUT_OF_BOUNDS;
            if (pushes && top == SECANT_AST_MAX_STACK_DEPTH) return SECANT_ERROR_STACK_OVERFLOW;
            switch (t.kind) {
            case TK_COLUMN: { Node nd{N_COL}; nd.index = ins[1]; stack[top++] = add(nd); break; }
            case TK_BANK: { Node nd{N_BANK}; nd.index = ins[1]; stack[top++] = add(nd); break; }
            case TK_AFFINE: {
                Node nd{N_AFFINE};
                nd.index = (uint32_t)affine_entry(ins[1], secant_ast_affine_bank_scale_get(ins), secant_ast_affine_bank_offset_get(ins));
                stack[top++] = add(nd);
                break;
            }
            case TK_LITERAL: { Node nd{N_LIT}; nd.bits = secant_ast_constant_bits_get(ins); stack[top++] = add(nd); break; }
            case TK_ARG: stack[top++] = args[ins[1]]; break;
            case TK_TOGGLE: {
                if (leaves_in_a_row < t.ways || top < t.ways) return SECANT_ERROR_BAD_PROGRAM;
                Node nd{N_TOGGLE};
                nd.ways = t.ways; nd.bit0 = ins[1]; nd.bit1 = t.ways == 4 ? ins[2] : 0xff;
                for (size_t i = 0; i < t.ways; ++i) nd.child[i] = stack[top - t.ways + i];
                top -= t.ways;
                stack[top++] = add(nd);
                break;
            }
            case TK_CALL: {
                if (ins[1] >= routines.count || !routines.items[ins[1]]) return SECANT_ERROR_ROUTINE_IDX_OUT_OF_BOUNDS;
                if (depth >= kRoutineDepth) return SECANT_ERROR_ROUTINE_DEPTH_EXCEEDED;
                const size_t want = arity[ins[1]];
                if (top < want) return SECANT_ERROR_STACK_UNDERFLOW;
                int value = -1;
                const SecantResult r = frame(routines.items[ins[1]], stack + (top - want), want, depth + 1, &value);
                if (r != SECANT_SUCCESS) return r;
                top -= want;
                stack[top++] = value;
                break;
            }
            case TK_RETURN:
                if (top != 1u) return SECANT_ERROR_BAD_PROGRAM;
                *result = stack[0];
                return SECANT_SUCCESS;
            case TK_OPERATION: {
                if (!t.arity) return SECANT_ERROR_BAD_PROGRAM;
                if (top < t.arity) return SECANT_ERROR_STACK_UNDERFLOW;
                Node nd{t.node == 1 ? N_UN : t.node == 2 ? N_BIN : N_FMA};
                nd.op = t.op;
                for (unsigned i = 0; i < t.arity; ++i) nd.child[i] = stack[top - t.arity + i];
                top -= t.arity;
                stack[top++] = add(nd);
                ++n_ops;
                break;
            }
            }
            leaves_in_a_row = direct_leaf(t.kind) ? leaves_in_a_row + 1 : 0;
            at += t.width;
        }
        return SECANT_ERROR_BAD_PROGRAM;
    }
};

struct Operand {
    unsigned kind;
    unsigned index;
};

/* The instruction runs of a record.  The row prelude comes in two runs: values no toggle can change,
 * which an item that covers several permutations computes once, and values a toggle reaches. */
enum Run { RUN_BANK = 0, RUN_SHARED = 1, RUN_ROW = 2, RUN_MAIN = 3, NUM_RUNS = 4 };

/* rough executed-instruction weights used for scheduling (SbProgram::cost) and for choosing
 * which row-only sub-expressions are worth a hoist slot */
int unary_weight(unsigned op) {
    switch (op) {
    case SB_UN_NEG: case SB_UN_ABS: return 1;
    case SB_UN_SIN: case SB_UN_COS: return 18;
    case SB_UN_EXP: case SB_UN_EX2: return 9;
    case SB_UN_LOG: return 14;
    default: return 12;
    }
}
int binary_weight(unsigned op) { return (op == SB_BIN_DIV || op == SB_BIN_RDIV) ? 11 : 1; }
int insn_weight(const SbInsn& ins) {
    const unsigned cs = ins.w0 & 0xffu;
    if (cs >= SB_CASE_BIN && cs < SB_CASE_UN) return 1 + binary_weight((cs - SB_CASE_BIN) / SB_NUM_KINDS);
    if (cs >= SB_CASE_UN && cs < SB_CASE_FMA) return 1 + unary_weight(cs - SB_CASE_UN);
    if (cs == SB_CASE_FMA) return 12;
    return 2;
}

/* Bookkeeping rule of the emitter: gen(id) leaves the value of node `id` in the accumulator and
 * never consumes a use; the instruction that reads a value (as its accumulator input or as its
 * operand) consumes one use of it.  A computed node with several parents is parked in a slot
 * right after it is computed; a slot is released when the last use of its node is consumed. */
struct Emitter {
    std::vector<Node>& nodes;
    const ProgramRules& rules;
    EncodedBatch& out;
    size_t lit_base;
    unsigned n_affine;
    std::vector<SbInsn> code[NUM_RUNS];
    std::vector<SbPatch> sites[NUM_RUNS]; /* SbPatch::insn is relative to the run until the record is assembled */
    Run run = RUN_MAIN;
    std::vector<uint8_t> slot_busy;
    unsigned slots_high = 0, btmp_high = 0;
    unsigned n_entries = 0, n_hoisted = 0;
    bool uses_scratch = false;
    SecantResult error = SECANT_SUCCESS;
    struct LeafEntry { NodeType type; uint32_t key; int entry; };
    std::vector<LeafEntry> leaf_entries;

    Emitter(std::vector<Node>& nodes_, const ProgramRules& rules_, EncodedBatch& out_, unsigned n_affine_)
        : nodes(nodes_), rules(rules_), out(out_), lit_base(out_.lits.size()), n_affine(n_affine_) {}

    static bool leaf_type(const Node& n) { return n.type <= N_TOGGLE; }
    /* a value that can be named as an operand without computing anything */
    bool ready(int id) const {
        const Node& n = nodes[id];
        return leaf_type(n) || n.slot >= 0 || (run != RUN_BANK && n.hoisted >= 0) || n.entry >= 0;
    }

    ValueClass classify(int id) {
        Node& n = nodes[id];
        if (n.cls != VC_UNKNOWN) return n.cls;
        ValueClass c = VC_LITERAL;
        int w = 0;
        switch (n.type) {
        case N_COL: c = rules.columns_are_slots ? VC_MIXED : VC_ROW; break;
        case N_BANK: case N_AFFINE: c = VC_BANK; break;
        case N_LIT: break;
        case N_TOGGLE:
            for (unsigned i = 0; i < n.ways; ++i) c = join(c, classify(n.child[i]));
            break;
        default:
            for (unsigned i = 0; i < arity_of(n); ++i) {
                c = join(c, classify(nodes[id].child[i]));
                w += nodes[nodes[id].child[i]].weight;
            }
            w += n.type == N_UN ? unary_weight(n.op) : n.type == N_BIN ? binary_weight(n.op) : 4;
        }
        nodes[id].cls = c;
        nodes[id].weight = w;
        return c;
    }

    /* Sub-expressions to move out of the main part: maximal computed nodes whose value depends on
     * the bank only (or on nothing), and maximal computed nodes that depend on the row only.
     * Inside a row-only expression, literal-only computed nodes still go to the bank part. */
    void collect(int id, bool inside_row, std::vector<int>& bank_roots, std::vector<int>& row_roots, std::vector<uint8_t>& seen) {
        const unsigned mark = inside_row ? 2u : 1u;
        if (seen[(size_t)id] & mark) return;
        seen[(size_t)id] |= (uint8_t)mark;
        const Node& n = nodes[id];
        if (leaf_type(n)) return;
        const ValueClass c = classify(id);
        if (c <= VC_BANK && rules.hoist_bank) {
            if (std::find(bank_roots.begin(), bank_roots.end(), id) == bank_roots.end()) bank_roots.push_back(id);
            return;
        }
        if (c == VC_ROW && rules.hoist_row && !inside_row) {
            if (std::find(row_roots.begin(), row_roots.end(), id) == row_roots.end()) row_roots.push_back(id);
            inside_row = true;
        }
        for (unsigned i = 0; i < arity_of(n); ++i) collect(nodes[id].child[i], inside_row, bank_roots, row_roots, seen);
    }

    /* whether a toggle lies anywhere below the node: such a value changes with the permutation */
    bool reaches_toggle(int id, std::vector<int8_t>& memo) {
        if (memo[(size_t)id] >= 0) return memo[(size_t)id] != 0;
        const Node& n = nodes[id];
        bool any = n.type == N_TOGGLE;
        for (unsigned i = 0; i < arity_of(n) && !any; ++i) any = reaches_toggle(nodes[id].child[i], memo);
        memo[(size_t)id] = any ? 1 : 0;
        return any;
    }
    /* maximal computed row-only nodes below `id` that no toggle reaches */
    void collect_shared(int id, std::vector<int>& shared, std::vector<int8_t>& memo) {
        const Node& n = nodes[id];
        if (leaf_type(n)) return;
        if (classify(id) == VC_ROW && !reaches_toggle(id, memo)) {
            if (std::find(shared.begin(), shared.end(), id) == shared.end()) shared.push_back(id);
            return;
        }
        for (unsigned i = 0; i < arity_of(n); ++i) collect_shared(nodes[id].child[i], shared, memo);
    }

    int alloc_slot() {
        for (size_t i = 0; i < slot_busy.size(); ++i)
            if (!slot_busy[i]) { slot_busy[i] = 1; return (int)i; }
        if (slot_busy.size() >= kMaxSlots) { error = SECANT_ERROR_REGISTER_OVERFLOW; return 0; }
        slot_busy.push_back(1);
        unsigned& high = run == RUN_BANK ? btmp_high : slots_high;
        if (slot_busy.size() > high) high = (unsigned)slot_busy.size();
        return (int)slot_busy.size() - 1;
    }

    /* Every hoisted expression and the main part are emitted as separate phases that share nothing
     * but hoisted values and table entries: parent counts, pending uses and slots start afresh, so
     * a node needed by two phases is simply computed in both (a slot written during one row pass
     * of the prelude could not be trusted by the main part of every bank group). */
    void begin_phase(Run r, int phase_root) {
        run = r;
        for (auto& n : nodes) { n.uses = 0; n.pending = 0; n.slot = -1; }
        slot_busy.clear();
        if (r != RUN_BANK) slot_busy.assign(rules.reserved_slots, 1);
        prepare(phase_root);
        for (auto& n : nodes) n.pending = n.uses;
    }

    /* Counts parent references of every reachable node and computes how many slots each needs
     * while it is being evaluated (Sethi-Ullman numbers, DAG-agnostic estimate). */
    void prepare(int id) {
        Node& n = nodes[id];
        if (n.uses++ > 0) return;
        if (ready(id)) { n.su = 0; return; }
        const unsigned arity = arity_of(n);
        for (unsigned i = 0; i < arity; ++i) prepare(nodes[id].child[i]);
        int need[3], cnt = 0;
        for (unsigned i = 0; i < arity; ++i)
            if (!ready(nodes[id].child[i])) need[cnt++] = nodes[nodes[id].child[i]].su;
        for (int i = 0; i < cnt; ++i)
            for (int j = i + 1; j < cnt; ++j)
                if (need[j] > need[i]) std::swap(need[i], need[j]);
        int su = 0; /* the k-th operand evaluated coexists with k parked predecessors */
        for (int i = 0; i < cnt; ++i) su = std::max(su, need[i] + i);
        nodes[id].su = su;
    }

    void push(uint32_t w0, uint32_t w1) { code[run].push_back(SbInsn{w0, w1}); }

    void consume(int id) {
        Node& n = nodes[id];
        if (--n.pending == 0 && n.slot >= 0) { slot_busy[(size_t)n.slot] = 0; n.slot = -1; }
    }

    void park(int id) {
        const int s = alloc_slot();
        nodes[id].slot = s;
        push(sb_w0(SB_CASE_STORE, 0, (unsigned)s), 0);
    }

    /* Index of a source constant: bank slots, then the program's affine entries, then its literals. */
    unsigned source_index(const Node& n) {
        if (n.type == N_BANK) return n.index;
        if (n.type == N_AFFINE) return (unsigned)rules.num_constants + n.index;
        float f;
        std::memcpy(&f, &n.bits, 4);
        size_t i = lit_base;
        for (; i < out.lits.size(); ++i)
            if (!std::memcmp(&out.lits[i], &f, 4)) break;
        if (i == out.lits.size()) out.lits.push_back(f);
        return (unsigned)(rules.num_constants + n_affine + (i - lit_base));
    }

    /* Constant-table entry holding a constant leaf (or a toggle among constant leaves): appends
     * "load it; store entry" to the bank part the first time the leaf is needed. */
    int entry_for(int id) {
        Node& n = nodes[id];
        if (n.entry >= 0) return n.entry;
        if (n.type != N_TOGGLE) {
            const uint32_t key = n.type == N_LIT ? n.bits : n.index;
            for (const LeafEntry& l : leaf_entries)
                if (l.type == n.type && l.key == key) return nodes[id].entry = l.entry;
        }
        const Run saved = run;
        run = RUN_BANK;
        emit_reading(SB_CASE_LOAD, id);
        const int e = (int)n_entries++;
        push(sb_w0(SB_CASE_STOREH, 0, (unsigned)e), 0);
        run = saved;
        nodes[id].entry = e;
        if (nodes[id].type != N_TOGGLE) leaf_entries.push_back(LeafEntry{nodes[id].type, nodes[id].type == N_LIT ? nodes[id].bits : nodes[id].index, e});
        return e;
    }

    /* Descriptor of a parked or hoisted node or of a direct (non-toggle) leaf, in the run being emitted. */
    Operand describe(int id) {
        const Node& n = nodes[id];
        if (n.slot >= 0) return Operand{SB_KIND_SLOT, (unsigned)n.slot};
        if (n.hoisted >= 0 && run != RUN_BANK) return Operand{SB_KIND_ROW, SB_ROW_HOISTED | (unsigned)n.hoisted};
        if (n.entry >= 0) return Operand{run == RUN_BANK ? (unsigned)SB_KIND_ROW : (unsigned)SB_KIND_CST, (unsigned)n.entry};
        if (n.type == N_COL) return rules.columns_are_slots ? Operand{SB_KIND_SLOT, n.index} : Operand{SB_KIND_ROW, n.index};
        if (!rules.split_parts || run == RUN_BANK) return Operand{SB_KIND_CST, source_index(n)};
        return Operand{SB_KIND_CST, (unsigned)entry_for(id)};
    }

    /* Emits instruction "case_base + kind(operand)" reading `id`; an unparked toggle turns the
     * instruction into a patch site with one alternative per selectable leaf.  Does not consume. */
    void emit_reading(unsigned case_base, int id) {
        const Node& n = nodes[id];
        const bool open_toggle = n.type == N_TOGGLE && n.slot < 0 && n.entry < 0;
        if (open_toggle && rules.split_parts && run != RUN_BANK && classify(id) <= VC_BANK) {
            /* a toggle among constants is resolved once per bank in the bank part */
            const int e = entry_for(id);
            push(sb_w0(case_base + SB_KIND_CST, 0, (unsigned)e), 0);
            return;
        }
        if (open_toggle) {
            SbPatch p;
            std::memset(&p, 0, sizeof(p));
            p.bit0 = n.bit0;
            p.bit1 = n.bit1;
            for (unsigned i = 0; i < 4; ++i) { /* describing a constant leaf may append to the bank part first */
                const Operand o = describe(nodes[id].child[i < nodes[id].ways ? i : 0]);
                p.alt[i] = SbInsn{sb_w0(case_base + o.kind, 0, o.index), 0};
            }
            p.insn = (uint16_t)code[run].size();
            if (code[run].size() > 0xffffu) error = SECANT_ERROR_REGISTER_OVERFLOW;
            /* a site of the bank part names itself in the second word (1 + its position among the
             * program's sites, which begin with the bank part's): the scalar machine serves several
             * permutations at once and lets every lane take its own alternative */
            if (run == RUN_BANK)
                for (unsigned i = 0; i < 4; ++i) p.alt[i].w1 = (uint32_t)sites[RUN_BANK].size() + 1u;
            sites[run].push_back(p);
            push(p.alt[0].w0, p.alt[0].w1);
        } else {
            const Operand o = describe(id);
            push(sb_w0(case_base + o.kind, 0, o.index), 0);
        }
    }

    static unsigned reversed(unsigned op) {
        if (op == SB_BIN_SUB) return SB_BIN_RSUB;
        if (op == SB_BIN_DIV) return SB_BIN_RDIV;
        return op;
    }
    static unsigned bin_case(unsigned op) { return SB_CASE_BIN + op * SB_NUM_KINDS; }

    void gen(int id) {
        if (error != SECANT_SUCCESS) return;
        if (ready(id)) { emit_reading(SB_CASE_LOAD, id); return; }
        const Node n = nodes[id]; /* copy: the vector may grow below */
        if (n.type == N_UN) {
            gen(n.child[0]);
            push(sb_w0(SB_CASE_UN + n.op, 0, 0), 0);
            consume(n.child[0]);
        } else if (n.type == N_BIN) {
            const int l = n.child[0], r = n.child[1];
            if (l == r || ready(r)) {          /* acc = l ; acc = acc op r (l == r: gen parks it first) */
                gen(l);
                emit_reading(bin_case(n.op), r);
            } else if (ready(l)) {             /* acc = r ; acc = l op acc */
                gen(r);
                emit_reading(bin_case(reversed(n.op)), l);
            } else {                           /* both computed: the hungrier one goes through a slot */
                const bool left_first = nodes[l].su >= nodes[r].su;
                const int first = left_first ? l : r, second = left_first ? r : l;
                gen(first);
                if (nodes[first].slot < 0) park(first);
                gen(second);
                emit_reading(bin_case(left_first ? reversed(n.op) : n.op), first);
            }
            consume(l);
            consume(r);
        } else {
            gen_fma(n);
        }
        if (nodes[id].uses > 1) park(id);
    }

    void gen_fma(const Node& n) {
        int ch[3] = {n.child[0], n.child[1], n.child[2]};
        if (run != RUN_BANK) uses_scratch = true;
        /* a toggle operand (selected by a patched LOAD) or a hoisted per-row value cannot be
         * named by the FMA instruction: load it and park it in a private slot */
        for (int i = 0; i < 3; ++i) {
            const int id = ch[i];
            const bool toggle = nodes[id].type == N_TOGGLE && nodes[id].slot < 0 && nodes[id].entry < 0;
            const bool hrow = nodes[id].hoisted >= 0 && nodes[id].slot < 0 && run != RUN_BANK;
            const bool table = run == RUN_BANK && nodes[id].entry >= 0 && nodes[id].slot < 0;
            if (!toggle && !hrow && !table) continue;
            emit_reading(SB_CASE_LOAD, id);
            Node t{N_UN};
            t.cls = VC_MIXED;
            nodes.push_back(t);
            const int temp = (int)nodes.size() - 1;
            park(temp);
            for (int j = i; j < 3; ++j)
                if (ch[j] == id) { ch[j] = temp; ++nodes[temp].uses; ++nodes[temp].pending; consume(id); }
        }
        int todo[3], cnt = 0;
        for (int i = 0; i < 3; ++i) {
            bool seen = false;
            for (int j = 0; j < i; ++j) seen = seen || ch[j] == ch[i];
            if (!seen && !ready(ch[i])) todo[cnt++] = ch[i];
        }
        for (int i = 0; i < cnt; ++i)
            for (int j = i + 1; j < cnt; ++j)
                if (nodes[todo[j]].su > nodes[todo[i]].su) std::swap(todo[i], todo[j]);
        int in_acc = -1;
        for (int i = 0; i < cnt; ++i) {
            gen(todo[i]);
            if (nodes[todo[i]].slot >= 0) continue;     /* shared: gen parked it already */
            int positions = 0;
            for (int j = 0; j < 3; ++j) positions += ch[j] == todo[i];
            if (i + 1 < cnt || positions > 1) park(todo[i]);
            else in_acc = todo[i];
        }
        unsigned kinds = 0, idx = 0;
        for (int i = 0; i < 3; ++i) {
            unsigned kind = SB_FMA_ACC, index = 0;
            if (ch[i] != in_acc) {
                const Operand o = describe(ch[i]);
                kind = o.kind;
                index = o.index;
            }
            if (index >= 512u) { error = SECANT_ERROR_REGISTER_OVERFLOW; index = 0; }
            kinds |= kind << (2 * i);
            idx |= index << (10 * i);
        }
        push(sb_w0(SB_CASE_FMA, kinds, 0), idx);
        for (int i = 0; i < 3; ++i) consume(ch[i]);
    }

    /* Computes node `id` in run `r` and leaves it where later runs can read it. */
    void hoist(Run r, int id) {
        begin_phase(r, id);
        gen(id);
        if (error != SECANT_SUCCESS) return;
        if (r == RUN_BANK) {
            const unsigned e = n_entries++;
            push(sb_w0(SB_CASE_STOREH, 0, e), 0);
            nodes[id].entry = (int32_t)e;
        } else {
            const unsigned h = n_hoisted++;
            push(sb_w0(SB_CASE_STOREH, 0, h), 0);
            nodes[id].hoisted = (int32_t)h;
        }
    }
};

}  // namespace

SecantResult routine_arities(const SecantAstProgramList& routines, uint8_t* arity) {
    if (routines.count > SECANT_AST_MAX_ROUTINES || (routines.count && !routines.items)) return SECANT_ERROR_INVALID_VALUE;
    for (size_t i = 0; i < routines.count; ++i) {
        const SecantAstInstruction* code = routines.items[i];
        unsigned count = 0;
        size_t at = 0, n = 0;
        bool done = false;
        if (!code) return SECANT_ERROR_ROUTINE_IDX_OUT_OF_BOUNDS;
        for (; n < SECANT_AST_MAX_PROGRAM_INSTRUCTIONS && !done; ++n) {
            const SecantAstInstruction* ins = code + at;
            const size_t width = secant_ast_instruction_size_get(ins);
            if (!width) return SECANT_ERROR_BAD_PROGRAM;
            if (ins[0] == SECANT_AST_INSTRUCTION_TYPE_ROUTINE_ARG_F32) {
                if (ins[1] >= SECANT_AST_MAX_INSTRUCTION_ARGS) return SECANT_ERROR_TOO_MANY_ARGS;
                if (ins[1] + 1u > count) count = ins[1] + 1u;
            }
            done = ins[0] == SECANT_AST_INSTRUCTION_TYPE_RETURN_F32;
            at += width;
        }
        if (!done) return SECANT_ERROR_BAD_PROGRAM;
        arity[i] = (uint8_t)count;
    }
    return SECANT_SUCCESS;
}

/* Token-level scan of one program up to its RETURN: the checks of read_token() plus the one rule
 * that needs context, a toggle must directly follow as many direct leaves as it selects among. */
SecantResult preflight(const SecantAstInstruction* program, const ProgramRules& rules) {
    if (!program) return SECANT_ERROR_BAD_PROGRAM;
    size_t leaves_in_a_row = 0;
    const SecantAstInstruction* ins = program;
    for (size_t n = 0; n < SECANT_AST_MAX_PROGRAM_INSTRUCTIONS; ++n) {
        Token t;
        const SecantResult status = read_token(ins, rules, &t);
        if (status != SECANT_SUCCESS) return status;
        if (t.kind == TK_RETURN) return SECANT_SUCCESS;
        if (t.kind == TK_TOGGLE && leaves_in_a_row < t.ways) return SECANT_ERROR_BAD_PROGRAM;
        leaves_in_a_row = direct_leaf(t.kind) ? leaves_in_a_row + 1 : 0;
        ins += t.width;
    }
    return SECANT_ERROR_BAD_PROGRAM;
}

SecantResult encode_program(const SecantAstInstruction* program, const SecantAstProgramList& routines,
                            const uint8_t* routine_arity, const ProgramRules& rules, EncodedBatch& out) {
    std::vector<Node> nodes;
    std::vector<SbAffine> affines;
    nodes.reserve(64);
    Parser parser{routines, routine_arity, rules, nodes, affines};
    int root = -1;
    SecantResult r = parser.frame(program, nullptr, 0, 0, &root);
    if (r != SECANT_SUCCESS) return r;

    SbProgram rec;
    std::memset(&rec, 0, sizeof(rec));
    rec.insn_off = (uint32_t)out.insns.size();
    rec.patch_off = (uint32_t)out.patches.size();
    rec.affine_off = (uint32_t)out.affines.size();
    rec.lit_off = (uint32_t)out.lits.size();

    Emitter em(nodes, rules, out, (unsigned)affines.size());
    em.slots_high = rules.reserved_slots;
    const ValueClass root_class = em.classify(root);
    if (rules.split_parts) { /* rollout records (columns_are_slots) have no row-only class: only bank roots turn up */
        std::vector<int> bank_roots, row_roots;
        std::vector<uint8_t> seen(nodes.size(), 0);
        em.collect(root, false, bank_roots, row_roots, seen);
        /* row-only expressions a toggle reaches change with the permutation; what lies below them and
         * does not is worth a value of its own, computed once for all permutations of an item */
        std::vector<int8_t> memo(nodes.size(), -1);
        std::vector<int> shared_roots, toggled_roots;
        for (int id : row_roots) {
            if (!em.reaches_toggle(id, memo)) { shared_roots.push_back(id); continue; }
            if (rules.hoist_toggled) toggled_roots.push_back(id);
            em.collect_shared(id, shared_roots, memo);
        }
        /* keep the costliest values when there are more than the kernel has room for */
        std::vector<int> chosen(shared_roots);
        chosen.insert(chosen.end(), toggled_roots.begin(), toggled_roots.end());
        std::stable_sort(chosen.begin(), chosen.end(), [&](int a, int b) { return nodes[a].weight > nodes[b].weight; });
        if (chosen.size() > rules.max_hoisted) chosen.resize(rules.max_hoisted);
        /* operands before the expressions that use them: children were created first */
        std::sort(bank_roots.begin(), bank_roots.end());
        std::sort(chosen.begin(), chosen.end());
        for (int id : bank_roots) em.hoist(RUN_BANK, id);
        for (int id : chosen)
            if (!em.reaches_toggle(id, memo)) em.hoist(RUN_SHARED, id);
        for (int id : chosen)
            if (em.reaches_toggle(id, memo)) em.hoist(RUN_ROW, id);
        if (em.error != SECANT_SUCCESS) return em.error;
    }
    em.begin_phase(RUN_MAIN, root); /* counts the RETURN as the root's first use */
    em.gen(root);
    if (em.error != SECANT_SUCCESS) return em.error;
    em.consume(root);

    if (rules.fuse_store_load) { /* a toggle site keeps its own instruction: its alternatives are whole instructions */
        std::vector<SbInsn>& code = em.code[RUN_MAIN];
        std::vector<uint8_t> is_site(code.size(), 0);
        for (const SbPatch& p : em.sites[RUN_MAIN]) is_site[p.insn] = 1;
        std::vector<SbInsn> fused;
        std::vector<uint32_t> moved(code.size(), 0);
        fused.reserve(code.size());
        for (size_t i = 0; i < code.size(); ++i) {
            const unsigned cs = code[i].w0 & 0xffu;
            moved[i] = (uint32_t)fused.size();
            if (cs == SB_CASE_STORE && i + 1 < code.size() && !is_site[i + 1]) {
                const unsigned next = code[i + 1].w0 & 0xffu;
                if (next >= SB_CASE_LOAD && next < SB_CASE_LOAD + SB_NUM_KINDS) {
                    SbInsn both = code[i];
                    both.w1 = SB_STORE_THEN_LOAD | ((uint32_t)(next - SB_CASE_LOAD) << 16) | (code[i + 1].w0 >> 16);
                    fused.push_back(both);
                    moved[i + 1] = moved[i]; /* a site never sits on the absorbed load */
                    ++i;
                    continue;
                }
            }
            fused.push_back(code[i]);
        }
        for (SbPatch& p : em.sites[RUN_MAIN]) p.insn = (uint16_t)moved[p.insn];
        code.swap(fused);
    }

    /* assemble: bank part | shared row prelude | row prelude | main part, each closed by END; patch
     * sites become positions inside the whole record */
    size_t offset[NUM_RUNS] = {0, 0, 0, 0}, total = 0;
    for (int k = 0; k < NUM_RUNS; ++k) {
        offset[k] = total;
        if (k == RUN_MAIN || !em.code[k].empty()) total += em.code[k].size() + 1;
    }
    uint64_t cost = 0, pre_cost = 0;
    for (const SbInsn& i : em.code[RUN_MAIN]) cost += (uint64_t)insn_weight(i);
    for (const SbInsn& i : em.code[RUN_SHARED]) pre_cost += (uint64_t)insn_weight(i);
    for (const SbInsn& i : em.code[RUN_ROW]) pre_cost += (uint64_t)insn_weight(i);
    for (int k = 0; k < NUM_RUNS; ++k) {
        if (k != RUN_MAIN && em.code[k].empty()) continue;
        out.insns.insert(out.insns.end(), em.code[k].begin(), em.code[k].end());
        out.insns.push_back(SbInsn{sb_w0(SB_CASE_END, 0, 0), 0});
        for (SbPatch p : em.sites[k]) {
            const size_t at = offset[k] + p.insn;
            if (at > 0xffffu) return SECANT_ERROR_REGISTER_OVERFLOW;
            p.insn = (uint16_t)at;
            out.patches.push_back(p);
        }
    }

    const size_t n_patch = out.patches.size() - rec.patch_off;
    const size_t n_lits = out.lits.size() - rec.lit_off;
    if (total > 0xffffu || n_patch > 0xffffu || affines.size() + n_lits + rules.num_constants > 511u || em.n_entries > 511u ||
        em.n_hoisted > 255u)
        return SECANT_ERROR_REGISTER_OVERFLOW;
    out.affines.insert(out.affines.end(), affines.begin(), affines.end());
    rec.n_insn = (uint16_t)total;
    rec.n_patch = (uint16_t)n_patch;
    rec.n_affine = (uint16_t)affines.size();
    rec.n_lits = (uint16_t)n_lits;
    rec.n_slots = (uint16_t)em.slots_high;
    rec.n_ops = (uint16_t)(parser.n_ops > 0xffffu ? 0xffffu : parser.n_ops);
    rec.pre_off = (uint16_t)offset[RUN_SHARED];
    rec.mid_off = (uint16_t)offset[RUN_ROW];
    rec.main_off = (uint16_t)offset[RUN_MAIN];
    rec.n_hoisted = (uint16_t)em.n_hoisted;
    rec.n_cst = (uint16_t)em.n_entries;
    rec.n_btmp = (uint16_t)em.btmp_high;
    const bool bank_independent = rules.split_parts && !rules.columns_are_slots && (root_class == VC_LITERAL || root_class == VC_ROW);
    rec.flags = (uint16_t)((bank_independent ? SB_PROG_BANK_INDEPENDENT : 0) | (em.uses_scratch ? SB_PROG_USES_SCRATCH : 0));
    /* cost of one row pass: the main part (plus the loss epilogue) per bank group, the prelude once;
     * the kernel scales the first term by the bank groups an item covers */
    rec.cost = (uint32_t)std::min<uint64_t>(0xffffu, cost + 6) | ((uint32_t)std::min<uint64_t>(0xffffu, pre_cost) << 16);
    out.programs.push_back(rec);
    out.max_insn = std::max<unsigned>(out.max_insn, (unsigned)total);
    out.max_extra = std::max<unsigned>(out.max_extra, (unsigned)(affines.size() + n_lits));
    out.max_slots = std::max(out.max_slots, em.slots_high);
    out.max_patch = std::max<unsigned>(out.max_patch, (unsigned)n_patch);
    out.max_hoisted = std::max(out.max_hoisted, em.n_hoisted);
    out.max_cst = std::max(out.max_cst, em.n_entries);
    out.max_btmp = std::max(out.max_btmp, em.btmp_high);
    out.uses_scratch = out.uses_scratch || em.uses_scratch;
    return SECANT_SUCCESS;
}

}  // namespace sb
