/*
 * encoder.cpp - postfix bytecode -> accumulator-machine record.
 *
 * Stage 1 (parse) walks the byte stream exactly like the reference evaluator and
 * specializer do (projects/secant/s_cpu.c:193-414, s_cubin_specialize.c:1203-1368):
 * same per-token checks in the same order, routine calls expanded in place with their
 * arguments bound once.  It builds an expression DAG (a routine argument used several
 * times becomes a shared node).
 * Stage 2 (emit) linearises the DAG for a machine with one accumulator: a binary node
 * whose other operand is a leaf costs one instruction, a node with two computed
 * operands spills the first through a slot.  The deeper operand is evaluated first
 * (Sethi-Ullman order), which only changes the order pure sub-expressions are computed
 * in, never how values are rounded or associated.
 */
#include "encoder.h"

#include <cmath>
#include <cstring>

namespace sb {

void EncodedBatch::clear() {
    programs.clear(); insns.clear(); patches.clear(); affines.clear(); lits.clear();
    max_insn = 1; max_extra = 0; max_slots = 0; max_patch = 0; max_hoisted = 0;
}

namespace {

bool is_f32_opcode(unsigned op) {
    return op == SECANT_AST_INSTRUCTION_TYPE_AFFINE_BANK_F32 || op == SECANT_AST_INSTRUCTION_TYPE_COLUMN_F32 ||
           op == SECANT_AST_INSTRUCTION_TYPE_BANK_CONSTANT_F32 || op == SECANT_AST_INSTRUCTION_TYPE_TOGGLE2_F32 ||
           op == SECANT_AST_INSTRUCTION_TYPE_TOGGLE4_F32 ||
           (op >= SECANT_AST_INSTRUCTION_TYPE_CONSTANT_BITS_F32 && op <= SECANT_AST_INSTRUCTION_TYPE_TANH_F32) ||
           op == SECANT_AST_INSTRUCTION_TYPE_EXP_F32 || op == SECANT_AST_INSTRUCTION_TYPE_LOG_F32;
}

enum NodeType : uint8_t { N_COL, N_BANK, N_AFFINE, N_LIT, N_TOGGLE, N_UN, N_BIN, N_FMA };

struct Node {
    NodeType type;
    uint8_t op = 0;       /* SB_UN_* for N_UN, SB_BIN_{ADD,SUB,MUL,DIV,MIN,MAX} for N_BIN */
    uint8_t ways = 0;     /* toggle: 2 or 4 */
    uint8_t bit0 = 0, bit1 = 0xff;
    int32_t child[4] = {-1, -1, -1, -1};
    uint32_t index = 0;   /* column / bank slot / affine entry */
    uint32_t bits = 0;    /* literal */
    int32_t uses = 0;     /* parents (a routine argument may have several) */
    int32_t pending = 0;  /* uses not yet emitted */
    int32_t slot = -1;    /* spill slot holding the value, once computed */
    int32_t su = 0;       /* slots needed to compute the node into the accumulator */
    int8_t varies = -1;   /* depends on a coefficient bank (memoised, -1 = unknown) */
    int32_t hoisted = -1; /* index of the per-row value the prelude left, once hoisted */
    int32_t weight = 0;   /* rough instruction cost of the sub-expression */
};

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

    SecantResult frame(const SecantAstInstruction* code, const int* args, size_t num_args, unsigned depth, int* result) {
        int stack[SECANT_AST_MAX_STACK_DEPTH];
        size_t top = 0, direct_run = 0, at = 0;
        if (!code) return SECANT_ERROR_BAD_PROGRAM;
        for (size_t n = 0; n < SECANT_AST_MAX_PROGRAM_INSTRUCTIONS; ++n) {
            const SecantAstInstruction* ins = code + at;
            const unsigned op = ins[0];
            const size_t width = secant_ast_instruction_size_get(ins);
            bool direct = false;
            if (!width) return SECANT_ERROR_BAD_PROGRAM;
            if (!is_f32_opcode(op)) return SECANT_ERROR_UNSUPPORTED_OP;
            switch (op) {
            case SECANT_AST_INSTRUCTION_TYPE_COLUMN_F32: {
                if (ins[1] >= rules.num_columns) return SECANT_ERROR_BAD_PROGRAM;
                if (top == SECANT_AST_MAX_STACK_DEPTH) return SECANT_ERROR_STACK_OVERFLOW;
                Node nd{N_COL}; nd.index = ins[1];
                stack[top++] = add(nd); direct = true;
                break;
            }
            case SECANT_AST_INSTRUCTION_TYPE_BANK_CONSTANT_F32:
            case SECANT_AST_INSTRUCTION_TYPE_AFFINE_BANK_F32: {
                if (!rules.banks_allowed || ins[1] >= rules.num_constants) return SECANT_ERROR_BAD_PROGRAM;
                if (top == SECANT_AST_MAX_STACK_DEPTH) return SECANT_ERROR_STACK_OVERFLOW;
                if (op == SECANT_AST_INSTRUCTION_TYPE_AFFINE_BANK_F32) {
                    const float scale = secant_ast_affine_bank_scale_get(ins), offset = secant_ast_affine_bank_offset_get(ins);
                    if (!std::isfinite(scale) || !std::isfinite(offset)) return SECANT_ERROR_BAD_PROGRAM;
                    Node nd{N_AFFINE}; nd.index = (uint32_t)affine_entry(ins[1], scale, offset);
                    stack[top++] = add(nd);
                } else {
                    Node nd{N_BANK}; nd.index = ins[1];
                    stack[top++] = add(nd);
                }
                direct = true;
                break;
            }
            case SECANT_AST_INSTRUCTION_TYPE_CONSTANT_BITS_F32: {
                if (top == SECANT_AST_MAX_STACK_DEPTH) return SECANT_ERROR_STACK_OVERFLOW;
                Node nd{N_LIT}; nd.bits = secant_ast_constant_bits_get(ins);
                stack[top++] = add(nd); direct = true;
                break;
            }
            case SECANT_AST_INSTRUCTION_TYPE_TOGGLE2_F32:
            case SECANT_AST_INSTRUCTION_TYPE_TOGGLE4_F32: {
                const size_t ways = op == SECANT_AST_INSTRUCTION_TYPE_TOGGLE2_F32 ? 2u : 4u;
                if (!rules.banks_allowed || ins[1] >= rules.toggle_bits || direct_run < ways || top < ways)
                    return SECANT_ERROR_BAD_PROGRAM;
                if (ways == 4u && (ins[2] >= rules.toggle_bits || ins[2] == ins[1])) return SECANT_ERROR_BAD_PROGRAM;
                Node nd{N_TOGGLE}; nd.ways = (uint8_t)ways; nd.bit0 = ins[1]; nd.bit1 = ways == 4u ? ins[2] : 0xff;
                for (size_t i = 0; i < ways; ++i) nd.child[i] = stack[top - ways + i];
                top -= ways;
                stack[top++] = add(nd);
                break;
            }
            case SECANT_AST_INSTRUCTION_TYPE_ROUTINE_ARG_F32:
                if (!args || ins[1] >= num_args) return SECANT_ERROR_ROUTINE_ARG_IDX_OUT_OF_BOUNDS;
                if (top == SECANT_AST_MAX_STACK_DEPTH) return SECANT_ERROR_STACK_OVERFLOW;
                stack[top++] = args[ins[1]];
                break;
            case SECANT_AST_INSTRUCTION_TYPE_ROUTINE_F32: {
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
            case SECANT_AST_INSTRUCTION_TYPE_RETURN_F32:
                if (top != 1u) return SECANT_ERROR_BAD_PROGRAM;
                *result = stack[0];
                return SECANT_SUCCESS;
            default: {
                Node nd{N_UN};
                unsigned want = 1;
                switch (op) {
                case SECANT_AST_INSTRUCTION_TYPE_ADD_F32: nd.type = N_BIN; nd.op = SB_BIN_ADD; want = 2; break;
                case SECANT_AST_INSTRUCTION_TYPE_SUB_F32: nd.type = N_BIN; nd.op = SB_BIN_SUB; want = 2; break;
                case SECANT_AST_INSTRUCTION_TYPE_MUL_F32: nd.type = N_BIN; nd.op = SB_BIN_MUL; want = 2; break;
                case SECANT_AST_INSTRUCTION_TYPE_DIV_F32: nd.type = N_BIN; nd.op = SB_BIN_DIV; want = 2; break;
                case SECANT_AST_INSTRUCTION_TYPE_MIN_F32: nd.type = N_BIN; nd.op = SB_BIN_MIN; want = 2; break;
                case SECANT_AST_INSTRUCTION_TYPE_MAX_F32: nd.type = N_BIN; nd.op = SB_BIN_MAX; want = 2; break;
                case SECANT_AST_INSTRUCTION_TYPE_FMA_F32: nd.type = N_FMA; want = 3; break;
                case SECANT_AST_INSTRUCTION_TYPE_NEG_F32: nd.op = SB_UN_NEG; break;
                case SECANT_AST_INSTRUCTION_TYPE_SQRT_F32: nd.op = SB_UN_SQRT; break;
                case SECANT_AST_INSTRUCTION_TYPE_RCP_F32: nd.op = SB_UN_RCP; break;
                case SECANT_AST_INSTRUCTION_TYPE_ABS_F32: nd.op = SB_UN_ABS; break;
                case SECANT_AST_INSTRUCTION_TYPE_SIN_F32: nd.op = SB_UN_SIN; break;
                case SECANT_AST_INSTRUCTION_TYPE_COS_F32: nd.op = SB_UN_COS; break;
                case SECANT_AST_INSTRUCTION_TYPE_EX2_F32: nd.op = SB_UN_EX2; break;
                case SECANT_AST_INSTRUCTION_TYPE_LG2_F32: nd.op = SB_UN_LG2; break;
                case SECANT_AST_INSTRUCTION_TYPE_RSQRT_F32: nd.op = SB_UN_RSQRT; break;
                case SECANT_AST_INSTRUCTION_TYPE_TANH_F32: nd.op = SB_UN_TANH; break;
                case SECANT_AST_INSTRUCTION_TYPE_EXP_F32: nd.op = SB_UN_EXP; break;
                case SECANT_AST_INSTRUCTION_TYPE_LOG_F32: nd.op = SB_UN_LOG; break;
                default: return SECANT_ERROR_BAD_PROGRAM; /* NONE: decodable but not evaluable */
                }
                if (top < want) return SECANT_ERROR_STACK_UNDERFLOW;
                for (unsigned i = 0; i < want; ++i) nd.child[i] = stack[top - want + i];
                top -= want;
                stack[top++] = add(nd);
                ++n_ops;
                break;
            }
            }
            direct_run = direct ? direct_run + 1 : 0;
            at += width;
        }
        return SECANT_ERROR_BAD_PROGRAM;
    }
};

struct Operand {
    unsigned kind;
    unsigned index;
    uint32_t imm;
};

/* Bookkeeping rule of the emitter: gen(id) leaves the value of node `id` in the
 * accumulator and never consumes a use; the instruction that reads a value (as its
 * accumulator input or as its operand) consumes one use of it.  A computed node with
 * several parents is parked in a slot right after it is computed; a slot is released when
 * the last use of its node is consumed. */
struct Emitter {
    std::vector<Node>& nodes;
    const ProgramRules& rules;
    EncodedBatch& out;
    size_t insn_base, lit_base;
    unsigned n_affine;
    std::vector<uint8_t> slot_busy;
    unsigned slots_high;
    SecantResult error;

    static bool leaf_type(const Node& n) { return n.type <= N_TOGGLE; }
    bool ready(int id) const { return leaf_type(nodes[id]) || nodes[id].slot >= 0 || nodes[id].hoisted >= 0; }

    int alloc_slot() {
        for (size_t i = 0; i < slot_busy.size(); ++i)
            if (!slot_busy[i]) { slot_busy[i] = 1; return (int)i; }
        if (slot_busy.size() >= kMaxSlots) { error = SECANT_ERROR_REGISTER_OVERFLOW; return 0; }
        slot_busy.push_back(1);
        if (slot_busy.size() > slots_high) slots_high = (unsigned)slot_busy.size();
        return (int)slot_busy.size() - 1;
    }

    /* The prelude expressions and the main part are emitted as separate phases that share
     * nothing but hoisted values: parent counts, pending uses and slots start afresh, so a
     * node needed by two phases is simply computed in both (a slot written by the prelude of
     * one row pass could not be trusted by the main part of every bank group). */
    void begin_phase(int phase_root) {
        for (auto& n : nodes) { n.uses = 0; n.pending = 0; n.slot = -1; }
        std::fill(slot_busy.begin(), slot_busy.end(), 0);
        for (unsigned i = 0; i < rules.reserved_slots && i < slot_busy.size(); ++i) slot_busy[i] = 1;
        prepare(phase_root);
        for (auto& n : nodes) n.pending = n.uses;
    }

    /* Counts parent references of every reachable node and computes how many slots each
     * needs while it is being evaluated (Sethi-Ullman numbers, DAG-agnostic estimate). */
    void prepare(int id) {
        Node& n = nodes[id];
        if (n.uses++ > 0) return;
        if (leaf_type(n) || n.hoisted >= 0) { n.su = 0; return; } /* a hoisted value is read like a leaf */
        const unsigned arity = n.type == N_UN ? 1 : n.type == N_BIN ? 2 : 3;
        for (unsigned i = 0; i < arity; ++i) prepare(nodes[id].child[i]);
        int need[3], cnt = 0;
        for (unsigned i = 0; i < arity; ++i)
            if (!leaf_type(nodes[nodes[id].child[i]]) && nodes[nodes[id].child[i]].hoisted < 0) need[cnt++] = nodes[nodes[id].child[i]].su;
        for (int i = 0; i < cnt; ++i)
            for (int j = i + 1; j < cnt; ++j)
                if (need[j] > need[i]) { int t = need[i]; need[i] = need[j]; need[j] = t; }
        int su = 0; /* the k-th operand evaluated coexists with k parked predecessors */
        for (int i = 0; i < cnt; ++i) su = su > need[i] + i ? su : need[i] + i;
        nodes[id].su = su;
    }

    void push(uint32_t w0, uint32_t w1) { out.insns.push_back(SbInsn{w0, w1}); }

    void consume(int id) {
        Node& n = nodes[id];
        if (--n.pending == 0 && n.slot >= 0) { slot_busy[(size_t)n.slot] = 0; n.slot = -1; }
    }

    void park(int id) {
        const int s = alloc_slot();
        nodes[id].slot = s;
        push(sb_w0(SB_CASE_STORE, 0, (unsigned)s), 0);
    }

    /* Descriptor of a parked node or of a direct (non-toggle) leaf.  Immediates are only
     * legal for LOAD and binary instructions; FMA reads literals from the constant area. */
    Operand describe(int id, bool allow_imm) {
        const Node& n = nodes[id];
        if (n.slot >= 0) return Operand{SB_KIND_SLOT, (unsigned)n.slot, 0};
        if (n.hoisted >= 0) return Operand{SB_KIND_ROW, SB_ROW_HOISTED | (unsigned)n.hoisted, 0};
        switch (n.type) {
        case N_COL: return rules.columns_are_slots ? Operand{SB_KIND_SLOT, n.index, 0} : Operand{SB_KIND_ROW, n.index, 0};
        case N_BANK: return Operand{SB_KIND_CST, n.index, 0};
        case N_AFFINE: return Operand{SB_KIND_CST, (unsigned)rules.num_constants + n.index, 0};
        default: break;
        }
        (void)allow_imm; /* literals always live in the program's part of the constant area */
        float f;
        std::memcpy(&f, &n.bits, 4);
        size_t i = lit_base;
        for (; i < out.lits.size(); ++i)
            if (!std::memcmp(&out.lits[i], &f, 4)) break;
        if (i == out.lits.size()) out.lits.push_back(f);
        return Operand{SB_KIND_CST, (unsigned)(rules.num_constants + n_affine + (i - lit_base)), 0};
    }

    /* Emits instruction "case_base + kind(operand)" reading `id`; an unparked toggle turns the
     * instruction into a patch site with one alternative per selectable leaf.  Does not consume. */
    void emit_reading(unsigned case_base, int id) {
        const Node& n = nodes[id];
        if (n.type == N_TOGGLE && n.slot < 0) {
            SbPatch p;
            std::memset(&p, 0, sizeof(p));
            p.insn = (uint16_t)(out.insns.size() - insn_base);
            p.bit0 = n.bit0;
            p.bit1 = n.bit1;
            for (unsigned i = 0; i < 4; ++i) {
                const Operand o = describe(n.child[i < n.ways ? i : 0], true);
                p.alt[i] = SbInsn{sb_w0(case_base + o.kind, 0, o.index), o.imm};
            }
            out.patches.push_back(p);
            push(p.alt[0].w0, p.alt[0].w1);
        } else {
            const Operand o = describe(id, true);
            push(sb_w0(case_base + o.kind, 0, o.index), o.imm);
        }
    }

    static unsigned reversed(unsigned op) {
        if (op == SB_BIN_SUB) return SB_BIN_RSUB;
        if (op == SB_BIN_DIV) return SB_BIN_RDIV;
        return op;
    }
    static unsigned bin_case(unsigned op) { return SB_CASE_BIN + op * SB_NUM_KINDS; }

    /* Does the value of `id` depend on the coefficient bank?  Also accumulates a rough cost. */
    bool varies(int id) {
        Node& n = nodes[id];
        if (n.varies >= 0) return n.varies != 0;
        bool v = false;
        int w = 0;
        switch (n.type) {
        case N_BANK: case N_AFFINE: v = true; break;
        case N_COL: case N_LIT: break;
        case N_TOGGLE:
            for (unsigned i = 0; i < n.ways; ++i) v = varies(n.child[i]) || v;
            break;
        default: {
            const unsigned arity = n.type == N_UN ? 1 : n.type == N_BIN ? 2 : 3;
            for (unsigned i = 0; i < arity; ++i) { v = varies(nodes[id].child[i]) || v; w += nodes[nodes[id].child[i]].weight; }
            if (n.type == N_UN) w += (n.op == SB_UN_NEG || n.op == SB_UN_ABS) ? 1 : 20;
            else if (n.type == N_BIN) w += n.op == SB_BIN_DIV ? 10 : 1;
            else w += 4;
        }
        }
        nodes[id].varies = v ? 1 : 0;
        nodes[id].weight = w;
        return v;
    }
    /* Maximal bank-independent computed sub-expressions below `id`. */
    void collect_invariants(int id, std::vector<int>& found, std::vector<uint8_t>& seen) {
        if (seen[(size_t)id]) return;
        seen[(size_t)id] = 1;
        const Node& n = nodes[id];
        if (leaf_type(n)) return;
        if (!varies(id)) { found.push_back(id); return; }
        const unsigned arity = n.type == N_UN ? 1 : n.type == N_BIN ? 2 : 3;
        for (unsigned i = 0; i < arity; ++i) collect_invariants(nodes[id].child[i], found, seen);
    }
    /* Emits the prelude: every kept invariant sub-expression is computed and parked in a slot
     * that stays reserved for the rest of the program.  Returns how many were hoisted. */
    unsigned emit_prelude(int root) {
        std::vector<int> found;
        std::vector<uint8_t> seen(nodes.size(), 0);
        collect_invariants(root, found, seen);
        if (found.empty()) return 0;
        for (size_t i = 0; i < found.size(); ++i)          /* heaviest first, then keep the budget */
            for (size_t j = i + 1; j < found.size(); ++j)
                if (nodes[found[j]].weight > nodes[found[i]].weight) { int t = found[i]; found[i] = found[j]; found[j] = t; }
        if (found.size() > rules.max_hoisted) found.resize(rules.max_hoisted);
        for (size_t i = 0; i < found.size(); ++i)          /* operands before the expressions that use them */
            for (size_t j = i + 1; j < found.size(); ++j)
                if (found[j] < found[i]) { int t = found[i]; found[i] = found[j]; found[j] = t; }
        unsigned h = 0;
        for (int id : found) {
            begin_phase(id);
            gen(id);
            if (error != SECANT_SUCCESS) return 0;
            push(sb_w0(SB_CASE_STOREH, 0, h), 0);
            nodes[id].hoisted = (int32_t)h++;
        }
        push(sb_w0(SB_CASE_END, 0, 0), 0);
        return (unsigned)found.size();
    }

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
        /* a toggle operand (selected by a patched LOAD) or a hoisted per-row value cannot be
         * named by the FMA instruction: load it and park it in a private slot */
        for (int i = 0; i < 3; ++i) {
            const int id = ch[i];
            const bool toggle = nodes[id].type == N_TOGGLE && nodes[id].slot < 0;
            const bool hrow = nodes[id].hoisted >= 0 && nodes[id].slot < 0;
            if (!toggle && !hrow) continue;
            emit_reading(SB_CASE_LOAD, id);
            Node t{N_UN};
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
                if (nodes[todo[j]].su > nodes[todo[i]].su) { int t = todo[i]; todo[i] = todo[j]; todo[j] = t; }
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
                const Operand o = describe(ch[i], false);
                kind = o.kind;
                index = o.index;
            }
            if (index >= 1024u) { error = SECANT_ERROR_REGISTER_OVERFLOW; index = 0; }
            kinds |= kind << (2 * i);
            idx |= index << (10 * i);
        }
        push(sb_w0(SB_CASE_FMA, kinds, 0), idx);
        for (int i = 0; i < 3; ++i) consume(ch[i]);
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

SecantResult preflight(const SecantAstInstruction* program, const ProgramRules& rules) {
    size_t at = 0, direct = 0;
    if (!program) return SECANT_ERROR_BAD_PROGRAM;
    for (size_t n = 0; n < SECANT_AST_MAX_PROGRAM_INSTRUCTIONS; ++n) {
        const SecantAstInstruction* ins = program + at;
        const unsigned op = ins[0];
        const size_t width = secant_ast_instruction_size_get(ins);
        if (!width) return SECANT_ERROR_BAD_PROGRAM;
        if (!is_f32_opcode(op)) return SECANT_ERROR_UNSUPPORTED_OP;
        if (op == SECANT_AST_INSTRUCTION_TYPE_RETURN_F32) return SECANT_SUCCESS;
        if (op == SECANT_AST_INSTRUCTION_TYPE_COLUMN_F32) {
            if (ins[1] >= rules.num_columns) return SECANT_ERROR_BAD_PROGRAM;
            ++direct;
        } else if (op == SECANT_AST_INSTRUCTION_TYPE_BANK_CONSTANT_F32 || op == SECANT_AST_INSTRUCTION_TYPE_AFFINE_BANK_F32) {
            if (!rules.banks_allowed || ins[1] >= rules.num_constants) return SECANT_ERROR_BAD_PROGRAM;
            if (op == SECANT_AST_INSTRUCTION_TYPE_AFFINE_BANK_F32 &&
                (!std::isfinite(secant_ast_affine_bank_scale_get(ins)) || !std::isfinite(secant_ast_affine_bank_offset_get(ins))))
                return SECANT_ERROR_BAD_PROGRAM;
            ++direct;
        } else if (op == SECANT_AST_INSTRUCTION_TYPE_CONSTANT_BITS_F32) {
            ++direct;
        } else {
            if (op == SECANT_AST_INSTRUCTION_TYPE_TOGGLE2_F32 || op == SECANT_AST_INSTRUCTION_TYPE_TOGGLE4_F32) {
                const size_t ways = op == SECANT_AST_INSTRUCTION_TYPE_TOGGLE2_F32 ? 2u : 4u;
                if (!rules.banks_allowed || ins[1] >= rules.toggle_bits || direct < ways ||
                    (ways == 4u && (ins[2] >= rules.toggle_bits || ins[1] == ins[2])))
                    return SECANT_ERROR_BAD_PROGRAM;
            }
            direct = 0;
        }
        at += width;
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

    Emitter em{nodes, rules, out, out.insns.size(), out.lits.size(), (unsigned)affines.size(), {}, 0, SECANT_SUCCESS};
    em.slot_busy.assign(rules.reserved_slots, 1);
    em.slots_high = rules.reserved_slots;
    unsigned hoisted = 0;
    if (rules.hoist_invariants && !rules.columns_are_slots) hoisted = em.emit_prelude(root);
    if (em.error != SECANT_SUCCESS) return em.error;
    const size_t main_off = hoisted ? out.insns.size() - rec.insn_off : 0;
    em.begin_phase(root); /* counts the RETURN as the root's first use */
    em.gen(root);
    if (em.error != SECANT_SUCCESS) return em.error;
    em.push(sb_w0(SB_CASE_END, 0, 0), 0);
    em.consume(root);

    const size_t n_insn = out.insns.size() - rec.insn_off;
    const size_t n_patch = out.patches.size() - rec.patch_off;
    const size_t n_lits = out.lits.size() - rec.lit_off;
    if (n_insn > 0xffffu || n_patch > 0xffffu || affines.size() + n_lits + rules.num_constants > 1023u)
        return SECANT_ERROR_REGISTER_OVERFLOW;
    out.affines.insert(out.affines.end(), affines.begin(), affines.end());
    rec.n_insn = (uint16_t)n_insn;
    rec.n_patch = (uint16_t)n_patch;
    rec.n_affine = (uint16_t)affines.size();
    rec.n_lits = (uint16_t)n_lits;
    rec.n_slots = (uint16_t)em.slots_high;
    rec.n_ops = (uint16_t)(parser.n_ops > 0xffffu ? 0xffffu : parser.n_ops);
    rec.main_off = (uint16_t)main_off;
    rec.n_hoisted = (uint16_t)hoisted;
    out.programs.push_back(rec);
    if (n_insn > out.max_insn) out.max_insn = (unsigned)n_insn;
    if (affines.size() + n_lits > out.max_extra) out.max_extra = (unsigned)(affines.size() + n_lits);
    if (em.slots_high > out.max_slots) out.max_slots = em.slots_high;
    if (n_patch > out.max_patch) out.max_patch = (unsigned)n_patch;
    if (hoisted > out.max_hoisted) out.max_hoisted = hoisted;
    return SECANT_SUCCESS;
}

}  // namespace sb
