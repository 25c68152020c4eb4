"""Program bytecode builders and seeded synthetic workloads.

Byte layout of tokens follows the reference encoders
(projects/secant/secant_instructions.h:86-120, 253-322).  The workload generators produce
the synthetic stand-ins for the benchmark configurations: seeded random postfix programs
with the operation set {+, -, *, protected /, sin, cos, exp, protected log}, where the
protected forms are routine calls over base opcodes, as the reference's own random
tests express them (projects/secant/tests/support/ast_stress.c:47-113, 547-577):

    pdiv(x, y) = x * y / (y * y + 0.01)    (projects/secant/bench/corpus/README.md:62-68)
    plog(x)    = log(abs(x) + 1)            (natural-log analogue of the reference's safe_lg2)
"""
import ctypes as C
import struct

import numpy as np

OP = dict(
    NONE=0x80, LIT=0x81, ROUTINE=0x82, RET=0x83, ARG=0x84, ADD=0x85, SUB=0x86, MUL=0x87, DIV=0x88, NEG=0x89, SQRT=0x8A,
    RCP=0x8B, ABS=0x8C, MIN=0x8D, MAX=0x8E, FMA=0x8F, SIN=0x90, COS=0x91, EX2=0x92, LG2=0x93, RSQRT=0x94, TANH=0x95,
    COL=0xB6, EXP=0xBA, LOG=0xBB, BANK=0xBC, TOG2=0xBD, TOG4=0xBE, AFFINE=0xBF,
)
UNARY = ("NEG", "SQRT", "RCP", "ABS", "SIN", "COS", "EX2", "LG2", "RSQRT", "TANH", "EXP", "LOG")
BINARY = ("ADD", "SUB", "MUL", "DIV", "MIN", "MAX")


def col(i):
    return bytes([OP["COL"], i])


def bank(i):
    return bytes([OP["BANK"], i])


def lit(x):
    return bytes([OP["LIT"]]) + struct.pack("<f", np.float32(x))


def lit_bits(bits):
    return bytes([OP["LIT"]]) + struct.pack("<I", bits)


def affine(slot, scale, offset):
    return bytes([OP["AFFINE"], slot]) + struct.pack("<ff", np.float32(scale), np.float32(offset))


def tog2(bit):
    return bytes([OP["TOG2"], bit])


def tog4(bit0, bit1):
    return bytes([OP["TOG4"], bit0, bit1])


def routine(i):
    return bytes([OP["ROUTINE"], i])


def arg(i):
    return bytes([OP["ARG"], i])


def op(name):
    return bytes([OP[name]])


RET = bytes([OP["RET"]])

PDIV = arg(0) + arg(1) + op("MUL") + arg(1) + arg(1) + op("MUL") + lit(0.01) + op("ADD") + op("DIV") + RET
PLOG = arg(0) + op("ABS") + lit(1.0) + op("ADD") + op("LOG") + RET
PROTECTED_ROUTINES = [PDIV, PLOG]  # routine 0 = pdiv (4 ops), routine 1 = plog (3 ops)


class PackedPrograms:
    """Programs as one byte blob plus offsets, and as the pointer arrays the C API takes."""

    def __init__(self, asts, routines=()):
        self.asts = [bytes(a) for a in asts]
        self.routines = [bytes(r) for r in routines]
        self.ast_blob, self.ast_off = self._pack(self.asts)
        self.routine_blob, self.routine_off = self._pack(self.routines)
        self._ast_buf = (C.c_uint8 * max(1, len(self.ast_blob))).from_buffer_copy(self.ast_blob or b"\0")
        self._routine_buf = (C.c_uint8 * max(1, len(self.routine_blob))).from_buffer_copy(self.routine_blob or b"\0")
        self._ast_ptrs = self._pointers(self._ast_buf, self.ast_off)
        self._routine_ptrs = self._pointers(self._routine_buf, self.routine_off)

    @staticmethod
    def _pack(items):
        offsets = np.zeros(max(1, len(items)), dtype=np.uint64)
        at = 0
        for i, it in enumerate(items):
            offsets[i] = at
            at += len(it)
        return b"".join(items), offsets

    @staticmethod
    def _pointers(buf, offsets):
        base = C.addressof(buf)
        arr = (C.POINTER(C.c_uint8) * len(offsets))()
        addresses = (base + offsets.astype(np.uint64)).astype(np.uint64)
        C.memmove(arr, addresses.ctypes.data, 8 * len(offsets))
        return arr

    def fill(self, program_set):
        """Writes the pointer/count views into an abi.ProgramSet."""
        program_set.asts.items = C.cast(self._ast_ptrs, C.POINTER(C.POINTER(C.c_uint8)))
        program_set.asts.count = len(self.asts)
        if self.routines:
            program_set.routines.items = C.cast(self._routine_ptrs, C.POINTER(C.POINTER(C.c_uint8)))
        program_set.routines.count = len(self.routines)

    def subset(self, indices):
        return PackedPrograms([self.asts[i] for i in indices], self.routines)


# --------------------------------------------------------------------------- RNG ----

_MASK = (1 << 64) - 1


def splitmix64(state):
    """One step of SplitMix64 (the generator the reference's stress tests use,
    projects/secant/tests/support/ast_stress.c:125-132); returns (new_state, output)."""
    state = (state + 0x9E3779B97F4A7C15) & _MASK
    z = state
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    return state, z ^ (z >> 31)


def _stream(seed, index, count):
    """`count` 64-bit outputs of SplitMix64 keyed by (seed, index), vectorised."""
    key = (seed * 0x9E3779B97F4A7C15 + index * 0xD1B54A32D192ED03 + 0x2545F4914F6CDD1D) & _MASK
    steps = (np.arange(1, count + 1, dtype=np.uint64) * np.uint64(0x9E3779B97F4A7C15)) + np.uint64(key)
    z = steps
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def uniform(seed, index, count, lo, hi):
    u = (_stream(seed, index, count) >> np.uint64(40)).astype(np.float64) / float(1 << 24)
    return (lo + (hi - lo) * u).astype(np.float32)


def normal(seed, index, count, sigma=1.0):
    n = (count + 1) // 2
    u1 = ((_stream(seed, index, n) >> np.uint64(11)).astype(np.float64) + 1.0) / float(1 << 53)
    u2 = (_stream(seed ^ 0x5BD1E995, index, n) >> np.uint64(11)).astype(np.float64) / float(1 << 53)
    r = np.sqrt(-2.0 * np.log(u1))
    z = np.concatenate([r * np.cos(2 * np.pi * u2), r * np.sin(2 * np.pi * u2)])[:count]
    return (sigma * z).astype(np.float32)


# ---------------------------------------------------------------- random programs ----

# operation set of the benchmark configurations: (token bytes, arity)
_OPS = [
    (op("ADD"), 2), (op("SUB"), 2), (op("MUL"), 2), (routine(0), 2),  # + - * pdiv
    (op("SIN"), 1), (op("COS"), 1), (op("EXP"), 1), (routine(1), 1),  # sin cos exp plog
]


def random_program(rng_words, max_tokens, num_columns, num_constants=0, literal_range=1.0, toggle_bits=0, ops=None):
    """One random postfix program of at most `max_tokens` tokens (RET not counted).

    Tokens are drawn left to right while keeping the stack closable within the budget:
    with `room` tokens left and `depth` values on the stack, depth - 1 binary operations
    must still fit.  Leaves are columns, bank constants (when num_constants > 0) or f32
    literals in [-literal_range, literal_range]; with toggle_bits > 0 a third of the leaves
    are two-way toggles over two direct leaves (three tokens)."""
    words = iter(rng_words)

    def nxt(n):
        return int(next(words) % n)

    def leaf_bytes():
        k = nxt(4)
        if k == 0:
            return lit((nxt(2001) - 1000) / 1000.0 * literal_range)
        if num_constants and k == 1:
            return bank(nxt(num_constants))
        return col(nxt(num_columns))

    binary = [o[0] for o in (ops or _OPS) if o[1] == 2]
    unary = [o[0] for o in (ops or _OPS) if o[1] == 1]
    target = 1 + nxt(max_tokens)
    out = []
    depth = used = 0
    while True:
        if used >= target and depth >= 1:
            if depth == 1:
                break
            action = 2
        else:
            room = max_tokens - used
            actions = []
            if depth == 0 or room - 1 >= depth:
                actions.append(0)
            if unary and depth >= 1 and room - 1 >= depth - 1:
                actions.append(1)
            if depth >= 2:
                actions.append(2)
            action = actions[nxt(len(actions))]
        if action == 0:
            if toggle_bits and max_tokens - used - 3 >= depth and nxt(3) == 0:
                out.append(leaf_bytes() + leaf_bytes() + tog2(nxt(toggle_bits)))
                used += 3
            else:
                out.append(leaf_bytes())
                used += 1
            depth += 1
        elif action == 1:
            out.append(unary[nxt(len(unary))])
            used += 1
        else:
            out.append(binary[nxt(len(binary))])
            used += 1
            depth -= 1
    return b"".join(out) + RET


ARITHMETIC_OPS = [(op("ADD"), 2), (op("SUB"), 2), (op("MUL"), 2), (op("NEG"), 1), (op("ABS"), 1)]


def random_population(seed, count, max_tokens, num_columns, num_constants=0, literal_range=1.0, toggle_bits=0,
                      first_index=0, ops=None):
    """`count` seeded programs; program i depends only on (seed, first_index + i)."""
    asts = []
    for i in range(count):
        words = _stream(seed, first_index + i, 4 * max_tokens + 16).tolist()
        asts.append(random_program(words, max_tokens, num_columns, num_constants, literal_range, toggle_bits, ops))
    return PackedPrograms(asts, PROTECTED_ROUTINES)


def gated_population(seed, count, max_tokens, num_columns, num_constants, toggle_bits):
    """Programs whose sub-expressions are gated by toggles: each gate multiplies a random
    sub-program by TOGGLE2(1.0, 0.0), the direct-leaf encoding of "this subtree is on or
    off" (toggles may only select among direct leaves, projects/secant/docs/toggles.md:45-52)."""
    asts = []
    for i in range(count):
        words = _stream(seed, i, 8 * max_tokens + 64).tolist()
        it = iter(words)
        gates = 1 + int(next(it) % 3)
        budget = max(3, (max_tokens - 4 * gates - (gates - 1)) // gates)
        parts = []
        for g in range(gates):
            sub_words = [next(it) for _ in range(4 * budget + 16)]
            body = random_program(sub_words, budget, num_columns, num_constants, 1.0, toggle_bits)[:-1]
            bit = int(next(it) % toggle_bits)
            parts.append(body + lit(1.0) + lit(0.0) + tog2(bit) + op("MUL"))
        prog = parts[0]
        for p in parts[1:]:
            prog += p + op("ADD")
        asts.append(prog + RET)
    return PackedPrograms(asts, PROTECTED_ROUTINES)


def count_ops(packed):
    """Arithmetic nodes per program after routine inlining (work accounting: each
    add/sub/mul/div/sin/... counts one, pdiv four, plog three; leaves and toggles zero)."""
    routine_ops = []
    for r in packed.routines:
        routine_ops.append(_count_tokens(r, routine_ops))
    return np.array([_count_tokens(a, routine_ops) for a in packed.asts], dtype=np.int64)


_WIDTH = {OP["AFFINE"]: 10, OP["LIT"]: 5, OP["TOG4"]: 3, OP["ROUTINE"]: 2, OP["ARG"]: 2, OP["BANK"]: 2, OP["TOG2"]: 2,
          OP["COL"]: 2}


def _count_tokens(code, routine_ops):
    at = 0
    n = 0
    while True:
        o = code[at]
        if o == OP["RET"]:
            return n
        if o == OP["ROUTINE"]:
            n += routine_ops[code[at + 1]]
        elif o not in _WIDTH:
            n += 1
        at += _WIDTH.get(o, 1)
