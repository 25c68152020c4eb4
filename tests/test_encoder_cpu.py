"""Host logic without a GPU: the production encoder (via the test hooks) must produce
records that evaluate bit-identically to the CPU oracle, and must reject malformed programs
with the reference's result codes (projects/secant/tests/cpu_test.c:219-283,
tests/toggle_test.c:96-134)."""
import ctypes as C

import numpy as np
import pytest

import support as S
from secant_b200 import abi, programs as P


def encode(packed, columns, constants, banks_allowed=True, toggle_bits=0, preflight=True, hoist=False, flat=False,
           max_hoisted=0, rollout=False):
    """hoist: bank-only and row-only sub-expressions move to the bank part and the row prelude;
    flat: one-part records with direct constant addressing;
    rollout: the rollout kernel's form (columns are the integrator's state slots, bank-only
    sub-expressions in the bank part, nothing else hoisted)."""
    handle = C.c_void_p()
    flags = int(preflight) | (2 if hoist else 0) | (4 if flat else 0) | (16 if rollout else 0) | (max_hoisted << 8)
    code = S.hooks().sbt_encode(*S.blob_args(packed), C.c_size_t(columns), C.c_size_t(constants), int(banks_allowed),
                                toggle_bits, flags, C.byref(handle))
    return code, handle


def info(handle, index):
    """n_insn, n_slots, n_ops, n_patch, n_affine, n_lits, pre_off, main_off, n_hoisted, n_cst, n_btmp, flags, mid_off"""
    out = (C.c_uint32 * 13)()
    S.hooks().sbt_info(handle, C.c_size_t(index), out)
    return list(out)


def host_eval(handle, index, x, bank, perm, row):
    value = C.c_float()
    code = S.hooks().sbt_eval(handle, C.c_size_t(index), S.fptr(x), C.c_size_t(x.shape[1]), C.c_size_t(row),
                              S.fptr(bank) if bank is not None else None, C.c_uint64(perm), C.byref(value))
    assert code == 0
    return np.float32(value.value)


def same(a, b):
    a, b = np.float32(a), np.float32(b)
    return (np.isnan(a) and np.isnan(b)) or a.view(np.uint32) == b.view(np.uint32)


MODES = [dict(), dict(hoist=True), dict(hoist=True, max_hoisted=1), dict(flat=True), dict(rollout=True)]


@pytest.mark.parametrize("mode", MODES, ids=["split", "hoisted", "hoisted-one-row-value", "flat", "rollout"])
@pytest.mark.parametrize("seed,max_tokens,bits", [(3, 15, 0), (4, 32, 3), (5, 48, 8)])
def test_records_evaluate_like_the_oracle(seed, max_tokens, bits, mode):
    pop = P.random_population(seed, 150, max_tokens, 6, 8, 2.0, toggle_bits=bits)
    n = 29
    x = np.stack([P.uniform(seed, c, n, -2, 2) for c in range(6)])
    banks = np.stack([P.normal(seed + 1, b, 8) for b in range(3)])
    code, handle = encode(pop, 6, 8, True, bits, **mode)
    assert code == 0
    configs = 3 << bits
    for cfg in sorted({0, 1, configs // 2, configs - 1}):
        _, want = S.oracle_toggle_materialize(pop, x, banks, 8, bits, cfg)
        for a in range(len(pop.asts)):
            for row in (0, n // 2, n - 1):
                got = host_eval(handle, a, x, banks[cfg >> bits], cfg & ((1 << bits) - 1), row)
                assert same(got, want[a, row]), (a, cfg, row, pop.asts[a].hex())
    S.hooks().sbt_free(handle)


def test_gated_programs_and_fixture_forms():
    pop = P.gated_population(9, 60, 48, 6, 8, 8)
    x = np.stack([P.normal(9, c, 11) for c in range(6)])
    banks = np.stack([P.normal(10, b, 8) for b in range(4)])
    code, handle = encode(pop, 6, 8, True, 8)
    assert code == 0
    for cfg in (0, 77, 255, 256 + 13, 1023):
        _, want = S.oracle_toggle_materialize(pop, x, banks, 8, 8, cfg)
        for a in range(len(pop.asts)):
            assert same(host_eval(handle, a, x, banks[cfg >> 8], cfg & 255, 5), want[a, 5])


def hand(*parts):
    return b"".join(parts) + P.RET


def test_fma_routines_and_shared_arguments():
    sq = P.arg(0) + P.arg(0) + P.op("MUL") + P.RET                       # x*x, argument used twice
    mix = P.arg(0) + P.arg(1) + P.arg(0) + P.op("FMA") + P.arg(1) + P.op("SUB") + P.RET
    progs = [
        hand(P.col(0), P.col(1), P.op("ADD"), P.col(2), P.op("SIN"), P.op("MUL"), P.routine(0)),
        hand(P.col(0), P.col(1), P.col(2), P.op("FMA")),
        hand(P.col(0), P.op("EXP"), P.lit(2.0), P.col(1), P.op("COS"), P.op("FMA")),
        hand(P.col(0), P.col(1), P.op("MUL"), P.col(1), P.col(2), P.op("SUB"), P.routine(1)),
        hand(P.col(0), P.col(1), P.op("MUL"), P.col(1), P.col(2), P.op("SUB"), P.col(0), P.col(2), P.op("DIV"), P.op("FMA")),
        hand(P.bank(0), P.col(1), P.tog2(0), P.lit(0.5), P.bank(1), P.tog2(1), P.col(2), P.op("FMA")),
        hand(P.col(0), P.op("SQRT"), P.op("RSQRT"), P.op("RCP"), P.op("ABS"), P.op("NEG"), P.op("TANH"), P.op("EX2"), P.op("LG2")),
        hand(P.col(0), P.col(1), P.op("MIN"), P.col(2), P.op("MAX"), P.lit(3.0), P.op("DIV"), P.lit(1.5), P.op("SUB")),
        hand(P.lit(2.0), P.col(0), P.op("SUB"), P.lit(4.0), P.col(1), P.op("DIV"), P.op("MUL")),
        hand(P.affine(1, 2.0, -0.5), P.col(0), P.op("MUL"), P.affine(1, 2.0, -0.5), P.op("ADD")),
        hand(P.col(0), P.col(1), P.op("ADD"), P.routine(0), P.col(2), P.routine(1)),
    ]
    pop = P.PackedPrograms(progs, [sq, mix])
    x = np.stack([P.uniform(1, c, 7, 0.1, 2) for c in range(3)])
    banks = np.stack([P.normal(2, b, 2) for b in range(2)])
    for mode in MODES:
        check_hand_written(pop, progs, x, banks, mode)


def check_hand_written(pop, progs, x, banks, mode):
    code, handle = encode(pop, 3, 2, True, 2, **mode)
    assert code == 0
    for cfg in range(8):
        _, want = S.oracle_toggle_materialize(pop, x, banks, 2, 2, cfg)
        for a in range(len(progs)):
            for row in range(7):
                assert same(host_eval(handle, a, x, banks[cfg >> 2], cfg & 3, row), want[a, row]), (a, cfg, row)


def test_structural_errors_match_the_reference_codes():
    deep = b"".join(P.lit(1.0) for _ in range(129)) + P.RET
    cases = [
        (deep, abi.ERROR_STACK_OVERFLOW),
        (P.col(0) + P.op("ADD") + P.RET, abi.ERROR_STACK_UNDERFLOW),
        (P.col(0) + P.col(1) + P.RET, abi.ERROR_BAD_PROGRAM),               # two values left at RETURN
        (bytes([0x97, 1, 0, 0, 0, 0x99]), abi.ERROR_UNSUPPORTED_OP),         # s32 constant / return
        (bytes([0xB7, 0]) + P.RET, abi.ERROR_BAD_PROGRAM),                   # retired opcode
        (P.col(9) + P.RET, abi.ERROR_BAD_PROGRAM),                           # column out of range
        (P.bank(5) + P.RET, abi.ERROR_BAD_PROGRAM),
        (P.col(0) + P.col(1) + P.op("ADD") + P.bank(0) + P.tog2(0) + P.RET, abi.ERROR_BAD_PROGRAM),  # toggle over computed value
        (P.col(0) + P.col(1) + P.bank(0) + P.bank(1) + P.tog4(0, 0) + P.RET, abi.ERROR_BAD_PROGRAM),
        (P.col(0) + P.col(1) + P.tog2(3) + P.RET, abi.ERROR_BAD_PROGRAM),    # bit beyond toggle_bits
        (P.col(0) + P.routine(4) + P.RET, abi.ERROR_ROUTINE_IDX_OUT_OF_BOUNDS),
        (P.arg(0) + P.RET, abi.ERROR_ROUTINE_ARG_IDX_OUT_OF_BOUNDS),
        (P.affine(0, float("nan"), 0.0) + P.RET, abi.ERROR_BAD_PROGRAM),
        (P.col(0) + P.col(1) + P.op("ADD"), abi.ERROR_BAD_PROGRAM),          # never returns (runs into the 1024 limit / bad bytes)
    ]
    for code_bytes, want in cases:
        padded = code_bytes + bytes(12000) if code_bytes[-1:] != P.RET else code_bytes
        code, handle = encode(P.PackedPrograms([padded], [P.PDIV]), 3, 2, True, 2)
        assert code == want, (code_bytes.hex()[:40], abi.result_name(code), abi.result_name(want))
    # recursion deeper than eight frames
    rec = P.PackedPrograms([P.col(0) + P.routine(0) + P.RET], [P.arg(0) + P.routine(0) + P.RET])
    code, _ = encode(rec, 1, 0, True, 0)
    assert code == abi.ERROR_ROUTINE_DEPTH_EXCEEDED
    many = P.PackedPrograms([P.col(0) + P.RET], [P.arg(4) + P.RET])
    code, _ = encode(many, 1, 0, True, 0)
    assert code == abi.ERROR_TOO_MANY_ARGS
    # banks and toggles are only legal for the toggle shape
    code, _ = encode(P.PackedPrograms([P.bank(0) + P.RET]), 3, 2, False, 0)
    assert code == abi.ERROR_BAD_PROGRAM


def test_work_accounting_counts_inlined_routines():
    pop = P.PackedPrograms([P.col(0) + P.col(1) + P.routine(0) + P.routine(1) + P.RET], P.PROTECTED_ROUTINES)
    code, handle = encode(pop, 2, 0, True, 0)
    assert code == 0
    assert info(handle, 0)[2] == 7 == int(P.count_ops(pop)[0])  # pdiv = 4 operations, plog = 3
