"""Pins the CPU oracle (oracle/secant_oracle.c) on vectors produced by the reference's own
host evaluator (tests/golden/reference_vectors.npz, made by tests/golden/make_golden.py) and
on the closed forms of the reference's fixtures.  Integer-exact: every float must match the
reference bit for bit, because both sides use the same libm and the same operation order."""
import os

import numpy as np
import pytest

import support as S
from secant_b200 import programs as P

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_vectors.npz"))


def packed(prefix):
    def split(blob, off):
        blob = bytes(blob.tobytes())
        off = [int(o) for o in off] + [len(blob)]
        return [blob[off[i]:off[i + 1]] for i in range(len(off) - 1)]
    return P.PackedPrograms(split(G[prefix + "_ast_blob"], G[prefix + "_ast_off"]),
                            split(G[prefix + "_routine_blob"], G[prefix + "_routine_off"]))


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def toggle_expected(ast, p, x, c):
    """Closed forms of the seven fixture programs (projects/secant/tests/toggle_fixture.h:57-78)."""
    if ast == 0:
        return (x[1] if p & 1 else x[0]) * c[0]
    if ast == 1:
        return (c[1] if p & 2 else x[2]) + (c[0] if p & 1 else x[0])
    if ast == 2:
        return [x[0], c[0], x[2], c[1]][(p & 1) | ((p >> 1) & 2)]
    if ast == 3:
        return (c[1] if p & 4 else c[0]) - (c[0] if p & 4 else c[1])
    if ast == 4:
        return (c[0] if p & 1 else x[0]) * (c[1] if p & 2 else x[1]) + (c[0] if p & 4 else x[2])
    if ast == 5:
        return c[1] if p & 2 else np.float32(1.0)
    return [c[0], c[1], x[0], x[1]][((p >> 2) & 1) | ((p & 1) << 1)] + c[0]


def test_fixture_toggle_sse_bit_exact_and_padding():
    fx = packed("fixture")
    x, y, banks = G["fixture_x"], G["fixture_y"], G["fixture_banks"]
    for pass_idx in range(2):
        b = banks if pass_idx == 0 else (banks + np.float32(0.137)).astype(np.float32)
        out = np.full((7, 2, 109), -123.0, dtype=np.float32)
        code, got, _ = S.oracle_toggle_sse(fx, x, y, b, 2, 3, out=out, out_ld=109)
        assert code == 0
        want = G[f"fixture_sse_pass{pass_idx}"]
        assert np.array_equal(bits(got[:, :, :104]), bits(want[:, :, :104]))
        assert np.all(got[:, :, 104:] == -123.0)  # padding between score vectors is preserved
        # and the closed forms, accumulated the way the reference test does it
        for a in range(7):
            for t in range(2):
                for bank in range(13):
                    for p in range(8):
                        acc = np.float32(0)
                        for row in range(17):
                            e = np.float32(toggle_expected(a, p, x[:, row], b[bank])) - y[t, row]
                            acc = np.float32(acc + np.float32(e * e))
                        assert abs(got[a, t, bank * 8 + p] - acc) < 1e-5 * (1 + abs(acc))


def test_fixture_error_codes():
    fx = packed("fixture")
    x, y, banks = G["fixture_x"], G["fixture_y"], G["fixture_banks"]
    out = np.full((7, 2, 52), 1234.0, dtype=np.float32)
    code, got, _ = S.oracle_toggle_sse(fx, x, y, banks, 2, 2, out=out)
    assert code == int(G["fixture_bits2_code"]) == 9  # BAD_PROGRAM before anything is cleared
    assert np.all(got == 1234.0)
    bad = packed("bad")
    for i, want in enumerate(G["bad_codes"]):
        code, _, _ = S.oracle_toggle_sse(bad.subset([i]), x, y, banks, 2, 3)
        assert code == int(want) == 9
    # short bank buffer, stride below the constant count, output aliasing the input
    import ctypes as C
    short = banks.reshape(-1)[:37].copy()
    out = np.zeros((7, 2, 104), dtype=np.float32)
    lib = S.oracle()
    args = S.blob_args(fx)
    def call(bank_arr, nelem, stride, outp):
        return lib.so_toggle_sse(*args, C.c_size_t(3), C.c_size_t(2), S.fptr(x), C.c_size_t(x.size), C.c_size_t(17), S.fptr(y),
                                 C.c_size_t(y.size), C.c_size_t(17), S.fptr(bank_arr), C.c_size_t(nelem), C.c_size_t(stride),
                                 C.c_size_t(0), C.c_size_t(17), C.c_size_t(2), C.c_size_t(13), C.c_uint32(3), outp,
                                 C.c_size_t(out.size), C.c_size_t(104), None)
    assert call(short, 37, 3, S.fptr(out)) == 3   # INSUFFICIENT_BUFFER
    assert call(banks, 38, 1, S.fptr(out)) == 1   # INVALID_VALUE: stride < constants
    assert call(banks, 38, 3, S.fptr(x)) == 1     # INVALID_VALUE: output overlaps input


def test_affine_leaf_exact_values():
    code, got, _ = S.oracle_toggle_sse(packed("affine"), G["affine_x"], G["affine_y"], G["affine_banks"], 1, 1)
    assert code == 0
    assert got.reshape(-1).tolist() == [6.25, 25.0, 16.0, 25.0] == G["affine_sse"].reshape(-1).tolist()


def test_static_programs_with_routine():
    st = packed("static")
    code, mat = S.oracle_materialize(st, G["static_x"])
    assert code == 0 and np.array_equal(bits(mat), bits(G["static_materialize"]))
    code, sse, _ = S.oracle_sse(st, G["static_x"], G["static_y"])
    assert code == 0 and np.array_equal(bits(sse), bits(G["static_sse"]))
    x = G["static_x"]
    assert np.allclose(mat[0], x[0] + x[1], rtol=1e-6)
    assert np.allclose(mat[1], np.sin(x[2]), rtol=1e-6)
    assert np.allclose(mat[2], x[0] * x[1] / (x[1] * x[1] + 1e-6), rtol=1e-5)


def test_random_populations_bit_exact():
    code, got, _ = S.oracle_toggle_sse(packed("random"), G["random_x"], G["random_y"], G["random_banks"], 4, 3)
    assert code == 0
    assert np.array_equal(bits(got), bits(G["random_sse"]))
    c1 = packed("c1")
    code, mat = S.oracle_materialize(c1, G["c1_x"])
    assert code == 0 and np.array_equal(bits(mat), bits(G["c1_materialize"]))
    code, sse, _ = S.oracle_sse(c1, G["c1_x"], G["c1_y"])
    assert code == 0 and np.array_equal(bits(sse), bits(G["c1_sse"]))


def test_against_reference_library_when_present():
    ref = S.reference_lib()
    if ref is None:
        pytest.skip("reference evaluator not built on this machine")
    pop = P.random_population(77, 200, 32, 8, 16, 3.0, toggle_bits=3)
    x = np.stack([P.uniform(11, c, 41, -3, 3) for c in range(8)])
    y = np.stack([P.normal(12, 0, 41)])
    banks = np.stack([P.normal(13, b, 16) for b in range(5)])
    code, got, _ = S.oracle_toggle_sse(pop, x, y, banks, 16, 3)
    rcode, want = S.reference_toggle_sse(ref, pop, x, y, banks, 16, 3)
    assert code == rcode == 0
    assert np.array_equal(bits(got), bits(want))


def test_best_config_and_topk_rules():
    import ctypes as C
    lib = S.oracle()
    scores = np.array([[3.0, np.nan, 1.0, 1.0, -1.0, np.inf], [np.nan, np.inf, -2.0, np.nan, np.nan, np.nan]], dtype=np.float32)
    best = np.zeros(2, dtype=np.float32)
    arg = np.zeros(2, dtype=np.uint64)
    valid = np.zeros(2, dtype=np.uint64)
    lib.so_best_config(S.fptr(scores), C.c_size_t(2), C.c_size_t(6), C.c_size_t(6), S.fptr(best),
                       arg.ctypes.data_as(S.U64P), valid.ctypes.data_as(S.U64P))
    assert best[0] == 1.0 and arg[0] == 2 and valid[0] == 3      # ties go to the lowest index
    assert np.isinf(best[1]) and arg[1] == 2**64 - 1 and valid[1] == 0
    flat = np.array([5.0, 1.0, np.nan, 1.0, 0.5, -3.0, np.inf, 2.0], dtype=np.float32)
    idx = np.zeros(4, dtype=np.uint64)
    lib.so_topk.restype = C.c_size_t
    n = lib.so_topk(S.fptr(flat), C.c_size_t(8), C.c_size_t(4), idx.ctypes.data_as(S.U64P))
    assert n == 4 and idx.tolist() == [4, 1, 3, 7]


def test_grouped_topk_rule_on_a_hand_checked_grid():
    """Valid = 0 <= score < FLT_MAX, -0 orders as +0 and keeps its bits, ties go to the lower flat
    index, unfilled ranks are {FLT_MAX, UINT64_MAX} (projects/odezza/core/o_score_reduce.cu:36-62)."""
    import ctypes as C
    grid = np.array([[3, 1, -0.0, 1], [np.nan, -2, 5, np.inf]], dtype=np.float32)
    mse = np.zeros((2, 3), np.float32); idx = np.zeros((2, 3), np.uint64); counts = np.zeros((2, 3), np.uint64)
    assert S.oracle().so_grouped_topk(S.fptr(grid), C.c_size_t(2), C.c_size_t(4), C.c_uint32(0), C.c_uint32(0), C.c_size_t(3),
                                      S.fptr(mse), idx.ctypes.data_as(S.U64P), counts.ctypes.data_as(S.U64P)) == 0
    assert idx.tolist() == [[2, 1, 3], [6, 2 ** 64 - 1, 2 ** 64 - 1]]
    assert np.signbit(mse[0, 0]) and mse[0].tolist() == [0.0, 1.0, 1.0] and mse[1, 0] == 5 and mse[1, 1] == np.float32(3.402823466e38)
    assert counts.tolist() == [[4, 0, 0], [1, 3, 1]]
    # per (system, permutation): one toggle bit, two banks -> groups (s0,p0) (s0,p1) (s1,p0) (s1,p1), each over 2 banks
    mse = np.zeros((4, 1), np.float32); idx = np.zeros((4, 1), np.uint64); counts = np.zeros((4, 3), np.uint64)
    assert S.oracle().so_grouped_topk(S.fptr(grid), C.c_size_t(2), C.c_size_t(2), C.c_uint32(1), C.c_uint32(1), C.c_size_t(1),
                                      S.fptr(mse), idx.ctypes.data_as(S.U64P), counts.ctypes.data_as(S.U64P)) == 0
    assert idx[:, 0].tolist() == [2, 1, 6, 2 ** 64 - 1] and counts[:, 0].tolist() == [2, 2, 1, 0]


def test_gram_statistics_restatement_matches_the_reference_library():
    """so_gram_stats against the reference host evaluator's Gram-statistics run (projects/secant/
    s_cpu.c:724-848) bit for bit: cohorts of 5 with a ragged last one, two targets, routines."""
    ref = S.reference_lib()
    if ref is None:
        pytest.skip("oracle/_ref/libsecant_ref.so is built only where the reference checkout exists")
    pop = P.random_population(61, 23, 15, 4)
    x = np.stack([P.uniform(62, c, 301, -1, 1) for c in range(4)])
    y = np.stack([P.normal(63, t, 301) for t in range(2)])
    code, want = S.reference_gram_stats(ref, pop, x, y, 5)
    assert code == 0
    code, got, _ = S.oracle_gram_stats(pop, x, y, 5)
    assert code == 0
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert np.all(got[-1].reshape(-1)[3:5] == 0)                       # the last cohort holds 3 programs: unused sums stay zero
