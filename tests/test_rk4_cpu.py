"""The CPU restatement of the RK4 rollout scorer on closed forms (no GPU).

The reference pins its scoring kernel with a constant-slope system whose error grows
linearly in time (projects/odezza/tests/o_scoring_cuda_test.c:56-80: expected MSE =
mean(elapsed^2) * slope_error^2) and with an invalid-data matrix that must yield FLT_MAX
(:160-186).  The same cases, in this repository's uniform trajectory layout."""
import numpy as np

import support as S
from secant_b200 import programs as P

FLT_MAX = np.float32(3.402823466e38)


def slope_case():
    # two trajectories observed at t = 0, 0.25, 1.0 on the line x(t) = x0 + t; system i has slope 1 + i
    times = np.array([0.0, 0.25, 1.0], dtype=np.float32)
    reference = np.array([[1.0, 1.25, 2.0, 2.0, 2.25, 3.0]], dtype=np.float32)
    systems = P.PackedPrograms([P.bank(0) + P.RET for _ in range(4)])
    constants = np.array([[1.0], [2.0], [3.0], [4.0]], dtype=np.float32)
    return systems, reference, times, constants


def test_constant_slope_closed_form():
    systems, reference, times, constants = slope_case()
    code, scores = S.oracle_rk4(systems, 1, reference, 2, times, constants, substeps=4)
    assert code == 0
    want = np.array([0.53125 * e * e for e in range(4)], dtype=np.float32)   # mean(0.25^2, 1^2) = 0.53125
    assert np.allclose(scores, want, atol=2e-6)


def test_invalid_data_policy_is_flt_max_never_nan():
    systems, reference, times, constants = slope_case()
    bad = reference.copy(); bad[0, 3] = np.nan                         # non-finite initial state
    _, scores = S.oracle_rk4(systems, 1, bad, 2, times, constants)
    assert np.all(scores == FLT_MAX)
    _, scores = S.oracle_rk4(systems, 1, reference, 2, np.array([0.0, 0.5, 0.25], dtype=np.float32), constants)
    assert np.all(scores == FLT_MAX)                                    # times must increase
    blow = P.PackedPrograms([P.col(0) + P.col(0) + P.op("MUL") + P.lit(1e30) + P.op("MUL") + P.RET])
    _, scores = S.oracle_rk4(blow, 1, reference, 2, times, None)
    assert scores[0] == FLT_MAX                                          # overflow during integration


def test_exponential_decay_converges_to_analytic_solution():
    # x' = -x from x0 = 1: RK4 with h = 0.01 matches exp(-t) far below float32 resolution
    times = np.arange(0, 101, dtype=np.float32) * np.float32(0.01)
    reference = np.exp(-times.astype(np.float64)).astype(np.float32)[None, :]
    decay = P.PackedPrograms([P.col(0) + P.op("NEG") + P.RET])
    code, scores = S.oracle_rk4(decay, 1, reference, 1, times, None)
    assert code == 0 and scores[0] < 1e-13


def reference_launch_case():
    """The reference engine's own scoring test data (projects/odezza/tests/o_scoring_cuda_test.c:97-101,
    :156-160): two ragged trajectories {0,3,5} on the line x(t) = x0 + t with irregular times, two
    steps per observation, system i with slope 1 + i; expected MSE 0.4375 * i^2."""
    offsets = np.array([0, 3, 5], dtype=np.uint32)
    times = np.array([0.0, 0.25, 1.0, 0.0, 0.5], dtype=np.float32)
    reference = np.array([[1.0, 1.25, 2.0, 2.0, 2.5]], dtype=np.float32)
    systems = P.PackedPrograms([P.bank(0) + P.RET for _ in range(4)])
    constants = np.array([[1.0], [2.0], [3.0], [4.0]], dtype=np.float32)
    return systems, reference, times, offsets, constants


def invalid_launch_matrix():
    """(offsets, times, reference) variations the reference test expects to score FLT_MAX
    (projects/odezza/tests/o_scoring_cuda_test.c:162-186)."""
    _, reference, times, offsets, _ = reference_launch_case()
    nan, inf = np.float32(np.nan), np.float32(np.inf)
    cases = []
    def vary(o=None, t=None, r=None):
        oo, tt, rr = offsets.copy(), times.copy(), reference.copy()
        for i, v in (o or {}).items(): oo[i] = v
        for i, v in (t or {}).items(): tt[i] = v
        for i, v in (r or {}).items(): rr[0, i] = v
        cases.append((oo, tt, rr))
    vary(o={0: 1})                      # does not start at zero
    vary(o={1: 0})                      # empty first trajectory
    vary(o={2: 6})                      # runs past the data
    vary(o={2: 4})                      # does not cover the data
    vary(t={1: 0.0})                    # time does not increase
    vary(t={1: nan})
    vary(r={1: inf})                    # infinite observation
    vary(o={1: 1}, t={3: 1.25, 4: 1.5}, r={0: nan})     # singleton trajectory with a missing initial value
    vary(o={1: 1}, t={0: nan, 3: 1.25, 4: 1.5})         # singleton trajectory with a non-finite time
    vary(t={1: np.nextafter(np.float32(0), np.float32(1))})  # step underflows to zero
    return cases


def test_reference_launch_layout_closed_form_and_invalid_matrix():
    systems, reference, times, offsets, constants = reference_launch_case()
    code, scores = S.oracle_rk4(systems, 1, reference, 2, times, constants, substeps=2, offsets=offsets)
    assert code == 0
    assert np.allclose(scores, [0.4375 * e * e for e in range(4)], atol=2e-6)
    for oo, tt, rr in invalid_launch_matrix():
        code, scores = S.oracle_rk4(systems, 1, rr, 2, tt, constants, substeps=2, offsets=oo)
        assert code == 0 and np.all(scores == FLT_MAX), (oo, tt, rr)


def test_missing_observations_are_skipped_and_counted_out():
    systems, reference, times, offsets, constants = reference_launch_case()
    holes = reference.copy(); holes[0, 2] = np.nan                    # the t = 1.0 observation is missing
    _, scores = S.oracle_rk4(systems, 1, holes, 2, times, constants, substeps=2, offsets=offsets)
    assert np.all(scores == FLT_MAX)                                   # not allowed unless asked for
    _, scores = S.oracle_rk4(systems, 1, holes, 2, times, constants, substeps=2, offsets=offsets, allow_missing=True)
    want = [(0.25 ** 2 + 0.5 ** 2) / 2 * e * e for e in range(4)]       # two residuals left
    assert np.allclose(scores, want, atol=2e-6)
    holes[0, 3] = np.nan                                               # an initial value may never be missing
    _, scores = S.oracle_rk4(systems, 1, holes, 2, times, constants, substeps=2, offsets=offsets, allow_missing=True)
    assert np.all(scores == FLT_MAX)


# ---- second pin: the reference's own host-side scorer on its fixed shape -----------------------

_TO_ENGINE = {  # Secant opcode -> the reference engine's bytecode (projects/odezza/research/ast_tools/o_ast_tools.h:43-68)
    "RET": 0x80, "COL": 0x81, "BANK": 0x82, "LIT": 0x83, "TOG2": 0x84, "TOG4": 0x85, "ADD": 0x90, "SUB": 0x91, "MUL": 0x92,
    "DIV": 0x93, "NEG": 0x94, "SQRT": 0x95, "RCP": 0x96, "ABS": 0x97, "MIN": 0x98, "MAX": 0x99, "FMA": 0x9A, "SIN": 0x9B,
    "COS": 0x9C, "EX2": 0x9D, "LG2": 0x9E, "RSQRT": 0x9F, "TANH": 0xA0, "EXP": 0xA1, "LOG": 0xA2}


def to_engine_bytecode(code):
    """The same postfix program in the reference engine's token values (operand bytes unchanged)."""
    names = {v: k for k, v in P.OP.items()}
    out, at = bytearray(), 0
    while True:
        name = names[code[at]]
        width = P._WIDTH.get(code[at], 1)
        out.append(_TO_ENGINE[name])
        out += code[at + 1:at + width]
        at += width
        if name == "RET":
            return bytes(out)


def engine_reference_scorer():
    import ctypes as C
    import os
    path = os.path.join(S.ROOT, "oracle", "_ref", "libodezza_cpu_ref.so")
    if not os.path.exists(path):
        return None
    lib = C.CDLL(path)
    lib.so_ref_o_cpu_score.restype = C.c_float
    return lib


def test_oracle_against_the_reference_host_scorer_on_its_fixed_shape():
    """so_rk4_score against o_cpu_score (projects/odezza/research/ast_tools/o_ast_engine_benchmark.c:368-434,
    over o_ast_cpu_evaluate, o_ast_cpu.c:111-209), compiled from the reference tree by `make -C oracle
    odezza`: 4 states, 3 trajectories, 8 observations 0.05 apart, 5 toggle bits, 4 constants.  Seeded
    right-hand sides over every operation (both sides call the same libm), toggles included, 1 and 4
    steps per observation: the scores must agree bit for bit."""
    import ctypes as C
    import pytest
    lib = engine_reference_scorer()
    if lib is None:
        pytest.skip("oracle/_ref/libodezza_cpu_ref.so is built only where the reference checkout is present")
    S_, TR, OBS, K, BITS = 4, 3, 8, 4, 5
    ops = [(P.op(n), 2) for n in ("ADD", "SUB", "MUL", "DIV", "MIN", "MAX")] + \
          [(P.op(n), 1) for n in ("NEG", "ABS", "SQRT", "SIN", "COS", "TANH", "EXP", "LOG", "RCP")]
    rng = np.random.Generator(np.random.Philox(key=808))
    checked = finite = 0
    S.oracle().so_rk4_set_fixed_interval(C.c_float(0.05))
    try:
        for trial in range(60):
            pop = P.random_population(900 + trial, S_, 14, S_, K, 1.0, toggle_bits=BITS, ops=ops)
            pop = P.PackedPrograms(pop.asts)                     # no routines in the engine's format
            constants = rng.standard_normal((1, K)).astype(np.float32)
            initial = rng.uniform(-1, 1, size=(S_, TR)).astype(np.float32)
            targets = rng.uniform(-1, 1, size=(S_, TR, OBS)).astype(np.float32)
            flat = np.concatenate([initial.reshape(-1), targets.reshape(-1)]).astype(np.float32)   # the scorer's own layout
            mine = np.concatenate([initial[:, :, None], targets], axis=2).reshape(S_, TR * (OBS + 1))
            times = (np.arange(OBS + 1) * 0.05).astype(np.float32)
            engine = [to_engine_bytecode(a) for a in pop.asts]
            bufs = [(C.c_uint8 * len(e)).from_buffer_copy(e) for e in engine]
            ptrs = (C.POINTER(C.c_uint8) * S_)(*[C.cast(b, C.POINTER(C.c_uint8)) for b in bufs])
            sizes = (C.c_size_t * S_)(*[len(e) for e in engine])
            for perm in (0, 21, 31):
                for steps in (1, 4):
                    want = np.float32(lib.so_ref_o_cpu_score(ptrs, sizes, C.c_size_t(S_), S.fptr(constants), C.c_uint32(perm),
                                                             S.fptr(flat), C.c_uint32(steps)))
                    code, got = S.oracle_rk4(pop, S_, mine, TR, times, constants, substeps=steps, toggle_bits=BITS, permutation=perm)
                    assert code == 0
                    assert got[0].view(np.uint32) == want.view(np.uint32), (trial, perm, steps, float(got[0]), float(want))
                    checked += 1
                    finite += bool(want < FLT_MAX)
    finally:
        S.oracle().so_rk4_set_fixed_interval(C.c_float(0.0))
    assert checked == 360 and finite > 100       # both valid scores and the FLT_MAX policy were exercised


def _host_only_run(packed, num_states, systems, points=5, trajectories=2):
    """A request whose device addresses are placeholders: validation and the program scan come
    before anything is read, allocated or launched, so nothing may touch them.  The request
    points into `packed`, which the caller keeps alive."""
    import ctypes as C
    from secant_b200 import abi
    run = abi.Rk4Run()
    run.struct_size, run.version = C.sizeof(run), abi.RUN_VERSION
    packed.fill(run.programs)
    run.num_systems, run.num_states, run.num_constants, run.num_banks = systems, num_states, 0, 1
    total = points * trajectories
    run.reference.address, run.reference.num_elements, run.reference.leading_dimension = 0x1000, num_states * total, total
    run.num_trajectories, run.points_per_trajectory, run.times, run.steps_per_observation = trajectories, points, 0x2000, 1
    run.output.address, run.output.num_elements, run.output.leading_dimension = 0x3000, systems, 1
    return run


def test_the_first_malformed_program_in_order_decides_the_result():
    """Programs are scanned by several threads in pieces of 128 systems; whichever thread finds an
    error first, the call answers with the error of the first malformed program in program order,
    before any device is asked for (the reference validates every program before it launches,
    projects/odezza/core/o_scoring_pipeline.c:1541-1594)."""
    import ctypes as C
    from secant_b200 import abi, programs as P
    lib = abi.load()
    good = P.col(0) + P.lit(0.5) + P.op("MUL") + P.RET
    bad_column = P.col(7) + P.RET                                                # one state only
    bad_opcode = P.col(0) + bytes([0x9b]) + P.RET                                # an integer addition: not evaluable
    alone = []
    for bad in (bad_column, bad_opcode):
        one = P.PackedPrograms([bad])
        single = _host_only_run(one, 1, 1)
        alone.append(lib.secant_b200_rk4_score(C.byref(single)))
    assert alone[0] != alone[1] and abi.SUCCESS not in alone and abi.ERROR_DRIVER_FAILED not in alone
    systems = 3000                                                               # 24 pieces
    for where_column, where_opcode in ((40, 2900), (2900, 40), (700, 1400), (1400, 700), (127, 128), (128, 127), (2943, 2944), (2944, 2943)):
        asts = [good] * systems
        asts[where_column], asts[where_opcode] = bad_column, bad_opcode
        packed = P.PackedPrograms(asts)
        run = _host_only_run(packed, 1, systems)
        code = lib.secant_b200_rk4_score(C.byref(run))
        assert code == (alone[0] if where_column < where_opcode else alone[1]), (where_column, where_opcode, code)
