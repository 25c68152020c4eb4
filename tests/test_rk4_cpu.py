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
