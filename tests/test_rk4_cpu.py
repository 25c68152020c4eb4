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
