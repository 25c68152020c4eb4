"""GPU RK4 rollout scoring against the CPU restatement.

Right-hand sides built from exactly rounded operations integrate bit-identically on both
sides, so even a chaotic system (Lorenz, 1000 steps) must agree to summation-order precision
(1e-4 relative).  Right-hand sides with transcendental functions are compared on a short,
contracting horizon, where a 2-ulp difference of the math library cannot grow."""
import numpy as np
import pytest
import torch

import support as S
from secant_b200 import programs as P
from secant_b200.runner import rk4_score
from test_rk4_cpu import FLT_MAX, slope_case

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.tensor(np.ascontiguousarray(a), device="cuda")


def lorenz_programs():
    col, bank, op = P.col, P.bank, P.op
    return [col(1) + col(0) + op("SUB") + bank(0) + op("MUL") + P.RET,
            col(0) + bank(1) + col(2) + op("SUB") + op("MUL") + col(1) + op("SUB") + P.RET,
            col(0) + col(1) + op("MUL") + bank(2) + col(2) + op("MUL") + op("SUB") + P.RET]


def lorenz_reference(num_ics, steps, dt):
    """Reference rollout: the restated integrator itself on the true Lorenz system, float32."""
    rng = np.random.default_rng(4)
    ics = rng.uniform(-10, 10, size=(num_ics, 3)).astype(np.float32)
    ref = np.zeros((3, num_ics * (steps + 1)), dtype=np.float32)
    sigma, rho, beta = np.float32(10.0), np.float32(28.0), np.float32(8.0 / 3.0)
    h = np.float32(dt)

    def rhs(v):
        x, y, z = v
        return np.array([(y - x) * sigma, x * (rho - z) - y, x * y - beta * z], dtype=np.float32)
    for i in range(num_ics):
        v = ics[i].copy()
        ref[:, i * (steps + 1)] = v
        for k in range(1, steps + 1):
            k1 = rhs(v); k2 = rhs(v + h / 2 * k1); k3 = rhs(v + h / 2 * k2); k4 = rhs(v + h * k3)
            v = (v + h / 6 * (k1 + 2 * k2 + 2 * k3 + k4)).astype(np.float32)
            ref[:, i * (steps + 1) + k] = v
    return ref


def test_constant_slope_closed_form_and_invalid_policy(cuda):
    systems, reference, times, constants = slope_case()
    got = rk4_score(systems, 1, dev(reference), dev(times), dev(constants[:, None, :]), 1, 1, 0, 4).cpu().numpy()[:, 0]
    assert np.allclose(got, [0.53125 * e * e for e in range(4)], atol=2e-6)
    bad = reference.copy(); bad[0, 3] = np.nan
    got = rk4_score(systems, 1, dev(bad), dev(times), dev(constants[:, None, :]), 1, 1, 0, 1).cpu().numpy()
    assert np.all(got == FLT_MAX)
    blow = P.PackedPrograms([P.col(0) + P.col(0) + P.op("MUL") + P.lit(1e30) + P.op("MUL") + P.RET])
    assert rk4_score(blow, 1, dev(reference), dev(times)).cpu().numpy()[0, 0] == FLT_MAX
    # the record buffers' memory pool can be emptied between calls; the next call fills it again
    from secant_b200 import abi
    assert abi.load().secant_b200_release_cached_memory() == 0
    again = rk4_score(systems, 1, dev(reference), dev(times), dev(constants[:, None, :]), 1, 1, 0, 4).cpu().numpy()[:, 0]
    assert np.allclose(again, [0.53125 * e * e for e in range(4)], atol=2e-6)


def test_lorenz_candidates_match_oracle_over_a_chaotic_horizon(cuda):
    num_ics, steps, dt = 64, 1000, 0.01
    ref = lorenz_reference(num_ics, steps, dt)
    times = (np.arange(steps + 1, dtype=np.float32) * np.float32(dt)).astype(np.float32)
    rng = np.random.default_rng(8)
    n_sys = 24
    coeffs = np.tile(np.array([10.0, 28.0, 8.0 / 3.0], dtype=np.float32), (n_sys, 1))
    coeffs[1:] += rng.normal(0, 0.5, size=(n_sys - 1, 3)).astype(np.float32)
    coeffs[-1] = [10.0, 2000.0, -5.0]                                    # an explosive candidate
    pop = P.PackedPrograms(lorenz_programs() * n_sys)
    code, want, want64 = S.oracle_rk4(pop, 3, ref, num_ics, times, coeffs, want64=True)
    assert code == 0
    got = rk4_score(pop, 3, dev(ref), dev(times), dev(coeffs[:, None, :]), 3).cpu().numpy()[:, 0]
    assert np.array_equal(got == FLT_MAX, want == FLT_MAX)
    fin = want != FLT_MAX
    # trajectories are bit-identical; only the 192,000-term residual sum differs.  Against the
    # float64-accumulated sum the tolerance is 1e-4; the oracle's own sequential float32 sum
    # (the reference thread's order) is itself ~1e-4 low and is held to 5e-4.
    assert np.allclose(got[fin], want64[fin], rtol=1e-4, atol=1e-7)
    assert np.allclose(got[fin], want[fin], rtol=5e-4, atol=1e-7)
    assert want[0] < 1e-3 and want[1:-1].min() > 1.0                     # the true system wins by a wide margin
    assert int(np.argmin(got)) == int(np.argmin(want)) == 0


def test_banks_toggles_and_random_right_hand_sides(cuda):
    S_, K, nb, bits = 2, 3, 3, 1
    ops = [(P.op("ADD"), 2), (P.op("SUB"), 2), (P.op("MUL"), 2), (P.op("SIN"), 1), (P.op("COS"), 1), (P.op("TANH"), 1)]
    raw = P.random_population(12, 40 * S_, 14, S_, K, 1.0, toggle_bits=bits, ops=ops)
    # damp every candidate: rhs_s = tanh(program) - state_s keeps trajectories bounded and contracting
    asts = [a[:-1] + P.op("TANH") + P.col(i % S_) + P.op("SUB") + P.RET for i, a in enumerate(raw.asts)]
    pop = P.PackedPrograms(asts, raw.routines)
    points, ntraj = 21, 130                                             # more than one block of 128 trajectories
    times = (np.arange(points, dtype=np.float32) * np.float32(0.05)).astype(np.float32)
    ref = np.stack([P.uniform(13, s, ntraj * points, -1, 1) for s in range(S_)])
    banks = np.stack([np.stack([P.normal(14, sy * 10 + b, K) for b in range(nb)]) for sy in range(40)])
    got = rk4_score(pop, S_, dev(ref), dev(times), dev(banks), K, nb, bits, 2).cpu().numpy()
    for cfg in range(nb << bits):
        code, want = S.oracle_rk4(pop, S_, ref, ntraj, times, np.ascontiguousarray(banks[:, cfg >> bits, :]), 2, bits, cfg & 1)
        assert code == 0
        assert np.allclose(got[:, cfg], want, rtol=2e-4, atol=1e-6), cfg


def test_reference_launch_layout_ragged_trajectories_and_invalid_matrix(cuda):
    """The reference engine's own scoring test (projects/odezza/tests/o_scoring_cuda_test.c:97-186):
    ragged trajectories, irregular times, two steps per observation, closed form 0.4375 * e^2, and
    every invalid variation scores FLT_MAX."""
    from test_rk4_cpu import invalid_launch_matrix, reference_launch_case
    systems, reference, times, offsets, constants = reference_launch_case()
    off = torch.tensor(offsets.astype(np.int32), device="cuda")
    got = rk4_score(systems, 1, dev(reference), dev(times), dev(constants[:, None, :]), 1, steps_per_observation=2,
                    offsets=off).cpu().numpy()[:, 0]
    assert np.allclose(got, [0.4375 * e * e for e in range(4)], atol=2e-6)
    for oo, tt, rr in invalid_launch_matrix():
        got = rk4_score(systems, 1, dev(rr), dev(tt), dev(constants[:, None, :]), 1, steps_per_observation=2,
                        offsets=torch.tensor(oo.astype(np.int32), device="cuda")).cpu().numpy()
        assert np.all(got == FLT_MAX), (oo, tt, rr)


def test_ragged_missing_observations_against_the_oracle(cuda):
    """Random ragged layout (1 to 40 points per trajectory, 150 trajectories so that several
    128-trajectory groups and idle lanes occur), irregular steps, a tenth of the later observations
    missing; damped linear systems with per-system coefficients."""
    rng = np.random.default_rng(12)
    lengths = rng.integers(1, 41, size=150)
    lengths[5] = 1                                                      # a singleton: nothing to score, still validated
    offsets = np.concatenate([[0], np.cumsum(lengths)]).astype(np.uint32)
    total = int(offsets[-1])
    times = np.concatenate([np.cumsum(rng.uniform(0.01, 0.08, size=n)) for n in lengths]).astype(np.float32)
    reference = rng.normal(0, 1, size=(2, total)).astype(np.float32)
    later = np.ones(total, dtype=bool); later[offsets[:-1]] = False
    holes = later & (rng.random(total) < 0.1)
    reference[0, holes] = np.nan
    reference[1, np.roll(holes, 3) & later] = np.nan
    col, bank, op = P.col, P.bank, P.op
    n_sys = 20                                                           # x' = a y - b x, y' = -a x - b y
    pop = P.PackedPrograms([bank(0) + col(1) + op("MUL") + bank(1) + col(0) + op("MUL") + op("SUB") + P.RET,
                            bank(0) + col(0) + op("MUL") + op("NEG") + bank(1) + col(1) + op("MUL") + op("SUB") + P.RET] * n_sys)
    coeffs = np.stack([rng.uniform(0.5, 3, n_sys), rng.uniform(0.1, 1, n_sys)], axis=1).astype(np.float32)
    code, want, want64 = S.oracle_rk4(pop, 2, reference, len(lengths), times, coeffs, substeps=3, want64=True,
                                      offsets=offsets, allow_missing=True)
    assert code == 0 and np.all(want != FLT_MAX)
    off = torch.tensor(offsets.astype(np.int32), device="cuda")
    got = rk4_score(pop, 2, dev(reference), dev(times), dev(coeffs[:, None, :]), 2, steps_per_observation=3, offsets=off,
                    allow_missing=True).cpu().numpy()[:, 0]
    assert np.allclose(got, want64, rtol=1e-4, atol=1e-7)
    strict = rk4_score(pop, 2, dev(reference), dev(times), dev(coeffs[:, None, :]), 2, steps_per_observation=3,
                       offsets=off).cpu().numpy()
    assert np.all(strict == FLT_MAX)                                     # NaN observations need the opt-in


def test_sampled_parameter_pools_match_explicit_banks(cuda):
    """Coefficients drawn from shared pools (the reference engine's sampled parameters) must give the
    scores of the explicit bank table built with the same rule, bank by bank; a descriptor that
    points outside the pool makes that configuration invalid."""
    import ctypes as C
    from secant_b200 import abi
    rng = np.random.default_rng(21)
    n_sys, nb, K, pool_size = 12, 5, 2, 64
    uniform = rng.random(pool_size).astype(np.float32)
    normal = rng.normal(0, 1, pool_size).astype(np.float32)
    desc = [[(int(rng.integers(0, 40)), int(rng.integers(1, 5)), 1, 2.5, 0.5, 0.6, 2.8),        # a in [0.6, 2.8]
             (int(rng.integers(0, 40)), int(rng.integers(1, 5)), 2, 0.3, 0.5, 0.1, 1.0)] for _ in range(n_sys)]
    desc[3][1] = (0, 0, 0, 0.0, 0.25, 0.0, 0.0)          # fixed shift, the same for every bank
    desc[7][0] = (60, 3, 1, 1.0, 0.0, 0.0, 9.0)          # banks 2.. fall outside the pool
    raw = (abi.SampledParameter * (n_sys * K))()
    for i in range(n_sys):
        for k in range(K):
            raw[i * K + k] = abi.SampledParameter(*desc[i][k])
    blob = torch.tensor(np.frombuffer(bytes(raw), dtype=np.uint8).copy(), device="cuda")
    table = S.sampled_constants(desc, uniform, normal, nb)
    times = (np.arange(41, dtype=np.float32) * np.float32(0.05)).astype(np.float32)
    reference = np.concatenate([np.cos(times)[None, :], -np.sin(times)[None, :]]).astype(np.float32)
    reference = np.concatenate([reference, 0.5 * reference], axis=1)                     # two trajectories
    col, bank, op = P.col, P.bank, P.op
    pop = P.PackedPrograms([bank(0) + col(1) + op("MUL") + bank(1) + col(0) + op("MUL") + op("SUB") + P.RET,
                            bank(0) + col(0) + op("MUL") + op("NEG") + bank(1) + col(1) + op("MUL") + op("SUB") + P.RET] * n_sys)
    got = rk4_score(pop, 2, dev(reference), dev(times), None, K, num_banks=nb,
                    sampled=(blob, dev(uniform), dev(normal))).cpu().numpy()
    explicit = rk4_score(pop, 2, dev(reference), dev(times), dev(table), K, num_banks=nb).cpu().numpy()
    assert np.array_equal(got, explicit)                                                   # same constants, same bits
    assert np.all(got[7, 2:] == FLT_MAX) and np.all(got[7, :2] != FLT_MAX)
    for b in range(nb):
        code, want, want64 = S.oracle_rk4(pop, 2, reference, 2, times, np.ascontiguousarray(table[:, b, :]), want64=True)
        assert code == 0
        assert np.array_equal(got[:, b] == FLT_MAX, want == FLT_MAX)
        fin = want != FLT_MAX
        assert np.allclose(got[fin, b], want64[fin], rtol=1e-4, atol=1e-7)


@pytest.mark.parametrize("ntraj,nb", [(20, 1), (20, 2), (20, 3), (20, 5), (50, 1), (50, 2), (50, 3), (130, 2)],
                         ids=["20x1", "20x2", "20x3", "20x5", "50x1", "50x2", "50x3", "130x2"])
def test_constant_only_sub_expressions_in_every_form(cuda, ntraj, nb):
    """Right-hand sides whose constant-only parts take every form the bank part knows — a product
    and a quotient of coefficients, an affine leaf, a toggle between two coefficients and between a
    coefficient and a state, a fused multiply-add over constants, a function of a constant, a
    right-hand side that is a constant altogether — with one, two and four trajectories per lane and
    one to five coefficient sets per system.  All operations but the exponential round identically
    on both sides, the systems contract, so the scores agree to summation order."""
    col, bank, lit, op = P.col, P.bank, P.lit, P.op
    damp = lambda s: col(s) + op("SUB") + P.RET                           # ... - state_s
    forms = [
        [bank(0) + bank(1) + op("MUL") + col(1) + op("MUL") + damp(0),                     # (c0 c1) y - x
         bank(2) + lit(4.0) + op("DIV") + col(0) + op("MUL") + damp(1)],                   # (c2 / 4) x - y
        [P.affine(1, 0.5, 0.25) + col(1) + op("MUL") + damp(0),                            # (c1/2 + 1/4) y - x
         bank(0) + bank(2) + P.tog2(0) + col(0) + op("MUL") + damp(1)],                    # {c0|c2} x - y
        [bank(0) + col(1) + P.tog2(1) + lit(0.5) + op("MUL") + damp(0),                    # {c0|y}/2 - x
         bank(0) + bank(1) + bank(2) + op("FMA") + col(0) + op("MUL") + damp(1)],          # fma(c0,c1,c2) x - y
        [bank(1) + op("NEG") + op("EXP") + col(1) + op("MUL") + damp(0),                   # exp(-c1) y - x
         bank(2) + bank(0) + op("SUB") + P.RET],                                           # c2 - c0: no state at all
        [col(0) + bank(1) + bank(2) + op("MUL") + lit(0.125) + op("FMA") + damp(0),        # fma(x, c1 c2, 1/8) - x
         bank(0) + op("ABS") + op("SQRT") + col(0) + col(1) + op("MIN") + op("MUL") + damp(1)],
    ]
    pop = P.PackedPrograms([p for system in forms for p in system])
    n_sys, K, bits, points = len(forms), 3, 2, 25
    times = (np.arange(points, dtype=np.float32) * np.float32(0.04)).astype(np.float32)
    ref = np.stack([P.uniform(31, s, ntraj * points, -1, 1) for s in range(2)])
    banks = np.stack([np.stack([P.uniform(32, sy * 7 + b, K, 0.2, 1.5) for b in range(nb)]) for sy in range(n_sys)])
    got = rk4_score(pop, 2, dev(ref), dev(times), dev(banks), K, nb, bits, 2).cpu().numpy()
    for cfg in range(nb << bits):
        code, want, want64 = S.oracle_rk4(pop, 2, ref, ntraj, times, np.ascontiguousarray(banks[:, cfg >> bits, :]), 2, bits,
                                          cfg & 3, want64=True)
        assert code == 0 and np.all(want != FLT_MAX)
        assert np.allclose(got[:, cfg], want64, rtol=1e-4, atol=1e-7), cfg


@pytest.mark.parametrize("ntraj", [20, 50])
def test_an_exploding_coefficient_set_does_not_touch_its_neighbours(cuda, ntraj):
    """Coefficient sets of one system are scored independently: x' = c0 x^2 - x blows up for the
    large c0 of every second set (score FLT_MAX, whenever it happens) while the sets beside it
    stay finite and keep the oracle's scores."""
    col, bank, op = P.col, P.bank, P.op
    pop = P.PackedPrograms([bank(0) + col(0) + op("MUL") + col(0) + op("MUL") + col(0) + op("SUB") + P.RET] * 3)
    nb, points = 4, 40
    times = (np.arange(points, dtype=np.float32) * np.float32(0.05)).astype(np.float32)
    ref = P.uniform(41, 0, ntraj * points, 0.5, 1.5)[None, :]
    banks = np.zeros((3, nb, 1), dtype=np.float32)
    banks[:, 0::2, 0] = [[-0.5, 0.25], [0.1, -1.0], [0.3, 0.2]]         # tame
    banks[:, 1::2, 0] = [[3.0e4, 1.0e6], [5.0e3, 2.0e5], [1.0e30, 4.0e4]]  # explosive, sooner or later
    got = rk4_score(pop, 1, dev(ref), dev(times), dev(banks), 1, nb).cpu().numpy()
    for b in range(nb):
        code, want, want64 = S.oracle_rk4(pop, 1, ref, ntraj, times, np.ascontiguousarray(banks[:, b, :]), want64=True)
        assert code == 0
        assert np.array_equal(got[:, b] == FLT_MAX, want == FLT_MAX), b
        assert np.all((want == FLT_MAX) == (b % 2 == 1))
        fin = want != FLT_MAX
        assert np.allclose(got[fin, b], want64[fin], rtol=1e-4, atol=1e-7), b


def test_a_structural_error_in_a_later_piece_ends_the_call_with_its_code(cuda):
    """Errors a token scan cannot see (here a stack underflow) are found while a piece of 128
    systems is being encoded, possibly after earlier launches have started: the call waits for
    what it launched and answers with that code."""
    from secant_b200 import abi
    systems, reference, times, constants = slope_case()
    good = systems.asts[0]
    asts = [good] * 2600
    asts[2300] = P.col(0) + P.op("ADD") + P.RET
    coeffs = np.tile(constants[:1], (len(asts), 1))
    with pytest.raises(abi.SecantError) as failure:
        rk4_score(P.PackedPrograms(asts, systems.routines), 1, dev(reference), dev(times), dev(coeffs[:, None, :]), 1, 1, 0, 4)
    assert failure.value.code == abi.ERROR_STACK_UNDERFLOW
    again = rk4_score(systems, 1, dev(reference), dev(times), dev(constants[:, None, :]), 1, 1, 0, 4).cpu().numpy()[:, 0]
    assert np.allclose(again, [0.53125 * e * e for e in range(4)], atol=2e-6)          # the library is usable afterwards
