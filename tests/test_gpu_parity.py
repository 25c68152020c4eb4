"""GPU parity: the CUDA evaluator, called through the C-ABI, against the CPU oracle and the
golden vectors recorded from the reference's own host evaluator.

Tolerances (tests/parity.py): per-row predictions 1e-5 relative + 1e-6 absolute with
identical NaN/Inf masks; sums of squared errors 1e-4 relative against the oracle's float64
accumulation.  Where a program is ill-conditioned (its value moves by more than that when
the math library's transcendental results move by 2 ulp) the bound widens by the measured
sensitivity; the share of bins that cannot be compared at all is bounded in each test.
"""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import parity
import support as S
from secant_b200 import abi, programs as P
from secant_b200.runner import Runner
from test_oracle_golden import G, packed, toggle_expected

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.tensor(np.ascontiguousarray(a), device="cuda")


@pytest.mark.parametrize("packed_asts", [1, 3])
def test_fixture_closed_forms_padding_and_changed_banks(cuda, packed_asts):
    """projects/secant/tests/toggle_cuda_test.c:166-256 with its two recipes (3 kernels of 1 or 3 programs)."""
    fx = packed("fixture")
    x, y, banks = G["fixture_x"], G["fixture_y"], G["fixture_banks"]
    with Runner(abi.SHAPE_TOGGLE_SSE, 3, 2, 2, workers=3, streams=2, via_plan=True, num_kernels=3,
                asts_per_kernel=packed_asts) as rn:
        for pass_idx in range(2):
            b = banks if pass_idx == 0 else (banks + np.float32(0.137)).astype(np.float32)
            out = torch.full((7, 2, 109), -123.0, device="cuda")
            rn.run(rn.toggle_request(fx, dev(x), dev(y), dev(b), 13, 3, out, out_ld=109))
            got = out.cpu().numpy()
            want = G[f"fixture_sse_pass{pass_idx}"]
            assert np.all(got[:, :, 104:] == -123.0)
            assert np.allclose(got[:, :, :104], want[:, :, :104], rtol=1e-5, atol=1e-7)
            for a in range(7):
                for bank in (0, 5, 12):
                    for p in range(8):
                        e = np.array([toggle_expected(a, p, x[:, r], b[bank]) for r in range(17)], dtype=np.float64)
                        ref = ((e - y[1].astype(np.float64)) ** 2).sum()
                        assert abs(got[a, 1, bank * 8 + p] - ref) <= 1e-5 * (1 + abs(ref))
        # module counts come in the reference's unit: programs per recipe capacity (toggle_cuda_test.c:245)
        assert rn.stats.modules_loaded == (7 + 3 * packed_asts - 1) // (3 * packed_asts) == rn.stats.num_modules
        assert rn.stats.num_asts == 7 and rn.stats.runtime_seconds > 0


def test_affine_leaf_exact_values(cuda):
    with Runner(abi.SHAPE_TOGGLE_SSE, 1, 1, 1) as rn:
        got = rn.toggle_sse(packed("affine"), dev(G["affine_x"]), dev(G["affine_y"]), dev(G["affine_banks"]), 2, 1)
    assert got.cpu().numpy().reshape(-1).tolist() == [6.25, 25.0, 16.0, 25.0]


def test_golden_random_population_against_reference_vectors(cuda):
    pop = packed("random")
    x, y, banks = G["random_x"], G["random_y"], G["random_banks"]
    with Runner(abi.SHAPE_TOGGLE_SSE, 3, 2, 4, workers=2, streams=2) as rn:
        got = rn.toggle_sse(pop, dev(x), dev(y), dev(banks), 5, 3).cpu().numpy()
    slack = S.sse_slack(pop, x, y, banks, 4, 3)
    _, _, want64 = S.oracle_toggle_sse(pop, x, y, banks, 4, 3)
    assert parity.ill_conditioned_fraction(slack) < 0.05
    assert not parity.sse_mismatches(got, want64, slack).any()
    # and directly against what the reference library printed, on the well-conditioned bins
    calm = slack < 1e-6 * np.abs(want64)
    assert calm.mean() > 0.5
    assert np.allclose(got[calm], G["random_sse"][calm], rtol=2e-4, atol=1e-6)


@pytest.mark.parametrize("rows", [1, 127, 128, 129, 255, 256, 257, 4097])
@pytest.mark.parametrize("nb", [5, 2, 1], ids=["tile4x4", "tile8x2", "tile16x1"])
def test_tile_boundaries_all_register_tiles(cuda, rows, nb):
    """Row counts around the pass sizes of every register tile (the bank count selects the tile:
    4 rows x 4 banks from four banks on, 8 x 2 for two or three, 16 x 1 for one), and 4,097 rows:
    eight full tiles of 512 plus one row."""
    bits = 2
    pop = P.random_population(31, 40, 32, 5, 6, 2.0, toggle_bits=bits)
    x = np.stack([P.uniform(32, c, rows, -2, 2) for c in range(5)])
    y = np.stack([P.normal(33, t, rows) for t in range(1)])
    banks = np.stack([P.normal(34, b, 6) for b in range(nb)])
    with Runner(abi.SHAPE_TOGGLE_SSE, 5, 1, 6) as rn:
        got = rn.toggle_sse(pop, dev(x), dev(y), dev(banks), nb, bits).cpu().numpy()
    want64, slack = S.sse_reference_parallel(pop, x, y, banks, 6, bits)
    print(f"skipped bins: {int((~np.isfinite(slack)).sum())} of {slack.size}")
    assert parity.ill_conditioned_fraction(slack) < 0.1
    bad = parity.sse_mismatches(got, want64, slack)
    assert not bad.any(), (int(bad.sum()), np.argwhere(bad)[:4].tolist())


def test_config1_static_sse_and_per_row_materialize(cuda):
    """The CPU-runnable reference check: 64 programs of at most 15 tokens, 4096 rows, 4 features."""
    rows = 4096
    pop = P.random_population(1, 64, 15, 4, 0, 1.0)
    x = np.stack([P.uniform(1, c, rows, -1, 1) for c in range(4)])
    y = (x[0] * x[1] + np.sin(x[2]) + P.normal(1, 99, rows, 0.01))[None, :].astype(np.float32)
    with Runner(abi.SHAPE_MATERIALIZE, 4) as rn:
        mat = rn.materialize(pop, dev(x)).cpu().numpy()
    with Runner(abi.SHAPE_SSE, 4, 1) as rn:
        sse = rn.sse(pop, dev(x), dev(y)).cpu().numpy()
    base, sens = S.row_sensitivity(pop, x, None, 0, 0, 0)
    bad = parity.row_mismatches(mat, base, sens)
    assert not bad.any(), f"{int(bad.sum())} rows differ"
    assert np.array_equal(np.isnan(mat), np.isnan(base)) and np.array_equal(np.isinf(mat), np.isinf(base))
    plain = parity.row_mismatches(mat, base)
    assert plain.mean() < 0.002  # without the conditioning allowance nearly every row still agrees
    _, sse32, sse64 = S.oracle_sse(pop, x, y)
    with np.errstate(invalid="ignore", over="ignore"):
        slack = (2 * np.abs(base.astype(np.float64) - y.astype(np.float64)) * sens + sens * sens).sum(axis=1)[:, None]
    slack[np.isnan(slack)] = np.inf
    assert not parity.sse_mismatches(sse, sse64, slack).any()
    # identical ordering of the losses wherever the gap exceeds the tolerance
    order_ref = np.argsort(sse64[:, 0], kind="stable")
    finite = np.isfinite(sse64[order_ref, 0])
    ranked = sse64[order_ref, 0][finite]
    gaps_ok = np.diff(ranked) > 2e-4 * ranked[1:]
    got_ranked = sse[order_ref, 0][finite]
    assert np.all(np.diff(got_ranked)[gaps_ok] > 0)
    # golden prefix: first 512 rows were materialized by the reference itself
    gm = G["c1_materialize"]
    assert not parity.row_mismatches(mat[:, :512], gm, sens[:, :512]).any()


def test_static_programs_with_routine_and_two_targets(cuda):
    st = packed("static")
    with Runner(abi.SHAPE_MATERIALIZE, 3) as rn:
        mat = rn.materialize(st, dev(G["static_x"])).cpu().numpy()
    assert np.allclose(mat, G["static_materialize"], rtol=1e-5, atol=1e-6)
    with Runner(abi.SHAPE_SSE, 3, 2) as rn:
        sse = rn.sse(st, dev(G["static_x"]), dev(G["static_y"])).cpu().numpy()
    assert np.allclose(sse, G["static_sse"], rtol=1e-5, atol=1e-6)
    with Runner(abi.SHAPE_AFFINE_STATS, 3, 2) as rn:
        stats = rn.affine_stats(st, dev(G["static_x"]), dev(G["static_y"])).cpu().numpy()
    p = G["static_materialize"].astype(np.float64)
    t = G["static_y"].astype(np.float64)
    want = np.stack([p.sum(1), (p * p).sum(1), (p * t[0]).sum(1), (p * t[1]).sum(1)], axis=1)
    assert np.allclose(stats, want, rtol=1e-5, atol=1e-6)


def test_per_program_banks_and_resident_population(cuda):
    nb, K, A, rows = 6, 4, 50, 300
    pop = P.random_population(55, A, 24, 3, K, 1.0, ops=P.ARITHMETIC_OPS)
    x = np.stack([P.uniform(56, c, rows, -1, 1) for c in range(3)])
    y = np.stack([P.normal(57, 0, rows)])
    banks = np.stack([np.stack([P.normal(58, a * 100 + b, K) for b in range(nb)]) for a in range(A)])  # [ast][bank][slot]
    _, _, want64 = S.oracle_toggle_sse(pop, x, y, banks, K, 0, bank_stride=K, program_bank_stride=nb * K)
    with Runner(abi.SHAPE_TOGGLE_SSE, 3, 1, K, workers=2, streams=3) as rn:
        out = torch.empty((A, 1, nb), device="cuda")
        req = rn.toggle_request(pop, dev(x), dev(y), dev(banks), nb, 0, out, bank_stride=K, program_bank_stride=nb * K)
        rn.run(req)
        got = out.cpu().numpy()
        assert np.allclose(got, want64, rtol=1e-4, atol=1e-6, equal_nan=True)
        resident = rn.population(pop, 0)
        out.fill_(7.0)
        resident.run(req)
        assert np.array_equal(out.cpu().numpy(), got)       # same kernels, same order, same bits
        assert resident.num_ops == int(P.count_ops(pop).sum())
        # a slice of the population addressed through first_program_index
        half = pop.subset(range(25, 50))
        out2 = torch.empty((25, 1, nb), device="cuda")
        rn.run(rn.toggle_request(half, dev(x), dev(y), dev(banks), nb, 0, out2, bank_stride=K, program_bank_stride=nb * K,
                                 first_program_index=25))
        assert np.array_equal(out2.cpu().numpy(), got[25:])
        resident.destroy()


def test_batched_entries_share_one_program_upload(cuda):
    pop = P.random_population(61, 33, 24, 3, 4, 1.0, toggle_bits=2, ops=P.ARITHMETIC_OPS)
    data = []
    for e, (rows, nb) in enumerate([(97, 5), (300, 2)]):
        x = np.stack([P.uniform(62 + e, c, rows, -1, 1) for c in range(3)])
        y = np.stack([P.normal(64 + e, t, rows) for t in range(2)])
        b = np.stack([P.normal(66 + e, i, 4) for i in range(nb)])
        data.append((x, y, b, nb))
    with Runner(abi.SHAPE_TOGGLE_SSE, 3, 2, 4, workers=2, streams=2) as rn:
        outs, reqs, keep = [], [], []
        for x, y, b, nb in data:
            out = torch.empty((33, 2, nb << 2), device="cuda")
            tensors = (dev(x), dev(y), dev(b))
            keep.append(tensors)
            outs.append(out)
            reqs.append(rn.toggle_request(pop, *tensors, nb, 2, out))
        rn.run_batch(reqs)
        for out, (x, y, b, nb) in zip(outs, data):
            _, _, want64 = S.oracle_toggle_sse(pop, x, y, b, 4, 2)
            assert np.allclose(out.cpu().numpy(), want64, rtol=1e-4, atol=1e-6, equal_nan=True)


def test_errors_before_any_output_is_touched_and_runner_reuse(cuda):
    fx = packed("fixture")
    x, y, banks = dev(G["fixture_x"]), dev(G["fixture_y"]), dev(G["fixture_banks"])
    with Runner(abi.SHAPE_TOGGLE_SSE, 3, 2, 2) as rn:
        out = torch.full((7, 2, 52), 1234.0, device="cuda")
        code = rn.run(rn.toggle_request(fx, x, y, banks, 13, 2, out), check=False)  # programs use toggle bit 2
        assert code == abi.ERROR_BAD_PROGRAM and bool((out == 1234.0).all())
        assert rn.stats.num_modules == 0 and rn.stats.total_seconds == 0
        big = torch.full((7, 2, 104), 5.0, device="cuda")
        req = rn.toggle_request(fx, x, y, banks, 13, 3, big)
        req.base.output.address = x.data_ptr()
        assert rn.run(req, check=False) == abi.ERROR_INVALID_VALUE
        req = rn.toggle_request(fx, x, y, banks, 13, 3, big)
        req.base.constants.num_elements = 37
        assert rn.run(req, check=False) == abi.ERROR_INSUFFICIENT_BUFFER
        under = P.PackedPrograms([P.col(0) + P.op("ADD") + P.RET])
        one = torch.empty((1, 2, 104), device="cuda")
        assert rn.run(rn.toggle_request(under, x, y, banks, 13, 3, one), check=False) == abi.ERROR_STACK_UNDERFLOW
        # the handle stays usable after validation and structural failures
        rn.run(rn.toggle_request(fx, x, y, banks, 13, 3, big))
        assert np.allclose(big.cpu().numpy(), G["fixture_sse_pass0"][:, :, :104], rtol=1e-5, atol=1e-7)
        sse_shape = abi.init_header(abi.StaticRun(), abi.RUN_VERSION, abi.SHAPE_SSE)
        assert rn.run(sse_shape, check=False) == abi.ERROR_UNSUPPORTED_SHAPE


def test_size_independent_properties_at_a_million_rows(cuda):
    """Full row count of the headline configuration, checked through exact identities:
    a program equal to the target scores 0, target + 1 scores exactly N, and the scores of
    2048 + 1 programs do not depend on how rows are split across CTAs."""
    rows = 1 << 20
    x = torch.stack([torch.tensor(P.uniform(70, c, rows, -3, 3), device="cuda") for c in range(2)])
    y = x[0:1].clone()
    progs = [P.col(0) + P.RET, P.col(0) + P.lit(1.0) + P.op("ADD") + P.RET, P.col(0) + P.bank(0) + P.op("ADD") + P.RET]
    banks = dev(np.array([[0.0], [1.0], [-2.0], [0.5]], dtype=np.float32))
    with Runner(abi.SHAPE_TOGGLE_SSE, 2, 1, 1) as rn:
        got = rn.toggle_sse(P.PackedPrograms(progs), x, y, banks, 4, 0).cpu().numpy()
    assert got[0, 0].tolist() == [0.0] * 4
    assert got[1, 0].tolist() == [float(rows)] * 4
    assert got[2, 0].tolist() == [0.0, float(rows), 4.0 * rows, 0.25 * rows]


def _ulps(got, exact64):
    """Error of float32 results in units of the last place of the correctly rounded answer."""
    with np.errstate(all="ignore"):
        ref = exact64.astype(np.float32)
        ulp = np.spacing(np.abs(ref)).astype(np.float64)
        err = np.abs(got.astype(np.float64) - exact64) / ulp
    same_special = (np.isnan(got) & np.isnan(ref)) | (np.isinf(ref) & (got == ref)) | ((ref == 0) & (got == 0))
    return np.where(same_special, 0.0, err)


def test_device_functions_against_float64(cuda):
    """Every unary operation and the division on arguments from tiny to huge, with the special
    values: arithmetic is correctly rounded, transcendentals stay within 2-3 ulp of float64,
    and NaN / infinity appear exactly where the host functions produce them."""
    words = P._stream(77, 0, 1 << 16)
    mags = np.float32(10.0) ** (P.uniform(77, 1, 1 << 16, -6, 6))
    signs = np.where(words & 1, np.float32(1), np.float32(-1))
    x = (mags * signs).astype(np.float32)
    x[:24] = np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1.0, -1.0, 88.0, 88.72, 88.73, 89.5, -87.0, -88.0, -103.0,
                       -104.5, 1e-40, -1e-40, 3.4e38, 4095.9, 4096.0, 1e30, 86.0, 86.00001, 127.5], dtype=np.float32)
    x[24:4096] = P.uniform(77, 2, 4072, -100, 100)       # the range exp and trig arguments usually live in
    x[4096:6144] = (np.arange(2048, dtype=np.float64) * np.pi / 2).astype(np.float32)   # zeros of sin and cos
    y = np.roll(x, 7919).copy()
    unary = [("NEG", lambda a: -a, 0.0), ("ABS", np.abs, 0.0), ("SQRT", np.sqrt, 0.5), ("RCP", lambda a: 1.0 / a, 0.5),
             ("RSQRT", lambda a: 1.0 / np.sqrt(a), 2.0), ("SIN", np.sin, 2.0), ("COS", np.cos, 2.0),
             ("EXP", np.exp, 2.5), ("LOG", np.log, 2.0), ("EX2", np.exp2, 2.5), ("LG2", np.log2, 2.0), ("TANH", np.tanh, 2.5)]
    asts = [P.col(0) + P.op(name) + P.RET for name, _, _ in unary]
    asts.append(P.col(0) + P.col(1) + P.op("DIV") + P.RET)
    asts.append(P.col(1) + P.col(0) + P.col(0) + P.op("MUL") + P.op("DIV") + P.RET)   # operand on the left of a computed value
    pop = P.PackedPrograms(asts)
    with Runner(abi.SHAPE_MATERIALIZE, 2) as rn:
        got = rn.materialize(pop, dev(np.stack([x, y]))).cpu().numpy()
    x64, y64 = x.astype(np.float64), y.astype(np.float64)
    with np.errstate(all="ignore"):
        for i, (name, fn, bound) in enumerate(unary):
            exact = fn(x64)
            err = _ulps(got[i], exact)
            if name in ("EXP", "EX2"):    # results in the denormal range are rounded twice
                err = np.where(np.abs(exact) < 1.2e-38, np.minimum(err, bound), err)
            assert np.nanmax(err) <= bound + 0.5 * (bound > 0), (name, float(np.nanmax(err)), float(x[np.nanargmax(err)]))
            want = exact.astype(np.float32)
            assert np.array_equal(np.isnan(got[i]), np.isnan(want)), name
            assert np.array_equal(np.isinf(got[i]), np.isinf(want)), name
        assert np.array_equal(got[len(unary)].view(np.uint32)[~np.isnan(got[len(unary)])],
                              (x / y).view(np.uint32)[~np.isnan(x / y)])             # IEEE division, bit for bit
        assert np.array_equal(np.isnan(got[len(unary)]), np.isnan(x / y))
        xx = x * x
        want = y / xx
        assert np.array_equal(got[len(unary) + 1].view(np.uint32)[~np.isnan(want)], want.view(np.uint32)[~np.isnan(want)])


def test_toggle_heavy_population_with_best_variant(cuda):
    """The toggle-heavy benchmark configuration at reduced size: 48-token programs whose subtrees
    are gated by 8 toggle bits (256 variants) times 4 coefficient sets = 1,024 configurations per
    program, N(0,1) features; fused losses against the oracle, then the best variant per program
    (valid = finite and non-negative, lowest index wins ties)."""
    bits, nb, rows, F, K, A = 8, 4, 300, 6, 8, 24
    pop = P.gated_population(3, A, 48, F, K, bits)
    x = np.stack([P.normal(3, c, rows) for c in range(F)])
    y = np.stack([P.normal(3, 100, rows)])
    banks = np.stack([P.normal(3, 200 + b, K) for b in range(nb)])
    with Runner(abi.SHAPE_TOGGLE_SSE, F, 1, K, workers=2, streams=2) as rn:
        out = rn.toggle_sse(pop, dev(x), dev(y), dev(banks), nb, bits)
    got = out.cpu().numpy()
    _, _, want64 = S.oracle_toggle_sse(pop, x, y, banks, K, bits)
    slack = S.sse_slack(pop, x, y, banks, K, bits)
    assert got.shape == (A, 1, nb << bits)
    assert parity.ill_conditioned_fraction(slack) < 0.1
    assert not parity.sse_mismatches(got, want64, slack).any()
    from secant_b200 import runner as R
    sse, cfg, valid = (t.cpu().numpy() for t in R.score_fields(R.best_config(out.view(A, nb << bits))))
    grid = want64[:, 0, :]
    ok = np.isfinite(grid) & (grid >= 0)
    assert np.array_equal(valid.view(np.uint64), (np.isfinite(got[:, 0, :]) & (got[:, 0, :] >= 0)).sum(axis=1).astype(np.uint64))
    for a in range(A):
        if not ok[a].any():
            assert int(cfg[a]) == -1
            continue
        best = grid[a][ok[a]].min()
        chosen = int(cfg[a])
        # gated-off subtrees make many variants exactly equal, so the winner is checked as a member
        # of the oracle's set of minimisers (within the loss tolerance), and as the lowest index
        # among the device's own equal scores
        assert grid[a, chosen] - best <= 2e-4 * abs(best) + 2 * slack[a, 0, chosen] + 1e-6, (a, chosen)
        assert abs(float(sse[a]) - got[a, 0, chosen]) == 0
        assert not (got[a, 0, :chosen] <= got[a, 0, chosen]).any()


def test_zero_columns_constants_toggles_and_routine_toggle_propagation(cuda):
    """projects/secant/tests/toggle_cuda_test.c:431-497: a literal-only program with no input
    matrix, no constants and no toggle; then a toggle over two bank leaves that lives inside a
    routine, called from the program."""
    t = np.array([[0, .1, .2, .3, .4, .5, .6, .7, .8]], dtype=np.float32)
    literal = P.PackedPrograms([P.lit_bits(0x40000000) + P.RET])                      # 2.0f
    with Runner(abi.SHAPE_TOGGLE_SSE, 0, 1, 0, via_plan=True, num_kernels=1, asts_per_kernel=1) as rn:
        out = torch.full((1, 1, 2), -7.0, device="cuda")
        rn.run(rn.toggle_request(literal, None, dev(t), None, 1, 0, out, out_ld=2))
        got = out.cpu().numpy().reshape(-1)
    assert abs(got[0] - float(((2.0 - t.astype(np.float64)) ** 2).sum())) < 1e-5 and got[1] == -7.0
    routed = P.PackedPrograms([P.routine(0) + P.RET], [P.bank(0) + P.bank(1) + P.tog2(0) + P.RET])
    banks = np.array([[.7, -.3]], dtype=np.float32)
    with Runner(abi.SHAPE_TOGGLE_SSE, 0, 1, 2, via_plan=True, num_kernels=1, asts_per_kernel=1) as rn:
        got = rn.toggle_sse(routed, None, dev(t), dev(banks), 1, 1).cpu().numpy().reshape(-1)
    want = [float(((v - t.astype(np.float64)) ** 2).sum()) for v in (np.float32(.7), np.float32(-.3))]
    assert np.allclose(got, want, rtol=1e-6, atol=1e-6)
    _, _, want64 = S.oracle_toggle_sse(routed, None, t, banks, 2, 1)
    assert np.allclose(got, want64.reshape(-1), rtol=1e-6, atol=1e-6)


def test_box_scale_population_of_a_million_programs(cuda):
    """The sharded benchmark configuration's population size on one GPU (rows reduced): 2^20
    programs, 16 coefficient sets, 16 features.  The population repeats a block of 65,536
    programs, so every block of scores must repeat the first one bit for bit (one chunk of rows,
    hence one addition per bin), and the first programs are checked against the oracle."""
    block, repeats, rows, F, K, nb = 65536, 16, 256, 16, 16, 16
    base = P.random_population(5, block, 32, F, K, 1.0)
    pop = P.PackedPrograms(base.asts * repeats, base.routines)
    x = np.stack([P.uniform(5, c, rows, -1, 1) for c in range(F)])
    y = np.stack([P.normal(5, 100, rows)])
    banks = np.stack([P.normal(5, 200 + b, K) for b in range(nb)])
    with Runner(abi.SHAPE_TOGGLE_SSE, F, 1, K, workers=8, streams=2) as rn:
        out = rn.toggle_sse(pop, dev(x), dev(y), dev(banks), nb, 0)
        assert rn.stats.num_asts == block * repeats
    grid = out.view(repeats, block, nb)
    same = (grid == grid[0:1]) | (torch.isnan(grid) & torch.isnan(grid[0:1]))
    assert bool(same.all())
    head = base.subset(range(200))
    _, _, want64 = S.oracle_toggle_sse(head, x, y, banks, K, 0)
    slack = S.sse_slack(head, x, y, banks, K, 0)
    assert not parity.sse_mismatches(grid[0, :200].cpu().numpy()[:, None, :], want64, slack).any()


def test_fast_math_mode_meets_the_reference_gpu_tolerance(cuda):
    """secant_b200_runner_set_math(FAST) selects the approximations the reference's GPU kernels are
    compiled with; its results are held to the reference GPU test's own bound against the host
    evaluator, 2e-4 * (1 + |cpu|) (projects/secant/tests/toggle_cuda_test.c:158-165), on that
    test's two workloads: the closed-form fixture and the seeded random toggle population."""
    def close(got, want):
        return np.abs(got - want) <= 2e-4 * (1 + np.abs(want))
    fx = packed("fixture")
    with Runner(abi.SHAPE_TOGGLE_SSE, 3, 2, 2, workers=2, streams=2) as rn:
        assert rn.lib.secant_b200_runner_set_math(rn.handle, 2) == abi.ERROR_INVALID_VALUE
        args = (fx, dev(G["fixture_x"]), dev(G["fixture_y"]), dev(G["fixture_banks"]), 13, 3)
        accurate = rn.toggle_sse(*args).cpu().numpy()
        rn.set_math(True)
        fast = rn.toggle_sse(*args).cpu().numpy()
        rn.set_math(False)
        again = rn.toggle_sse(*args).cpu().numpy()
    want = G["fixture_sse_pass0"][:, :, :104]
    assert close(fast, want).all() and np.array_equal(accurate, again)
    pop = packed("random")
    with Runner(abi.SHAPE_TOGGLE_SSE, 3, 2, 4, workers=2, streams=2) as rn:
        rn.set_math(True)
        fast = rn.toggle_sse(pop, dev(G["random_x"]), dev(G["random_y"]), dev(G["random_banks"]), 5, 3).cpu().numpy()
    ref = G["random_sse"]
    finite = np.isfinite(ref)
    assert np.array_equal(np.isfinite(fast), finite)
    assert close(fast[finite], ref[finite]).mean() > 0.97     # ill-conditioned bins aside (the accurate mode widens them too)
