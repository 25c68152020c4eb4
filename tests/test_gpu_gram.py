"""The static Gram-statistics shape (projects/secant/secant.h:478-504) on the device: cohort sums,
the full Gram matrix and the cross sums with the targets against the CPU restatement (bit-identical
to the reference's host run, tests/test_oracle_golden.py) through its float64 sums."""
import numpy as np
import pytest
import torch

import support as S
from secant_b200 import abi, programs as P
from secant_b200.runner import Runner

pytestmark = pytest.mark.gpu


def dev(a):
    return torch.tensor(np.ascontiguousarray(a), device="cuda")


@pytest.mark.parametrize("programs,cohort,rows,targets", [(13, 3, 257, 2), (64, 32, 1000, 1), (70, 32, 4097, 3), (5000, 8, 700, 2)])
def test_gram_statistics_match_the_restatement(cuda, programs, cohort, rows, targets):
    ops = [(P.op("ADD"), 2), (P.op("SUB"), 2), (P.op("MUL"), 2), (P.op("SIN"), 1), (P.op("COS"), 1), (P.op("TANH"), 1)]
    pop = P.random_population(71 + programs, programs, 12, 5, ops=ops)
    x = np.stack([P.uniform(72, c, rows, -1, 1) for c in range(5)])
    y = np.stack([P.normal(73, t, rows) for t in range(targets)])
    with Runner(abi.SHAPE_GRAM_STATS, 5, targets, num_kernels=4, asts_per_kernel=cohort, workers=2, streams=2) as rn:
        got = rn.gram_stats(pop, dev(x), dev(y)).cpu().numpy()
        rn.set_scratch_limit(4 * 200 * programs)                       # a few hundred rows per range: many ranges, added in order
        ranged = rn.gram_stats(pop, dev(x), dev(y)).cpu().numpy()
        again = rn.gram_stats(pop, dev(x), dev(y)).cpu().numpy()
    code, _, want64 = S.oracle_gram_stats(pop, x, y, cohort)
    assert code == 0
    scale = np.abs(want64).max(axis=1, keepdims=True) + 1.0
    for name, out in (("whole", got), ("ranged", ranged)):
        assert np.isfinite(out).all(), name                            # every entry was cleared, inactive ones are zero
        assert np.all(np.abs(out - want64) <= 2e-5 * scale), (name, float(np.abs(out - want64).max()))
    assert np.array_equal(ranged.view(np.uint32), again.view(np.uint32))          # same request, same bits
    last = programs - (programs - 1) // cohort * cohort                # programs of the last cohort
    if last < cohort:
        assert np.all(got[-1, last:cohort] == 0)
        gram = got[-1, cohort:cohort + cohort * cohort].reshape(cohort, cohort)
        assert np.all(gram[last:, :] == 0) and np.all(gram[:, last:] == 0)


def test_gram_runner_through_the_reference_create_sequence_and_bad_requests(cuda):
    """The plan route (source, plan, runner) and the request checks of the shape: the statistics
    vector must cover a full cohort, and a population cannot be made for it."""
    import ctypes as C
    pop = P.PackedPrograms([P.col(0) + P.col(1) + P.op("ADD") + P.RET, P.col(1) + P.col(2) + P.op("MUL") + P.RET] * 3)
    x = np.stack([P.uniform(81, c, 300, -1, 1) for c in range(3)])
    y = np.stack([P.normal(82, 0, 300)])
    with Runner(abi.SHAPE_GRAM_STATS, 3, 1, num_kernels=2, asts_per_kernel=3, via_plan=True) as rn:
        got = rn.gram_stats(pop, dev(x), dev(y)).cpu().numpy()
        _, _, want64 = S.oracle_gram_stats(pop, x, y, 3)
        assert np.allclose(got, want64, rtol=2e-5, atol=2e-5)
        short = torch.zeros((2, 3 * (1 + 3 + 1) - 1), device="cuda")
        assert rn.run(rn.static_request(pop, dev(x), dev(y), short), check=False) == abi.ERROR_INVALID_VALUE
        pset = abi.ProgramSet()
        pop.fill(pset)
        handle = C.c_void_p()
        assert rn.lib.secant_b200_population_create(rn.handle, C.byref(pset), 0, C.byref(handle)) == abi.ERROR_UNSUPPORTED_SHAPE
