"""Device-side best-configuration and top-k reductions against the CPU oracle's restatement
of the reference rules (projects/secant-sr/toggle/src/cpu.c:45-67,
projects/odezza/core/o_score_reduce.cu:36-39).  Index work: results must match exactly."""
import ctypes as C

import numpy as np
import pytest
import torch

import support as S
from secant_b200 import runner as R

pytestmark = pytest.mark.gpu


def oracle_best(grid):
    a, c = grid.shape
    best = np.zeros(a, dtype=np.float32)
    arg = np.zeros(a, dtype=np.uint64)
    valid = np.zeros(a, dtype=np.uint64)
    S.oracle().so_best_config(S.fptr(grid), C.c_size_t(a), C.c_size_t(c), C.c_size_t(c), S.fptr(best),
                              arg.ctypes.data_as(S.U64P), valid.ctypes.data_as(S.U64P))
    return best, arg, valid


def oracle_topk(scores, k):
    idx = np.zeros(k, dtype=np.uint64)
    S.oracle().so_topk.restype = C.c_size_t
    n = S.oracle().so_topk(S.fptr(scores), C.c_size_t(scores.size), C.c_size_t(k), idx.ctypes.data_as(S.U64P))
    return idx[:n]


def noisy_scores(rng, shape):
    g = rng.random(shape, dtype=np.float32) * 10
    flat = g.reshape(-1)
    n = flat.size
    flat[rng.integers(0, n, n // 9)] = np.nan
    flat[rng.integers(0, n, n // 13)] = np.inf
    flat[rng.integers(0, n, n // 17)] = -1.0
    flat[rng.integers(0, n, n // 5)] = np.float32(0.5)   # plenty of exact ties
    flat[rng.integers(0, n, n // 50 + 1)] = 0.0
    flat[rng.integers(0, n, n // 70 + 1)] = -0.0
    return g


@pytest.mark.parametrize("shape", [(1, 1), (7, 104), (300, 1024), (33, 5000)])
def test_best_config_matches_rule(cuda, shape):
    rng = np.random.default_rng(shape[0] * 31 + shape[1])
    grid = noisy_scores(rng, shape)
    grid[0, :] = np.nan                                  # a vector with no valid score
    rec = R.best_config(torch.tensor(grid, device="cuda"))
    sse, cfg, valid = (t.cpu().numpy() for t in R.score_fields(rec))
    best, arg, nvalid = oracle_best(grid)
    assert np.array_equal(sse.view(np.uint32), best.view(np.uint32))
    assert np.array_equal(cfg.view(np.uint64), arg)
    assert np.array_equal(valid.view(np.uint64), nvalid)
    assert np.isinf(sse[0]) and cfg[0] == -1 and valid[0] == 0


def test_best_config_respects_leading_dimension(cuda):
    rng = np.random.default_rng(3)
    full = torch.tensor(noisy_scores(rng, (40, 128)), device="cuda")
    view = full[:, :77]                                   # 77 configurations, 128 apart
    sse, cfg, _ = (t.cpu().numpy() for t in R.score_fields(R.best_config(view)))
    best, arg, _ = oracle_best(np.ascontiguousarray(full.cpu().numpy()[:, :77]))
    assert np.array_equal(sse.view(np.uint32), best.view(np.uint32)) and np.array_equal(cfg.view(np.uint64), arg)


@pytest.mark.parametrize("count,k", [(1, 1), (5, 8), (4096, 1024), (4097, 64), (100000, 1024), (1 << 20, 1024), (300000, 2048)])
def test_topk_matches_ordering_rule(cuda, count, k):
    rng = np.random.default_rng(count + k)
    scores = noisy_scores(rng, (count,))
    idx, val = R.topk(torch.tensor(scores, device="cuda"), k)
    idx, val = idx.cpu().numpy(), val.cpu().numpy()
    want = oracle_topk(scores, k)
    assert np.array_equal(idx[: len(want)].view(np.uint64), want)
    assert np.all(idx[len(want):] == -1)
    got_vals = scores[want.astype(np.int64)]
    assert np.array_equal(np.nan_to_num(val[: len(want)], nan=-7), np.nan_to_num(got_vals, nan=-7))


def test_topk_all_invalid_orders_by_index(cuda):
    scores = torch.full((5000,), float("nan"), device="cuda")
    idx, _ = R.topk(scores, 16)
    assert idx.cpu().tolist() == list(range(16))


def oracle_grouped(grid, num_banks, bits, grouping, k):
    systems = grid.shape[0]
    perms = 1 << bits
    groups = systems if grouping == 0 else systems * perms if grouping == 1 else 1
    mse = np.zeros((groups, k), dtype=np.float32)
    idx = np.zeros((groups, k), dtype=np.uint64)
    counts = np.zeros((groups, 3), dtype=np.uint64)
    code = S.oracle().so_grouped_topk(S.fptr(grid), C.c_size_t(systems), C.c_size_t(num_banks), C.c_uint32(bits),
                                      C.c_uint32(grouping), C.c_size_t(k), S.fptr(mse), idx.ctypes.data_as(S.U64P),
                                      counts.ctypes.data_as(S.U64P))
    assert code == 0
    return mse, idx, counts


@pytest.mark.parametrize("grouping", [0, 1, 2])
@pytest.mark.parametrize("systems,num_banks,bits,k", [(1, 1, 0, 1), (7, 13, 3, 4), (5, 300, 2, 256), (40, 3, 1, 9)])
def test_grouped_topk_matches_the_reference_rule(cuda, grouping, systems, num_banks, bits, k):
    rng = np.random.default_rng(systems * 1000 + num_banks * 10 + bits + grouping)
    grid = noisy_scores(rng, (systems, num_banks << bits))
    flat = grid.reshape(-1)
    flat[rng.integers(0, flat.size, flat.size // 20 + 1)] = np.float32(3.402823466e38)     # FLT_MAX is not a score
    grid[0, :] = np.nan                                                                   # a system with no valid score
    mse, idx, counts = R.grouped_topk(torch.tensor(grid, device="cuda"), systems, num_banks, bits, grouping, k)
    want_mse, want_idx, want_counts = oracle_grouped(grid, num_banks, bits, grouping, k)
    assert np.array_equal(idx.cpu().numpy().view(np.uint64), want_idx)
    assert np.array_equal(mse.cpu().numpy().view(np.uint32), want_mse.view(np.uint32))     # original bits, -0 included
    assert np.array_equal(counts.cpu().numpy().view(np.uint64), want_counts)
