"""The allocation-free top-k entry point against the allocating one.

secant_b200_topk_static() exists for hosts that cannot let the library allocate device
memory (their own pool owns all of it, or their scoring loop must never pay for an
allocation).  It keeps its intermediate keys in a fixed array inside the library, shared by
every call, so the test runs it twice in a row on different inputs: the second call must
not be disturbed by what the first one left behind.  Index work, so results must be
identical to secant_b200_topk().  This file sorts last on purpose: a run that stops at the
first failure has then already executed every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from secant_b200 import abi

pytestmark = pytest.mark.gpu


def run_topk(entry, scores, k):
    idx = torch.full((k,), -5, dtype=torch.int64, device=scores.device)
    val = torch.full((k,), -5.0, dtype=torch.float32, device=scores.device)
    code = entry(scores.data_ptr(), scores.numel(), k, idx.data_ptr(), val.data_ptr(), C.c_void_p(0))
    torch.cuda.synchronize()
    return code, idx.cpu().numpy(), val.cpu().numpy()


def make_scores(seed, count):
    rng = np.random.default_rng(seed)
    s = (rng.random(count, dtype=np.float32) * 100).astype(np.float32)
    s[rng.integers(0, count, count // 7 + 1)] = np.nan
    s[rng.integers(0, count, count // 11 + 1)] = np.float32(3.25)   # ties
    s[rng.integers(0, count, count // 23 + 1)] = -2.0
    return torch.tensor(s, device="cuda")


def test_static_scratch_topk_matches_allocating_topk_twice_in_a_row(cuda):
    lib = abi.load()
    # first call: the largest supported problem, fills the whole shared array
    # second call: a smaller, different problem that reuses the now dirty array
    for seed, count, k in ((1, 1 << 20, 1024), (2, 70001, 257)):
        scores = make_scores(seed, count)
        code_a, idx_a, val_a = run_topk(lib.secant_b200_topk, scores, k)
        code_s, idx_s, val_s = run_topk(lib.secant_b200_topk_static, scores, k)
        assert code_a == 0 and code_s == 0
        assert np.array_equal(idx_s, idx_a)
        assert np.array_equal(val_s.view(np.uint32), val_a.view(np.uint32))
        assert idx_s[0] >= 0 and (val_s[:-1] <= val_s[1:]).all()


def test_static_scratch_topk_rejects_sizes_beyond_its_array(cuda):
    lib = abi.load()
    scores = make_scores(3, 4096)
    out = torch.zeros(2048, dtype=torch.int64, device="cuda")
    too_many = lib.secant_b200_topk_static(scores.data_ptr(), (1 << 20) + 1, 16, out.data_ptr(), 0, C.c_void_p(0))
    too_wide = lib.secant_b200_topk_static(scores.data_ptr(), 4096, 1025, out.data_ptr(), 0, C.c_void_p(0))
    assert too_many == abi.ERROR_INSUFFICIENT_BUFFER and too_wide == abi.ERROR_INSUFFICIENT_BUFFER
    assert lib.secant_b200_topk_static(0, 10, 1, out.data_ptr(), 0, C.c_void_p(0)) == abi.ERROR_INVALID_VALUE
