"""The compiled-topology comparator (tests/comparator.py) must compute what the oracle
computes, otherwise its timing means nothing: NVRTC-compiled expression code in the reference's
kernel layout against the float64-accumulated oracle sums, toggles and affine leaves included."""
import numpy as np
import pytest
import torch

import parity
import support as S
import comparator as K
from secant_b200 import programs as P


def test_generated_source_matches_reference_layout_rules():
    pop = P.random_population(5, 10, 24, 3, 4, 1.0, toggle_bits=2)
    source, kernels = K.generate_source(pop, 0, 10, 4, 3, 4, 2, 32, 64)
    assert kernels == 3 and source.count("__global__") == 3
    assert "tile[160]" in source and "secant_compiled_toggle_sse_002" in source


@pytest.mark.gpu
def test_compiled_topology_against_the_oracle(cuda):
    bits, nb, rows = 2, 5, 300
    pop = P.random_population(41, 21, 32, 4, 6, 2.0, toggle_bits=bits)
    x = np.stack([P.uniform(42, c, rows, -2, 2) for c in range(4)])
    y = np.stack([P.normal(43, t, rows) for t in range(2)])
    banks = np.stack([P.normal(44, b, 6) for b in range(nb)])
    _, _, want64 = S.oracle_toggle_sse(pop, x, y, banks, 6, bits)
    slack = S.sse_slack(pop, x, y, banks, 6, bits)
    dev = lambda a: torch.tensor(np.ascontiguousarray(a), device="cuda")
    compiled = K.CompiledPopulation(pop, 4, 6, 2, num_kernels=2, asts_per_kernel=4, tile_rows=32, threads_per_block=64,
                                    fast_math=False)
    assert len(compiled.modules) == 3 and compiled.compile_seconds > 0
    out = torch.zeros((21, 2, nb << bits), device="cuda")
    launches = compiled.score(dev(x), dev(y), dev(banks), nb, bits, out)
    torch.cuda.synchronize()
    compiled.close()
    assert launches == 6
    assert not parity.sse_mismatches(out.cpu().numpy(), want64, slack).any()
