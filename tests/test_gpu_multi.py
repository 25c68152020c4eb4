"""Two ranks on two GPUs: each scores its own block of a population, per-program best scores
are combined with one NCCL all-gather, and both ranks must arrive at the same top-k as a
single-process CPU oracle run of the whole population.  Skipped with fewer than two GPUs."""
import os
import subprocess
import sys
import textwrap

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def test_two_gpu_shards_agree_with_single_process_oracle(tmp_path):
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "rank.py"
    script.write_text(textwrap.dedent(f"""
        import os, sys
        sys.path.insert(0, {repr(os.path.join(ROOT, 'gpu-program-specialization_b200'))})
        sys.path.insert(0, {repr(os.path.join(ROOT, 'tests'))})
        import numpy as np, torch, torch.distributed as dist
        import support as S
        from secant_b200 import abi, programs as P, sharding, runner as R
        rank, world = int(os.environ['RANK']), int(os.environ['WORLD_SIZE'])
        torch.cuda.set_device(rank)
        dev = torch.device('cuda', rank)
        dist.init_process_group('nccl', device_id=dev)
        total, rows, nb, K = 301, 500, 6, 4
        pop = P.random_population(91, total, 24, 3, K, 1.0, ops=P.ARITHMETIC_OPS)
        x = np.stack([P.uniform(92, c, rows, -1, 1) for c in range(3)])
        y = np.stack([P.normal(93, 0, rows)])
        banks = np.stack([P.normal(94, b, K) for b in range(nb)])
        lo, hi = sharding.program_block(total, rank, world)
        mine = pop.subset(range(lo, hi))
        with R.Runner(abi.SHAPE_TOGGLE_SSE, 3, 1, K) as rn:
            grid = rn.toggle_sse(mine, torch.tensor(x, device=dev), torch.tensor(y, device=dev), torch.tensor(banks, device=dev), nb, 0)
        combine = sharding.Combine(total, world, rank, 32, dev)       # the step the benchmark runs
        top, records = combine(grid.view(hi - lo, nb))
        everyone = sharding.record_fields(records)[0][combine.global_index >= 0]
        _, _, want64 = S.oracle_toggle_sse(pop, x, y, banks, K, 0)
        ref_best = np.where(np.isfinite(want64[:, 0, :]), want64[:, 0, :], np.inf).min(axis=1)
        order = sorted(range(total), key=lambda i: (ref_best[i], i))[:32]
        got = top.cpu().tolist()
        gaps_ok = all(abs(ref_best[a] - ref_best[b]) <= 2e-4 * abs(ref_best[b]) + 1e-6 for a, b in zip(got, order) if a != b)
        assert got == order or gaps_ok, (got[:8], order[:8])
        assert np.allclose(everyone.cpu().numpy(), ref_best, rtol=1e-4, atol=1e-6)
        dist.barrier()
        dist.destroy_process_group()
        print('rank', rank, 'ok')
    """))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29621", str(script)],
                         capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, (out.stdout[-1500:], out.stderr[-3000:])
    assert out.stdout.count("ok") == 2
