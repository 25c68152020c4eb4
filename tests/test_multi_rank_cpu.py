"""Checks the sharding arithmetic used by the multi-GPU path, run as two
gloo ranks on the CPU: contiguous program blocks, an all-gather of per-program best scores,
and an identical deterministic top-k on every rank (ordering rule of
projects/odezza/core/o_score_reduce.cu:36-39)."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_two_rank_gather_and_topk_agree(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(textwrap.dedent(f"""
        import os, sys
        sys.path.insert(0, {repr(os.path.join(ROOT, 'gpu-program-specialization_b200'))})
        import numpy as np, torch, torch.distributed as dist
        from secant_b200 import sharding
        dist.init_process_group('gloo')
        rank, world = dist.get_rank(), dist.get_world_size()
        P = 1001
        rng = np.random.default_rng(5)
        scores = rng.random(P).astype(np.float32)
        scores[::17] = np.nan
        scores[3] = scores[900] = 0.0
        lo, hi = sharding.program_block(P, rank, world)
        local = torch.tensor(scores[lo:hi])
        gathered = sharding.all_gather_scores(local, P, world)
        assert np.array_equal(np.nan_to_num(gathered.numpy(), nan=-1), np.nan_to_num(scores, nan=-1))
        top = sharding.topk_indices(gathered, 64)
        ref = sorted([i for i in range(P) if np.isfinite(scores[i]) and scores[i] >= 0], key=lambda i: (scores[i], i))[:64]
        assert top.tolist() == ref, (top.tolist()[:5], ref[:5])
        dist.barrier()
        print('rank', rank, 'ok')
    """))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29611", str(script)],
                         capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    assert out.stdout.count("ok") == 2
