"""The combine step of the multi-GPU path, run as two gloo ranks on the CPU: the same
`sharding.Combine` the benchmark and the two-GPU test run (best configuration per program written
into the send buffer as 24-byte records, one all-gather, one top-k, global indices through the
block layout), with the process group on gloo and the two reductions supplied by the CPU checker's
restatements of the same rules (projects/secant-sr/toggle/src/cpu.c:45-67,
projects/odezza/core/o_score_reduce.cu:36-39)."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_two_rank_combine_agrees_with_a_single_process(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(textwrap.dedent(f"""
        import ctypes as C, os, sys
        sys.path.insert(0, {repr(os.path.join(ROOT, 'gpu-program-specialization_b200'))})
        sys.path.insert(0, {repr(os.path.join(ROOT, 'tests'))})
        import numpy as np, torch, torch.distributed as dist
        import support as S
        from secant_b200 import sharding

        class CheckerReductions:
            @staticmethod
            def best_config(grid, out):
                g = np.ascontiguousarray(grid.numpy(), dtype=np.float32)
                a, c = g.shape
                best = np.zeros(a, dtype=np.float32); cfg = np.zeros(a, dtype=np.uint64); valid = np.zeros(a, dtype=np.uint64)
                S.oracle().so_best_config(S.fptr(g), C.c_size_t(a), C.c_size_t(c), C.c_size_t(c), S.fptr(best),
                                          cfg.ctypes.data_as(S.U64P), valid.ctypes.data_as(S.U64P))
                sse, conf, count = sharding.record_fields(out)
                sse.copy_(torch.from_numpy(best)); conf.copy_(torch.from_numpy(cfg.view(np.int64))); count.copy_(torch.from_numpy(valid.view(np.int64)))
                return out
            @staticmethod
            def topk(keys, k):
                flat = np.ascontiguousarray(keys.numpy(), dtype=np.float32)
                idx = np.zeros(k, dtype=np.uint64)
                S.oracle().so_topk.restype = C.c_size_t
                S.oracle().so_topk(S.fptr(flat), C.c_size_t(flat.size), C.c_size_t(k), idx.ctypes.data_as(S.U64P))
                return torch.from_numpy(idx.view(np.int64))

        dist.init_process_group('gloo')
        rank, world = dist.get_rank(), dist.get_world_size()
        P, configs, k = 1001, 7, 64                                  # uneven blocks: 501 and 500 programs
        rng = np.random.default_rng(5)
        grid = rng.random((P, configs)).astype(np.float32)
        grid[::17] = np.nan                                           # programs without a valid score
        grid[3, 2] = grid[900, 5] = 0.0                               # a tie for the best score
        grid[40, :] = -1.0                                            # negative scores are invalid
        lo, hi = sharding.program_block(P, rank, world)
        combine = sharding.Combine(P, world, rank, k, torch.device('cpu'), reductions=CheckerReductions)
        top, records = combine(torch.from_numpy(grid[lo:hi]))
        valid = np.isfinite(grid) & (grid >= 0)
        best = np.where(valid, grid, np.inf).min(axis=1)
        want = sorted([i for i in range(P) if np.isfinite(best[i])], key=lambda i: (best[i], i))[:k]
        assert top.tolist() == want, (top.tolist()[:6], want[:6])
        assert want[:2] == [3, 900]
        sse, cfg, count = sharding.record_fields(records)
        own = combine.global_index >= 0
        assert np.array_equal(sse[own].numpy(), best)                 # every rank holds every program's record
        assert int(cfg[own][3]) == 2 and int(cfg[own][900]) == 5 and int(cfg[own][17]) == -1
        assert np.array_equal(count[own].numpy(), valid.sum(axis=1))
        dist.barrier()
        print('rank', rank, 'ok')
    """))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29611", str(script)],
                         capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0, (out.stdout[-1500:], out.stderr[-2500:])
    assert out.stdout.count("ok") == 2
