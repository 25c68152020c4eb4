"""Population sharding across ranks: contiguous program blocks, one all-gather of per-program best
scores, the same deterministic top-k on every rank.

The reference has no collective anywhere (its multi-GPU runtime merges on the host,
projects/odezza/runtime/README.md:139-161); the ordering rule is the reference's: valid scores
(finite and >= 0) before invalid ones, then score ascending, then index ascending
(projects/odezza/core/o_score_reduce.cu:36-39, projects/secant-sr/secant_sr.h:68-76).

`Combine` is the one implementation of the combine step: the benchmark, the two-GPU test and the
two-rank CPU test all run it.  What differs between them is passed in: the process group backend
(NCCL or gloo) and the two reductions (`DeviceReductions`: this library's kernels through the
C-ABI; the CPU test passes the checker's restatements of the same rules).
"""
import torch

SCORE_BYTES = 24   # SecantB200Score: float sse, uint32 reserved, uint64 configuration, uint64 valid configurations


def program_block(num_programs, rank, world):
    """[lo, hi) of the contiguous block owned by `rank`; blocks differ by at most one program."""
    base, extra = divmod(num_programs, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def record_fields(records):
    """(sse float32 view, configuration int64 view, valid int64 view) of a buffer of 24-byte records."""
    n = records.numel() // SCORE_BYTES
    sse = records.view(torch.float32).view(n, 6)[:, 0]
    words = records.view(torch.int64).view(n, 3)
    return sse, words[:, 1], words[:, 2]


class DeviceReductions:
    """The library's own reducers (secant_b200_best_config, secant_b200_topk) on torch's current stream."""

    @staticmethod
    def best_config(grid, out):
        from . import runner
        return runner.best_config(grid, out=out)

    @staticmethod
    def topk(keys, k):
        from . import runner
        return runner.topk(keys, k)[0]


class Combine:
    """Best configuration per program, one all-gather of the records, the same top-k everywhere.

    Every rank holds `slots` programs (a rank with a shorter block pads: the records of the padding
    are the "no valid score" record, which never ranks).  Global program index = position in the
    gathered buffer mapped through `program_block`.  The best-configuration reducer writes straight
    into the all-gather send buffer; nothing passes through the host."""

    def __init__(self, num_programs, world, rank, k, device, reductions=DeviceReductions, group=None):
        self.num_programs, self.world, self.rank, self.k = num_programs, world, rank, min(k, num_programs)
        self.slots = (num_programs + world - 1) // world
        self.lo, self.hi = program_block(num_programs, rank, world)
        self.reductions, self.group = reductions, group
        self.send = torch.zeros(self.slots * SCORE_BYTES, dtype=torch.uint8, device=device)
        self.recv = torch.zeros(world * self.slots * SCORE_BYTES, dtype=torch.uint8, device=device) if world > 1 else self.send
        sse, cfg, valid = record_fields(self.send)          # padding records: {+inf, UINT64_MAX, 0}
        sse.fill_(float("inf"))
        cfg.fill_(-1)
        valid.fill_(0)
        # position in the gathered buffer -> global program index (-1 for padding)
        index = torch.full((world * self.slots,), -1, dtype=torch.int64)
        for r in range(world):
            lo, hi = program_block(num_programs, r, world)
            index[r * self.slots: r * self.slots + (hi - lo)] = torch.arange(lo, hi)
        self.global_index = index.to(device)

    def __call__(self, grid):
        """grid: this rank's [programs][configurations] scores.  Returns (top-k global program indices,
        the gathered records)."""
        import torch.distributed as dist
        local = self.hi - self.lo
        assert grid.shape[0] == local
        self.reductions.best_config(grid, self.send[: local * SCORE_BYTES])
        if self.world > 1:
            dist.all_gather_into_tensor(self.recv, self.send, group=self.group)
        keys = record_fields(self.recv)[0]
        top = self.reductions.topk(keys, self.k)
        return self.global_index[top], self.recv
