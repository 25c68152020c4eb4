"""Population sharding across ranks: contiguous program blocks, one all-gather of
per-program scores, the same deterministic top-k on every rank.

The reference has no collective anywhere (its multi-GPU runtime merges on the host,
projects/odezza/runtime/README.md:139-161); the ordering rule is the reference's:
valid scores (finite and >= 0) before invalid ones, then score ascending, then index
ascending (projects/odezza/core/o_score_reduce.cu:36-39, projects/secant-sr/secant_sr.h:68-76).
"""
import torch


def program_block(num_programs, rank, world):
    """[lo, hi) of the contiguous block owned by `rank`; blocks differ by at most one program."""
    base, extra = divmod(num_programs, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def all_gather_scores(local, num_programs, world):
    """Gathers equally padded blocks with one collective and strips the padding."""
    import torch.distributed as dist
    width = (num_programs + world - 1) // world
    send = torch.full((width,), float("nan"), dtype=local.dtype, device=local.device)
    send[: local.numel()] = local
    recv = torch.empty((world * width,), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(recv, send)
    parts = []
    for r in range(world):
        lo, hi = program_block(num_programs, r, world)
        parts.append(recv[r * width: r * width + (hi - lo)])
    return torch.cat(parts)


def topk_indices(scores, k):
    """Indices of the k best scores under (valid first, score ascending, index ascending)."""
    valid = torch.isfinite(scores) & (scores >= 0)
    key = torch.where(valid, scores, torch.full_like(scores, float("inf")))
    order = torch.sort(key, stable=True).indices      # stable sort keeps index order inside ties
    order = order[valid[order]]
    return order[:k]
