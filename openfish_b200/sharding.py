"""Multi-GPU plumbing: chunks are independent, so a batch is split by chunk index with no
data-path collective (the reference's intended multi-GPU use is one host thread per device,
src/main.c:23,207-212).  torch.distributed only carries the timing reduction and, for tests,
the gather of results."""
import numpy as np


def shard_range(n_chunks, rank, world):
    """Contiguous chunk range [lo, hi) of `rank`; earlier ranks take the remainder (the same
    split the reference's CPU decoder uses over threads, src/decode_cpu.c:278-292)."""
    each, extra = divmod(n_chunks, world)
    lo = rank * each + min(rank, extra)
    return lo, lo + each + (1 if rank < extra else 0)


def slice_scores(scores_TNC, lo, hi):
    """This rank's [T][hi-lo][C] tensor (a copy: a shard must be contiguous)."""
    s = scores_TNC[:, lo:hi, :]
    return s.contiguous() if hasattr(s, "contiguous") else np.ascontiguousarray(s)


def max_over_ranks(value, device=None):
    """Max of a per-rank float over all ranks (1 process: the value itself)."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device or "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value, device=None):
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device or "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def gather_rows(rows, n_chunks):
    """Concatenate per-rank uint8 result rows [n_local][T] on rank 0 in chunk order
    (None on other ranks)."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return np.asarray(rows)
    world, rank = dist.get_world_size(), dist.get_rank()
    T = rows.shape[1]
    most = max(shard_range(n_chunks, r, world)[1] - shard_range(n_chunks, r, world)[0] for r in range(world))
    pad = torch.zeros((most, T), dtype=torch.uint8)
    pad[: rows.shape[0]] = torch.as_tensor(np.asarray(rows))
    out = [torch.zeros_like(pad) for _ in range(world)] if rank == 0 else None
    dist.gather(pad, out, dst=0)
    if rank != 0:
        return None
    parts = []
    for r in range(world):
        lo, hi = shard_range(n_chunks, r, world)
        parts.append(out[r][: hi - lo].numpy())
    return np.concatenate(parts, 0)
