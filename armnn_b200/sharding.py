"""Batch sharding across the GPUs of one box: one process and one LoadedNetwork per GPU, contiguous slices of
batch rows, weights replicated, no collective on the data path (every operator of the hot path is independent
across batch rows).  The only cross-rank step is the optional gather of the output slices on the host side."""
import os


def shard_range(global_batch, world_size, rank):
    """Rows [start, stop) of rank `rank`: contiguous, sizes differ by at most one, union = [0, global_batch)."""
    if not (0 <= rank < world_size):
        raise ValueError("rank %d outside world of size %d" % (rank, world_size))
    base, extra = divmod(global_batch, world_size)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def env_rank():
    """(rank, local_rank, world_size) from the torchrun environment (1 process = 1 GPU)."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")))


def gather_rows(local_rows, global_batch, group=None):
    """All ranks receive the full [global_batch, ...] tensor assembled from every rank's slice.  Host-side
    convenience for callers that want the whole result in one place; not used inside the timed path."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    sizes = [b - a for a, b in (shard_range(global_batch, world, r) for r in range(world))]
    most = max(sizes)
    # all_gather wants equal shapes: pad ragged slices to the largest one, trim after the exchange
    padded = torch.zeros((most,) + tuple(local_rows.shape[1:]), dtype=local_rows.dtype, device=local_rows.device)
    padded[:local_rows.shape[0]] = local_rows
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p[:n] for p, n in zip(parts, sizes)], dim=0)
