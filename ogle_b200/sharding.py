"""Image sharding across the GPUs of one box: host-side logic only.

The hot path has no cross-image coupling, so N GPUs run N independent replicas
(one process, session, stream and CUDA graph each). Inputs are split by image
index; detections are gathered on the host. Nothing here touches the data path
on the device: no NCCL collective, no peer access.
"""
import torch.distributed as dist


def shard_range(n_images, rank, world):
    """Contiguous block [lo, hi) of image indices owned by `rank`; sizes differ by at most one."""
    base, rem = divmod(n_images, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def gather_detections(local, lo, group=None, dst=0):
    """local: list of per-image detection records for images lo, lo+1, ... of this rank.
    Returns on `dst` the list for ALL images in image order (None elsewhere). Uses the
    object gather of the given (CPU-capable, e.g. gloo) process group."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    payload = (lo, local)
    out = [None] * world if rank == dst else None
    dist.gather_object(payload, out, dst=dst, group=group)
    if rank != dst:
        return None
    merged = {}
    for start, items in out:
        for i, item in enumerate(items):
            if start + i in merged:
                raise ValueError(f"image {start + i} reported by two ranks")
            merged[start + i] = item
    return [merged[i] for i in sorted(merged)]


def max_over_ranks(value, group=None):
    """Slowest rank's value (timings are reported as the max over ranks)."""
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
