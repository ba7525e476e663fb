"""Batch sharding across GPUs: one process per GPU, weights replicated, no collective on the
hot path; the only exchange is one gather of the logits after the last layer.

The reference has no working multi-GPU form of this path (its ``nn.DataParallel`` wrapper,
pytorch/imagenet.py:270-275, would make every replica read packed weights that live on cuda:0,
pytorch/deepshift/utils.py:54-58 and kernels.py:70).  Inference is independent per image, so the
batch is simply split.
"""
import os

import torch
import torch.distributed as dist


def shard_bounds(total, world_size, rank):
    """[begin, end) of the images rank `rank` owns out of `total`: contiguous, sizes differ by at
    most one, earlier ranks take the remainder."""
    if world_size < 1 or not (0 <= rank < world_size) or total < 0:
        raise ValueError("bad shard request: total=%d world_size=%d rank=%d" % (total, world_size, rank))
    base, rem = divmod(total, world_size)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def init_from_env(backend=None, timeout_s=180):
    """Joins the process group described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT (as
    torchrun sets them).  Returns (rank, world_size, local_rank); a single process needs no group.
    ``timeout_s``: how long a collective waits for a rank that never arrives before it fails (the
    default of the backends is ten minutes; inference steps take milliseconds)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(local)
        import datetime
        dist.init_process_group(backend=backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s))
    return rank, world, local


def gather_logits(local_logits, world_size=None):
    """All ranks receive the logits of all shards, concatenated in rank order.  Shards may differ
    in size by one image (shard_bounds); they are padded to a common size for the collective."""
    if world_size is None:
        world_size = dist.get_world_size() if dist.is_initialized() else 1
    if world_size == 1:
        return local_logits
    n = torch.tensor([local_logits.shape[0]], dtype=torch.int64, device=local_logits.device)
    sizes = [torch.zeros_like(n) for _ in range(world_size)]
    dist.all_gather(sizes, n)
    sizes = [int(s.item()) for s in sizes]
    m = max(sizes)
    padded = local_logits
    if local_logits.shape[0] < m:
        pad = torch.zeros((m - local_logits.shape[0],) + tuple(local_logits.shape[1:]),
                          dtype=local_logits.dtype, device=local_logits.device)
        padded = torch.cat([local_logits, pad], 0)
    parts = [torch.empty_like(padded) for _ in range(world_size)]
    dist.all_gather(parts, padded.contiguous())
    return torch.cat([p[:s] for p, s in zip(parts, sizes)], 0)


def gather_logits_equal(local_logits, out=None):
    """Same for equal shard sizes (the benchmark's weak scaling): one all_gather into `out`."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return local_logits
    world = dist.get_world_size()
    if out is None:
        out = torch.empty((world * local_logits.shape[0],) + tuple(local_logits.shape[1:]),
                          dtype=local_logits.dtype, device=local_logits.device)
    dist.all_gather_into_tensor(out, local_logits.contiguous())
    return out
