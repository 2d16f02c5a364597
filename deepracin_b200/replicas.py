"""Batch-sharded replicas: the multi-GPU story of this path.

Images are independent (the reference itself processes one image per dR_apply), so N GPUs run N
independent replicas of the prepared graph, each on a contiguous slice of the global batch; there is
no exchange step and therefore no collective on the data path.  torch.distributed is only plumbing:
a barrier around timed regions, a max over ranks of device times, and an optional gather of the
per-image outputs to rank 0 ("outputs gathered by host copies").  Works with the nccl backend on
GPUs and with gloo on CPU (which is how the host-side logic is tested).
"""
import os

import numpy as np


def world():
    """(rank, world_size, local_rank) from the launcher's environment (torchrun sets these)."""
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def shard_bounds(global_batch, world_size, rank):
    """Contiguous image-major slice [lo, hi) of the global batch owned by `rank`; sizes differ by at most one."""
    if world_size < 1 or not 0 <= rank < world_size or global_batch < 0:
        raise ValueError("bad shard request")
    base, extra = divmod(global_batch, world_size)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard(images, world_size, rank):
    lo, hi = shard_bounds(images.shape[0], world_size, rank)
    return images[lo:hi]


def init(backend=None, device=None):
    """Initialises torch.distributed when WORLD_SIZE > 1; returns the module or None for a single process."""
    rank, size, local = world()
    if size <= 1:
        return None
    import torch
    import torch.distributed as dist
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if dist.is_initialized():
        return dist
    if backend == "nccl":
        # NCCL prints its version banner on stdout at NCCL_DEBUG=VERSION; callers print machine-read lines there
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"
        torch.cuda.set_device(local if device is None else device)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local if device is None else device))
    else:
        dist.init_process_group(backend)
    return dist


def barrier(dist):
    if dist is not None:
        dist.barrier()


def max_over_ranks(dist, value, cuda=False):
    if dist is None:
        return float(value)
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64, device="cuda" if cuda else "cpu")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gather_outputs(dist, local_out, global_batch, cuda=False):
    """Per-image outputs of every replica, concatenated in global image order on every rank.
    local_out: numpy [local_batch, ...]; shards may be ragged."""
    if dist is None:
        return np.asarray(local_out)
    import torch
    rank, size = dist.get_rank(), dist.get_world_size()
    sizes = [shard_bounds(global_batch, size, r)[1] - shard_bounds(global_batch, size, r)[0] for r in range(size)]
    width = int(np.prod(local_out.shape[1:])) if local_out.ndim > 1 else 1
    pad = max(sizes)
    dev = "cuda" if cuda else "cpu"
    buf = torch.zeros(pad, width, dtype=torch.float32, device=dev)
    buf[:local_out.shape[0]] = torch.from_numpy(np.ascontiguousarray(local_out, dtype=np.float32).reshape(local_out.shape[0], width)).to(dev)
    parts = [torch.empty_like(buf) for _ in range(size)]
    dist.all_gather(parts, buf)
    out = np.concatenate([p[:n].cpu().numpy() for p, n in zip(parts, sizes)], axis=0)
    return out.reshape((global_batch,) + tuple(local_out.shape[1:]))


def finish(dist):
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
