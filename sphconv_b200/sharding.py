"""Batch sharding across GPUs: scans are independent (a scan never interacts with another one: tiles are
shared across the batch only as a list index, row ids and z_ptr are per-tensor prefix sums,
src/sphconv/rules.cu:72-80,204-227), so rank r of R takes a contiguous slice of the batch, builds its own
SparseConvTensor (its z_ptr starts at 0) and runs the path locally.  Forward needs no collective; training
adds ONE all-reduce over a flat fp32 buffer holding every layer's weight gradient."""
from typing import Iterable, List, Tuple

import torch


def shard_range(n_scans: int, world: int, rank: int) -> Tuple[int, int]:
    """[first, last) scan ids of `rank`; sizes differ by at most one."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("bad world/rank %d/%d" % (world, rank))
    base, extra = divmod(n_scans, world)
    first = rank * base + min(rank, extra)
    return first, first + base + (1 if rank < extra else 0)


def slice_batch(z_idx: torch.Tensor, z_ptr: torch.Tensor, feature: torch.Tensor, first: int, last: int):
    """Scans [first, last) of a range-voxel batch as a self-contained batch (z_ptr re-based to start at 0)."""
    B, H, W = z_ptr.shape
    flat = z_ptr.reshape(B, -1)
    row0 = 0 if first == 0 else int(flat[first - 1, -1])
    row1 = row0 if last == first else int(flat[last - 1, -1])
    zp = (z_ptr[first:last] - row0).contiguous()
    return z_idx[row0:row1].contiguous(), zp, feature[row0:row1].contiguous()


def flatten_grads(params: Iterable[torch.nn.Parameter]) -> Tuple[torch.Tensor, List[torch.nn.Parameter]]:
    """One flat fp32 buffer with every parameter's gradient (zeros where a parameter has none)."""
    plist = [p for p in params if p.requires_grad]
    total = sum(p.numel() for p in plist)
    dev = plist[0].device if plist else torch.device("cpu")
    flat = torch.zeros(total, dtype=torch.float32, device=dev)
    off = 0
    for p in plist:
        if p.grad is not None:
            flat[off:off + p.numel()] = p.grad.reshape(-1).float()
        off += p.numel()
    return flat, plist


def unflatten_grads(flat: torch.Tensor, plist: List[torch.nn.Parameter]) -> None:
    off = 0
    for p in plist:
        g = flat[off:off + p.numel()].reshape(p.shape).to(p.dtype)
        if p.grad is None:
            p.grad = g.clone()
        else:
            p.grad.copy_(g)
        off += p.numel()


def allreduce_gradients(params: Iterable[torch.nn.Parameter], group=None, average: bool = False) -> int:
    """Sum (or average) the gradients of `params` over the process group with a single all-reduce.
    Returns the number of fp32 elements reduced."""
    import torch.distributed as dist
    flat, plist = flatten_grads(params)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
        if average:
            flat /= dist.get_world_size(group)
    unflatten_grads(flat, plist)
    return int(flat.numel())
