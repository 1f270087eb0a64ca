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


class GradBuffer:
    """One flat fp32 buffer that holds the gradient of every parameter of a model, written in place by the
    backward kernels and all-reduced in place with ONE collective.

    The weight-gradient kernels accumulate in fp32 (the reference sums fp32 per-tile partials,
    src/sphconv/rule_conv.cu:483-484,517).  Handing that result to autograd as `.grad` of a bf16/fp16 parameter
    rounds each rank's contribution to 8 or 11 mantissa bits BEFORE the cross-rank sum; here each convolution
    writes its fp32 result straight into its slice of this buffer (the parameter gets no `.grad` from autograd),
    the buffer is summed over the ranks as fp32, and `to_grads()` rounds once at the end.

        gb = GradBuffer(net.parameters())          # attaches a slice to every parameter
        gb.zero(); loss.backward(); gb.all_reduce(); gb.to_grads(); optimizer.step()

    Works with CPU tensors too (host-side tests over gloo)."""

    def __init__(self, params: Iterable[torch.nn.Parameter]):
        self.params = [p for p in params if p.requires_grad]
        total = sum(p.numel() for p in self.params)
        dev = self.params[0].device if self.params else torch.device("cpu")
        self.flat = torch.zeros(total, dtype=torch.float32, device=dev)
        self.views = []
        off = 0
        for p in self.params:
            v = self.flat[off:off + p.numel()].view(p.shape)
            p._sph_master_grad = v          # read by Conv3d.forward / ConvFunction.backward
            self.views.append(v)
            off += p.numel()

    def zero(self) -> None:
        self.flat.zero_()

    def all_reduce(self, group=None, average: bool = False) -> int:
        """Sum (or average) over the process group, in place; returns the number of fp32 elements reduced."""
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group)
            if average:
                self.flat /= dist.get_world_size(group)
        return int(self.flat.numel())

    def absorb_autograd(self) -> None:
        """Adds (and clears) `.grad` of parameters whose gradient came through autograd instead of a kernel that
        writes the buffer (dense layers mixed into the model)."""
        for p, v in zip(self.params, self.views):
            if p.grad is not None:
                v.add_(p.grad.float())
                p.grad = None

    def to_grads(self) -> None:
        """`.grad` of every parameter = its slice, rounded once to the parameter's dtype."""
        for p, v in zip(self.params, self.views):
            if p.grad is None or p.grad.dtype != p.dtype:
                p.grad = v.to(p.dtype)
            else:
                p.grad.copy_(v)

    def detach(self) -> None:
        for p in self.params:
            if hasattr(p, "_sph_master_grad"):
                del p._sph_master_grad


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
