"""Host <-> device pipelining around a per-batch function (no counterpart in the reference, which leaves
copies to the caller).

A scan batch arrives in pinned host memory and its result is wanted back in host memory.  Done on one stream
the three phases serialise: copy in, compute, copy out.  ``ScanPipeline`` puts the copies on two side streams
and keeps ``depth`` batches in flight, so the copy-out of batch i and the copy-in of batch i+2 run on the copy
engines while batch i+1 computes.  The compute itself stays on the caller's current stream and is unchanged.

    pipe = ScanPipeline(lambda f, zi, zp: {"feature": net(SparseConvTensor(f, shape, B, z_idx=zi, z_ptr=zp)).feature},
                        device="cuda:0")
    t0 = pipe.submit((feature0, z_idx0, z_ptr0))        # pinned host tensors
    t1 = pipe.submit((feature1, z_idx1, z_ptr1))
    out0 = pipe.result(t0)                              # dict of host tensors; valid until the slot is reused
"""
from typing import Callable, Dict, Sequence

import torch


class _Slot:
    def __init__(self):
        self.dev_in = []        # device staging buffers, one per input, grown on demand
        self.host_out = {}      # pinned host buffers by output name
        self.views = None       # host views of the last result
        self.h2d_done = torch.cuda.Event()
        self.compute_done = torch.cuda.Event()
        self.d2h_done = torch.cuda.Event()
        self.pending = False    # a result has been produced and not fetched yet
        self.used = False


def bind_host_to_device(device_index: int):
    """Restricts this process to the CPUs that sit next to GPU `device_index` (NVML's CPU affinity of the device), so
    that the pinned host buffers allocated afterwards land in that GPU's NUMA node: with one process per GPU on a
    two-socket host, results copied out by eight GPUs otherwise all pour into the memory of whichever node the
    processes happened to start on.  Call it once, before the first pin_memory().  Returns the CPU list it bound to, or
    None when NVML / the affinity call is unavailable (nothing is changed then)."""
    import os
    try:
        import pynvml
        pynvml.nvmlInit()
        uuid = str(torch.cuda.get_device_properties(device_index).uuid)
        if not uuid.startswith("GPU-"):
            uuid = "GPU-" + uuid
        handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode() if isinstance(uuid, str) else uuid)
        n_cpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (n_cpu + 63) // 64)
        cpus = [i for i in range(n_cpu) if (int(words[i // 64]) >> (i % 64)) & 1]
        allowed = sorted(set(cpus) & set(os.sched_getaffinity(0)))
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return allowed
    except Exception:
        return None


def _grow(n):
    return int(n * 1.25) + 16


class ScanPipeline:
    def __init__(self, run_fn: Callable[..., Dict[str, torch.Tensor]], device="cuda", depth: int = 2):
        if depth < 1:
            raise ValueError("depth must be at least 1")
        self.run_fn = run_fn
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("ScanPipeline needs a CUDA device")
        self.depth = depth
        self.copy_in = torch.cuda.Stream(self.device)
        self.copy_out = torch.cuda.Stream(self.device)
        self.slots = [_Slot() for _ in range(depth)]
        self.count = 0
        self.h2d_bytes = 0      # of the last submit
        self.d2h_bytes = 0

    def _stage_in(self, slot: _Slot, host: Sequence[torch.Tensor]):
        while len(slot.dev_in) < len(host):
            slot.dev_in.append(None)
        views = []
        nbytes = 0
        fresh = False
        for i, h in enumerate(host):
            if not h.is_pinned():
                raise RuntimeError("ScanPipeline inputs must be pinned host tensors (tensor.pin_memory())")
            buf = slot.dev_in[i]
            rows = h.shape[0] if h.dim() > 0 else 1
            if buf is None or buf.dtype != h.dtype or buf.shape[1:] != h.shape[1:] or buf.shape[0] < rows:
                buf = torch.empty((_grow(rows),) + tuple(h.shape[1:]), dtype=h.dtype, device=self.device)
                buf.record_stream(self.copy_in)     # written by the copy-in stream: not to be recycled under it
                slot.dev_in[i] = buf
                fresh = True
            views.append(buf[:rows] if h.dim() > 0 else buf[0])
            nbytes += h.numel() * h.element_size()
        self.h2d_bytes = nbytes
        return views, fresh

    def submit(self, host_inputs: Sequence[torch.Tensor]) -> int:
        """Enqueue copy-in, compute and copy-out of one batch; returns a ticket for ``result``."""
        ticket = self.count
        slot = self.slots[ticket % self.depth]
        if slot.pending:
            raise RuntimeError("ScanPipeline: fetch result(%d) before submitting batch %d (depth %d)"
                               % (ticket - self.depth, ticket, self.depth))
        compute = torch.cuda.current_stream(self.device)
        views, fresh = self._stage_in(slot, host_inputs)   # (re)allocation happens on the compute stream's pool
        with torch.cuda.stream(self.copy_in):
            if slot.used:
                self.copy_in.wait_event(slot.compute_done)   # the previous batch of this slot has read its inputs
            if fresh or not slot.used:
                # A new staging buffer comes from the compute stream's pool: the block may have just been freed by
                # work that is still running there (the other batch in flight), so the copy must not start before
                # everything enqueued on the compute stream so far has finished.
                self.copy_in.wait_stream(compute)
            for v, h in zip(views, host_inputs):
                v.copy_(h, non_blocking=True)
            slot.h2d_done.record(self.copy_in)
        compute.wait_event(slot.h2d_done)
        outs = self.run_fn(*views)
        slot.compute_done.record(compute)
        host_views = {}
        nbytes = 0
        with torch.cuda.stream(self.copy_out):
            self.copy_out.wait_event(slot.compute_done)
            for name, t in outs.items():
                rows = t.shape[0] if t.dim() > 0 else 1
                buf = slot.host_out.get(name)
                if buf is None or buf.dtype != t.dtype or buf.shape[1:] != t.shape[1:] or buf.shape[0] < rows:
                    buf = torch.empty((_grow(rows),) + tuple(t.shape[1:]), dtype=t.dtype).pin_memory()
                    slot.host_out[name] = buf
                hv = buf[:rows] if t.dim() > 0 else buf[0]
                hv.copy_(t, non_blocking=True)
                t.record_stream(self.copy_out)               # keep the allocator from reusing it under the copy
                host_views[name] = hv
                nbytes += t.numel() * t.element_size()
            slot.d2h_done.record(self.copy_out)
        self.d2h_bytes = nbytes
        slot.views = host_views
        slot.pending = True
        slot.used = True
        self.count += 1
        return ticket

    def result(self, ticket: int) -> Dict[str, torch.Tensor]:
        """Host tensors of batch ``ticket`` (blocks until its copy-out has finished).  The tensors are views of
        the slot's pinned buffers and are overwritten when the slot is reused ``depth`` submits later."""
        if ticket < 0 or ticket >= self.count or ticket < self.count - self.depth:
            raise RuntimeError("ScanPipeline: ticket %d is not in flight" % ticket)
        slot = self.slots[ticket % self.depth]
        if not slot.pending:
            raise RuntimeError("ScanPipeline: result(%d) was already fetched" % ticket)
        slot.d2h_done.synchronize()
        slot.pending = False
        return slot.views

    def drain(self):
        """Wait for everything in flight (results stay fetchable)."""
        torch.cuda.current_stream(self.device).wait_stream(self.copy_out)
        self.copy_out.synchronize()
