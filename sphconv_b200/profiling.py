"""Optional per-section CUDA-event timing on the current stream (off by default, a few microseconds per section)."""
import contextlib

import torch

_active = False
pair_counts = None        # dict name -> pairs: while set, count_pairs() accumulates into it (synchronising)
current_tag = ""          # name of the layer whose ops are being issued (set by Conv3d.forward)
_records = []   # (name, start_event, stop_event, meta)


def enable(flag=True):
    global _active
    _active = bool(flag)
    if not flag:
        _records.clear()


def is_active():
    return _active


@contextlib.contextmanager
def section(name, **meta):
    """Times the GPU work enqueued inside the block on the current stream when profiling is enabled."""
    if not _active:
        yield
        return
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    start.record()
    try:
        yield
    finally:
        stop.record()
        _records.append((name, start, stop, meta))


def collect(reset=True):
    """[(name, milliseconds, meta)] of every finished section; synchronises the device."""
    torch.cuda.synchronize()
    out = [(n, a.elapsed_time(b), m) for n, a, b, m in _records]
    if reset:
        _records.clear()
    return out


def count_pairs(name, rules):
    """When pair counting is switched on, add the number of (in,out) pairs of this rule set to pair_counts[name].
    Counts at once and keeps no reference to the (possibly GB-sized) rule tensors."""
    if pair_counts is None:
        return
    tb = rules if not isinstance(rules, torch.Tensor) else getattr(rules, "_sph", None)
    if tb is None:
        return
    n = int((tb.nbr >= 0).sum().item())
    pair_counts[name] = pair_counts.get(name, 0) + n
