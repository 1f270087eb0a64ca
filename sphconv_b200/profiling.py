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


_open = []                # stop events of the sections currently open on the current stream (innermost last)
current_rule_tag = ""     # name of the rule set being generated (set by Conv3d.forward), for side-stream sections


@contextlib.contextmanager
def section(name, stream=None, **meta):
    """Times the GPU work enqueued inside the block when profiling is enabled: on the current stream, or on
    `stream` (work a layer puts on a side stream).  A section on the current stream ends where `mark_stop()` was
    called inside it, else at the end of the block."""
    if not _active:
        yield
        return
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    if stream is not None:
        start.record(stream)
        try:
            yield
        finally:
            stop.record(stream)
            _records.append((name, start, stop, meta))
        return
    start.record()
    state = [stop, False]
    _open.append(state)
    try:
        yield
    finally:
        _open.pop()
        if not state[1]:
            stop.record()
        _records.append((name, start, stop, meta))


def mark_stop():
    """Ends the innermost open section here (its kernels are enqueued; what follows in the block is a wait on
    other streams' work that should not count as the section's time)."""
    if _active and _open and not _open[-1][1]:
        _open[-1][0].record()
        _open[-1][1] = True


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
