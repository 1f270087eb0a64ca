"""ScanPipeline (host -> device -> host with copies on side streams): every batch's result must equal the result
of running the same batch directly, for batches of different sizes pushed back to back through two slots."""
import pytest
import torch

import sphconv_b200 as sphconv
from sphconv_b200 import synthetic
from sphconv_b200.encoder import build_encoder8

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SMALL = dict(id=3, B=2, shape=[16, 32, 64], occ=0.9, nbins="uniform", nmax=4, depth="lognormal", C=4)


def _host_batch(first_scan, B):
    b = synthetic.make_batch(SMALL, batch=B, first_scan=first_scan)
    return (torch.as_tensor(b["feature"]).half().pin_memory(), torch.as_tensor(b["z_idx"]).pin_memory(),
            torch.as_tensor(b["z_ptr"]).pin_memory()), b["shape"]


def test_pipeline_matches_direct_calls():
    net = build_encoder8(dtype=torch.float16, device=DEV).eval()
    B = 2
    batches = [_host_batch(s, B) for s in (0, 7, 3, 11, 5)]
    shape = batches[0][1]

    def run(f, zi, zp):
        y = net(sphconv.SparseConvTensor(f, shape, B, z_idx=zi, z_ptr=zp))
        return {"feature": y.feature, "z_idx": y.z_idx, "z_ptr": y.z_ptr}

    with torch.no_grad():
        direct = []
        for host, _ in batches:
            out = run(*[t.to(DEV) for t in host])
            direct.append({k: v.cpu().clone() for k, v in out.items()})
        pipe = sphconv.ScanPipeline(run, device=DEV, depth=2)
        tickets, got = [], []
        for host, _ in batches:
            tickets.append(pipe.submit(host))
            if len(tickets) > 1:
                got.append({k: v.clone() for k, v in pipe.result(tickets.pop(0)).items()})
        got.append({k: v.clone() for k, v in pipe.result(tickets.pop(0)).items()})
        pipe.drain()
    assert len(got) == len(direct)
    for g, d in zip(got, direct):
        assert set(g) == set(d)
        for k in d:
            assert g[k].shape == d[k].shape and torch.equal(g[k], d[k]), k
    assert pipe.h2d_bytes > 0 and pipe.d2h_bytes > 0
    assert sphconv.check_status() == 0


def test_pipeline_slot_regrown_while_other_batch_in_flight():
    """The second use of a slot needs a staging buffer more than 1.25x larger than its first use: the new buffer comes
    from the compute stream's pool while the other slot's batch is still computing, and the copy-in must wait for
    that work.  Results must equal direct calls for every batch."""
    net = build_encoder8(dtype=torch.float16, device=DEV).eval()
    sizes = [1, 1, 4, 6, 2, 8]          # scans per batch: slot 0 sees 1 -> 4 -> 2, slot 1 sees 1 -> 6 -> 8
    batches = [_host_batch(10 * i, B) for i, B in enumerate(sizes)]
    shape = batches[0][1]

    def run_b(B):
        def run(f, zi, zp):
            y = net(sphconv.SparseConvTensor(f, shape, B, z_idx=zi, z_ptr=zp))
            return {"feature": y.feature, "z_idx": y.z_idx}
        return run

    with torch.no_grad():
        direct = [{k: v.cpu().clone() for k, v in run_b(B)(*[t.to(DEV) for t in host]).items()}
                  for (host, _), B in zip(batches, sizes)]
        cur = {"B": 1}
        pipe = sphconv.ScanPipeline(lambda f, zi, zp: run_b(cur["B"])(f, zi, zp), device=DEV, depth=2)
        tickets, got = [], []
        for (host, _), B in zip(batches, sizes):
            cur["B"] = B
            tickets.append(pipe.submit(host))
            if len(tickets) > 1:
                got.append({k: v.clone() for k, v in pipe.result(tickets.pop(0)).items()})
        got.append({k: v.clone() for k, v in pipe.result(tickets.pop(0)).items()})
        pipe.drain()
    for g, d in zip(got, direct):
        for k in d:
            assert g[k].shape == d[k].shape and torch.equal(g[k], d[k]), k
    assert sphconv.check_status() == 0


def test_pipeline_misuse_is_reported():
    pipe = sphconv.ScanPipeline(lambda x: {"y": x * 2}, device=DEV, depth=1)
    x = torch.arange(8, dtype=torch.float32).pin_memory()
    t = pipe.submit((x,))
    with pytest.raises(RuntimeError):
        pipe.submit((x,))                       # slot still holds an unfetched result
    assert torch.equal(pipe.result(t)["y"], x * 2)
    with pytest.raises(RuntimeError):
        pipe.result(t)                          # already fetched
    with pytest.raises(RuntimeError):
        pipe.submit((torch.zeros(4),))          # not pinned
