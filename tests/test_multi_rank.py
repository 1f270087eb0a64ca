"""Multi-rank host logic on CPU (gloo, world_size 2): batch sharding and the single flat all-reduce of the
weight gradients.  The per-rank compute itself is the single-GPU path covered by the GPU tests."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import conv_np, rules_np
from sphconv_b200 import sharding, synthetic
from sphconv_b200.encoder import encoder8_parameters


def test_shard_range_covers_everything():
    for n in (1, 7, 8, 64):
        for world in (1, 2, 3, 4, 8):
            got = [sharding.shard_range(n, world, r) for r in range(world)]
            assert got[0][0] == 0 and got[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(got, got[1:]))
            sizes = [b - a for a, b in got]
            assert max(sizes) - min(sizes) <= 1


def test_slice_batch_is_self_contained():
    rng = np.random.default_rng(0)
    B, shape = 5, [4, 6, 8]
    z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, 0.3)
    feat = rng.standard_normal((z_idx.shape[0], 3)).astype(np.float32)
    zi, zp, f = torch.as_tensor(z_idx), torch.as_tensor(z_ptr), torch.as_tensor(feat)
    rows = 0
    for r in range(3):
        a, b = sharding.shard_range(B, 3, r)
        szi, szp, sf = sharding.slice_batch(zi, zp, f, a, b)
        assert szp.shape[0] == b - a and int(szp.reshape(-1)[-1]) == szi.shape[0] == sf.shape[0]
        # the shard's rule set equals the oracle's on those scans alone
        sub_occ_idx, sub_occ_ptr = szi.numpy(), szp.numpy()
        res = rules_np.get_rules_subm(sub_occ_idx, sub_occ_ptr, b - a, shape, shape, [3, 3, 3], [1, 1, 1], [1, 1, 1],
                                      [1, 1, 1], [2, 2], padded=False)
        assert res["rule_size"].sum() > 0
        rows += szi.shape[0]
    assert rows == z_idx.shape[0]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # each rank: weight gradient of one SubM 4->16 layer on ITS scans, by the oracle (CPU stand-in for the kernel)
        B, shape = 4, [6, 8, 10]
        rng = np.random.default_rng(5)
        z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, 0.3)
        feat = rng.standard_normal((z_idx.shape[0], 4))
        a, b = sharding.shard_range(B, world, rank)
        zi, zp, f = sharding.slice_batch(torch.as_tensor(z_idx), torch.as_tensor(z_ptr), torch.as_tensor(feat), a, b)
        res = rules_np.get_rules_subm(zi.numpy(), zp.numpy(), b - a, shape, shape, [3, 3, 3], [1, 1, 1], [1, 1, 1],
                                      [1, 1, 1], [2, 2], padded=False)
        pairs = rules_np.canonical_from_table(res)
        dout = np.random.default_rng(100 + rank).standard_normal((zi.shape[0], 16))
        dw = conv_np.conv_wgrad(f.numpy(), dout, pairs, 27)
        w = torch.nn.Parameter(torch.zeros(3, 3, 3, 4, 16))
        bias = torch.nn.Parameter(torch.zeros(16))
        w.grad = torch.as_tensor(dw, dtype=torch.float32).reshape(3, 3, 3, 4, 16)
        n = sharding.allreduce_gradients([w, bias])
        assert n == w.numel() + bias.numel()
        gathered = [torch.zeros_like(w.grad) for _ in range(world)]
        dist.all_gather(gathered, torch.as_tensor(dw, dtype=torch.float32).reshape(3, 3, 3, 4, 16))
        assert torch.allclose(w.grad, sum(gathered), atol=1e-5)
        assert bias.grad is not None and float(bias.grad.abs().sum()) == 0.0
        if rank == 0:
            out.put(float(w.grad.abs().sum()))
    finally:
        dist.destroy_process_group()


def test_gloo_two_ranks_allreduce_wgrad():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert out.get(timeout=5) > 0


def _wgrad_of_scans(z_idx, z_ptr, feat, dout_of_scan, first, last, shape):
    """Oracle weight gradient of one SubM 4->16 layer over scans [first, last) (CPU stand-in for the kernels)."""
    zi, zp, f = sharding.slice_batch(torch.as_tensor(z_idx), torch.as_tensor(z_ptr), torch.as_tensor(feat), first, last)
    res = rules_np.get_rules_subm(zi.numpy(), zp.numpy(), last - first, shape, shape, [3, 3, 3], [1, 1, 1], [1, 1, 1],
                                  [1, 1, 1], [2, 2], padded=False)
    dout = np.concatenate([dout_of_scan[b] for b in range(first, last)], 0)
    return conv_np.conv_wgrad(f.numpy(), dout, rules_np.canonical_from_table(res), 27)


def _worker_master(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, shape = 4, [6, 8, 10]
        rng = np.random.default_rng(5)
        z_idx, z_ptr = synthetic.make_random_occupancy(rng, B, shape, 0.3)
        feat = rng.standard_normal((z_idx.shape[0], 4))
        flat = z_ptr.reshape(B, -1)[:, -1]
        starts = np.concatenate([[0], flat])
        dout_of_scan = [np.random.default_rng(100 + b).standard_normal((int(starts[b + 1] - starts[b]), 16))
                        for b in range(B)]
        # the layer's parameters in the 16-bit dtype of a training run; their gradient lives in the fp32 buffer
        w = torch.nn.Parameter(torch.zeros(3, 3, 3, 4, 16, dtype=torch.bfloat16))
        bias = torch.nn.Parameter(torch.zeros(16, dtype=torch.bfloat16))
        gb = sharding.GradBuffer([w, bias])
        assert gb.flat.dtype == torch.float32 and gb.flat.numel() == w.numel() + bias.numel()
        a, b = sharding.shard_range(B, world, rank)
        gb.zero()
        w._sph_master_grad.view(27, 4, 16).add_(torch.as_tensor(_wgrad_of_scans(z_idx, z_ptr, feat, dout_of_scan, a, b, shape),
                                                                dtype=torch.float32))
        assert gb.all_reduce() == gb.flat.numel()
        full = _wgrad_of_scans(z_idx, z_ptr, feat, dout_of_scan, 0, B, shape)
        got = w._sph_master_grad.view(27, 4, 16).double().numpy()
        # all-reduced gradient of the two shards == gradient of the whole batch on one rank, to fp32 rounding
        assert np.abs(got - full).max() <= 1e-5 * max(1.0, np.abs(full).max())
        gb.to_grads()
        assert w.grad.dtype == torch.bfloat16 and bias.grad.dtype == torch.bfloat16
        assert np.abs(w.grad.view(27, 4, 16).double().numpy() - full).max() <= 1e-2 * max(1.0, np.abs(full).max())
        if rank == 0:
            out.put(float(np.abs(full).sum()))
    finally:
        dist.destroy_process_group()


def test_gloo_two_ranks_master_gradient_buffer_equals_single_rank():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_master, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert out.get(timeout=5) > 0


def test_flat_buffer_size_of_the_encoder():
    # 27 * (4*16 + 16*16 + 16*32 + 2*32*32 + 32*64 + 2*64*64) weights: one ~1.4 MB all-reduce per step
    n = sum(int(np.prod(w.shape)) for w, _ in encoder8_parameters())
    assert n == 27 * (4 * 16 + 16 * 16 + 16 * 32 + 2 * 32 * 32 + 32 * 64 + 2 * 64 * 64) == 354240
