#!/usr/bin/env python
"""Benchmark of the sphconv hot path on B200: rule generation + rule-driven sparse convolution of the
SECOND-style 8-layer encoder over synthetic range-voxel scans.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg3|cfg4|cfg5] [--impl reference]

One step = one pass of the whole path over one batch of scans: five rule sets (the SubM pairs share
theirs) and eight convolutions.  Rank r of N processes its own scans (no data-path collective).
Prints ONE JSON line on rank 0.  `value` is scans/s with inputs resident in HBM; `e2e` is the same
through the module API with pinned HOST buffers (H2D of z_ptr/z_idx/features and D2H of the output
features and their oz_ptr/oz_idx inside the timed region).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from sphconv_b200 import synthetic  # noqa: E402

DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], tflops=p["bf16_tflops"], tflops_sustained=p.get("bf16_tflops_sustained"),
                    source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi samples of SM clock and throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.rows = []
        self.proc = None
        try:
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", uuid, "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, t0, t1):
        if self.proc is None:
            return None
        time.sleep(0.12)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        rows = [r for t, r in self.rows if t0 - 0.05 <= t <= t1 + 0.05 and len(r) >= 7] or \
               [r for t, r in self.rows if len(r) >= 7]
        if not rows:
            return None
        sm = sorted(float(r[0]) for r in rows)
        reasons = set()
        for r in rows:
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(rows[0][1]), "samples": len(rows),
                "reasons": sorted(reasons)}


def workload(name, world, rank, batch_override):
    """(config, scans per forward pass, forward passes per step, scaling, first scan id of this rank)."""
    cfg = dict(synthetic.CONFIGS[name])
    if name == "cfg5":          # 64 scans sharded over the ranks (fixed total work), run 8 scans at a time
        per_rank = batch_override or max(1, 64 // world)
        B = min(8, per_rank)
        chunks = max(1, per_rank // B)
        return cfg, B, chunks, "strong", rank * B * chunks
    B = batch_override or cfg["B"]   # every rank runs the configuration's batch (fixed per-GPU work)
    return cfg, B, 1, "weak", rank * B


def cpu_dense_scan(cfg, scan_id, threads, w_div=1):
    """The reference's CPU check for this path - dense fp32 conv3d over the densified grid
    (test/test_rules.py:14-60, test/test_grad.py:7-36) - for ONE scan of the workload, or for a strip of
    1/w_div of its azimuth columns (dense work is proportional to the grid, whatever the sparsity).
    Returns (seconds, checksum)."""
    from oracle import dense_ref
    from sphconv_b200.encoder import encoder8_parameters
    cfg = dict(cfg)
    cfg["shape"] = [cfg["shape"][0], cfg["shape"][1] // w_div, cfg["shape"][2]]
    b = synthetic.make_batch(cfg, batch=1, first_scan=scan_id)
    params = encoder8_parameters()
    torch.set_num_threads(threads)
    with torch.no_grad():
        t0 = time.perf_counter()
        y, _ = dense_ref.encoder_dense_forward(b["feature"], b["z_idx"], b["z_ptr"], 1, cfg["shape"],
                                               synthetic.ENCODER8, params)
        dt = time.perf_counter() - t0
    return dt, float(y.abs().sum())


def voxelize_section(cfg, B, dev, with_cpu):
    """Not part of the timed step: the GPU voxeliser (raw points -> range-voxel tensor) on B synthetic sweeps of
    120k points in the configuration's grid, timed with CUDA events, beside the reference's host voxeliser
    (its compiled module when oracle/_ref holds it, else the numpy restatement) on one sweep."""
    from sphconv_b200 import VoxelGenerator, _capi
    cart, sph = [6, -40, -3, 70.4, 40, 1], [6, -45, 87.5, 70.4, 45, 100]       # sphconv/datagen.py:84-85
    n_pts = 120000
    H, W, D = cfg["shape"]
    grid = [D, W, H]
    rng = np.random.default_rng(4242)
    scans = [synthetic.make_point_cloud(rng, n_pts, sph) for _ in range(B)]
    pts = torch.as_tensor(np.concatenate(scans, 0), device=dev)
    scan_ptr = torch.as_tensor(np.arange(B + 1, dtype=np.int32) * n_pts)
    gen = VoxelGenerator(cart, sph, 2, 200000, grid, "spherical")
    lib = _capi.lib()
    for _ in range(3):
        r = gen.generate(pts, scan_ptr, with_coordinates=False)
    torch.cuda.synchronize()
    reps = 10
    l0 = lib.sph_kernel_launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        r = gen.generate(pts, scan_ptr, with_coordinates=False)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    launches = (lib.sph_kernel_launches() - l0) // reps
    voxels = int(r["voxel_num"])
    alg_bytes = 16.0 * B * n_pts + 20.0 * voxels + 4.0 * B * H * W     # points in, feature + z_idx out, z_ptr out
    out = {"ms_per_batch": round(ms, 4), "scans": B, "points": B * n_pts, "voxels": voxels,
           "scans_per_s": round(B / (ms * 1e-3), 1), "kernel_launches": int(launches),
           "algorithmic_gbs": round(alg_bytes / (ms * 1e-3) / 1e9, 1),
           "what": "transform + cells + first-2-points mean + z_ptr/z_idx, device resident points, includes the "
                   "row-count read-back"}
    if with_cpu:
        from oracle import build_ref, voxelize_np
        utils = build_ref.load_utils()
        p0 = scans[0]
        rng6 = voxelize_np.system_range(cart, sph, "spherical")
        t0 = time.time()
        with np.errstate(all="ignore"):
            sys_pts = voxelize_np.system_points(p0, "spherical")
        if utils is not None:
            mv = 200000
            voxels_a = np.zeros((mv, 2, 4), np.float32)
            mask_a = np.zeros((mv, 2), np.float32)
            coors_a = np.zeros((mv, 3), np.int32)
            num_a = np.zeros((mv,), np.int32)
            lookup = np.full(tuple(grid[::-1]), -1, np.int32)
            t0 = time.time()
            with np.errstate(all="ignore"):
                sys_pts = voxelize_np.system_points(p0, "spherical")
            nv = utils.points_to_voxel_3d(p0, sys_pts, voxels_a, mask_a, coors_a, num_a, lookup, rng6, grid, 2, mv, 0)
            mean = voxels_a[:nv].sum(1) / num_a[:nv, None]
            kind = "reference"
        else:
            rr = voxelize_np.points_to_voxel(p0, sys_pts, rng6, grid, 2, 200000)
            mean = voxelize_np.simple_voxel(rr["voxels"], rr["num_points_per_voxel"])
            kind = "port"
        dt = time.time() - t0
        out["cpu"] = {"scans_per_s": round(1.0 / dt, 2), "kind": kind, "cores": 1,
                      "sample": "one sweep of %d points: transform, point2voxel walk, mean (no init_tensor)" % n_pts}
    return out


def run_reference(args):
    """Reference arm: the path's CPU form on the host cores (the reference has no CPU implementation of its
    CUDA kernels; its tests check them against dense torch conv3d, which is what is timed here).  One step = ONE
    WHOLE scan of the workload's grid (cfg5: a quarter-azimuth strip, since one of its scans is four cfg3 scans
    wide; the line says so)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = dict(synthetic.CONFIGS[args.workload])
    threads = os.cpu_count() or 1
    w_div = 4 if args.workload == "cfg5" else 1
    times = []
    for i in range(args.warmup + args.steps):
        dt, _ = cpu_dense_scan(cfg, i, threads, w_div)
        if i >= args.warmup:
            times.append(dt)
    total = sum(times)
    value = len(times) / w_div / total
    what = "one whole %s scan" % args.workload if w_div == 1 else \
        "a 1/%d azimuth strip (%dx%dx%d) of one %s scan, scaled to whole scans" % (
            w_div, cfg["shape"][0], cfg["shape"][1] // w_div, cfg["shape"][2], args.workload)
    sample = "each step = %s through all 8 layers (forward) as dense fp32 conv3d on the densified grid" % what
    line = {
        "impl": "reference", "metric": "backbone scans/sec", "value": value, "unit": "scans/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "%s: SECOND-style 8-layer encoder, dense fp32 on host cores" % args.workload,
                   "shape": cfg["shape"], "scans_per_step": 1.0 / w_div, "same_grid_as_gpu_arm": w_div == 1},
        "cpu_baseline": {"value": value, "unit": "scans/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "scans/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def kernel_of(lib, dcode, kind, k_ch, n_ch, esize, dtype_name):
    """Name of the kernel instantiation a conv / dgrad / wgrad layer launches (for grouping layers by kernel)."""
    tc = bool(lib.sph_conv_uses_tensor_cores(dcode, k_ch, n_ch))
    if kind == "wgrad":
        which = lib.sph_conv_wgrad_kernel(dcode, k_ch, n_ch)
        if which == 1:
            return "conv_wgrad_tc_kernel<%d>" % (k_ch * esize // 16), True
        return ("conv_wgrad_pairs_kernel<%d,%d>" % (k_ch, n_ch)) if which == 2 else "conv_wgrad_generic_kernel", False
    if not tc:
        if lib.sph_conv_uses_pair_kernel(dcode, k_ch, n_ch):
            return "conv_sparse_rows_kernel<%d,%d>" % (k_ch, n_ch), tc
        return "conv_gather_generic_kernel", tc
    # 64-byte rows run the form with the output row on the TMEM lane (conv_tc_rows.cu), wider rows the transposed one
    name = "conv_gather_rows_kernel" if k_ch * esize == 64 and n_ch % 16 == 0 else "conv_gather_tc_kernel"
    return "%s<%d,%s>" % (name, k_ch * esize // 16, "i8" if dtype_name == "int8" else "f16"), tc


class Workload:
    """One benchmark configuration on this rank: data, network, the step function and its timings."""

    def __init__(self, name, args, world, rank, dev, dist):
        import sphconv_b200 as sphconv
        from sphconv_b200 import quant, sharding
        from sphconv_b200.encoder import build_encoder8
        self.name, self.args, self.world, self.rank, self.dev, self.dist = name, args, world, rank, dev, dist
        self.sphconv = sphconv
        cfg, B, chunks, scaling, first_scan = workload(name, world, rank, args.batch if name == args.workload else 0)
        self.cfg, self.B, self.chunks, self.scaling = cfg, B, chunks, scaling
        self.dtype_name = {"cfg3": "fp16", "cfg4": "bf16", "cfg5": "int8"}[name]
        self.training = name == "cfg4"
        self.shape = cfg["shape"]
        self.h_in, self.d_in = [], []
        if name == "cfg5":
            net32 = build_encoder8(dtype=torch.float32, device=dev, fused=True).eval()
            cb = synthetic.make_batch(cfg, batch=1, first_scan=10_000)
            with torch.no_grad():
                self.net = quant.quantize_encoder(net32, sphconv.SparseConvTensor(
                    torch.as_tensor(cb["feature"], device=dev), self.shape, 1,
                    z_idx=torch.as_tensor(cb["z_idx"], device=dev), z_ptr=torch.as_tensor(cb["z_ptr"], device=dev)))
            del net32
            torch.cuda.empty_cache()
            self.feat_dtype = torch.int8
        else:
            self.feat_dtype = DTYPES[self.dtype_name]
            net = build_encoder8(dtype=self.feat_dtype, device=dev, fused=True)
            self.net = net.train() if self.training else net.eval()
        for c in range(chunks):
            batch = synthetic.make_batch(cfg, batch=B, first_scan=first_scan + c * B)
            f = torch.as_tensor(batch["feature"])
            f = self.net.quantize_input(f.to(dev)).cpu() if name == "cfg5" else f.to(self.feat_dtype)
            h = (f.pin_memory(), torch.as_tensor(batch["z_idx"]).pin_memory(), torch.as_tensor(batch["z_ptr"]).pin_memory())
            self.h_in.append(h)
            self.d_in.append(tuple(t.to(dev) for t in h))
        # cfg4: every wgrad kernel accumulates in fp32 straight into its slice of ONE flat buffer, which is
        # all-reduced in place (one NCCL call per step) and never rounded to bf16 on the way
        self.grads = sharding.GradBuffer(self.net.parameters()) if self.training else None
        self.grad_out = {}
        self.copy_bytes = {"h2d": 0, "d2h": 0}
        self.pipe = None

    def run_pass(self, f, zi, zp):
        sphconv = self.sphconv
        if not self.training:
            return self.net(sphconv.SparseConvTensor(f, self.shape, self.B, z_idx=zi, z_ptr=zp))
        self.grads.zero()
        x = sphconv.SparseConvTensor(f.detach().requires_grad_(True), self.shape, self.B, z_idx=zi, z_ptr=zp)
        y = self.net(x)
        n = y.feature.shape[0]
        if self.grad_out.get("n") != n:
            g = torch.Generator(device=self.dev).manual_seed(4)
            self.grad_out["g"] = torch.randn(y.feature.shape, generator=g, device=self.dev).to(y.feature.dtype)
            self.grad_out["n"] = n
        y.feature.backward(self.grad_out["g"])
        self.grads.all_reduce()
        return y

    def step_resident(self):
        for f, zi, zp in self.d_in:
            y = self.run_pass(f, zi, zp)
        return y

    def run_to_outputs(self, f, zi, zp):
        y = self.run_pass(f, zi, zp)
        if self.training:
            return {"flat_grad": self.grads.flat}
        return {"feature": y.feature, "z_idx": y.z_idx, "z_ptr": y.z_ptr}

    # End to end through the public API: pinned host inputs -> ScanPipeline (copy-in, compute, copy-out on three
    # streams, two batches in flight) -> pinned host results.  Every batch's copies are inside the timed region.
    def run_e2e(self, steps, flush_buf):
        from sphconv_b200 import ScanPipeline
        if self.pipe is None:
            self.pipe = ScanPipeline(self.run_to_outputs, device=self.dev, depth=2)
        pipe = self.pipe
        tickets = []
        h2d = d2h = 0
        for _ in range(steps):
            flush_buf.fill_(1.0)
            h2d = d2h = 0
            for host in self.h_in:
                tickets.append(pipe.submit(host))
                h2d += pipe.h2d_bytes
                d2h += pipe.d2h_bytes
                if len(tickets) > 1:
                    pipe.result(tickets.pop(0))     # the previous batch's result, while this one computes
        while tickets:
            pipe.result(tickets.pop(0))
        pipe.drain()
        self.copy_bytes["h2d"], self.copy_bytes["d2h"] = h2d, d2h

    def copy_only_ms(self, steps):
        """What the copies of the end-to-end run cost by themselves: the same bytes per step, H2D from and D2H into
        the pipeline's own pinned buffers, one cudaMemcpyAsync per tensor on two streams, nothing computed.  With N
        ranks this runs on all of them at once, so it shows what the host side can absorb."""
        pipe = self.pipe
        if pipe is None or not pipe.slots[0].host_out:
            return None
        s_in, s_out = pipe.copy_in, pipe.copy_out
        outs = [{k: torch.empty(v.shape, dtype=v.dtype, device=self.dev) for k, v in sl.views.items()}
                for sl in pipe.slots if sl.views]
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        s_in.wait_event(a)
        s_out.wait_event(a)
        for i in range(steps * len(self.h_in)):
            sl = pipe.slots[i % len(outs)]
            with torch.cuda.stream(s_in):
                for d, h in zip(sl.dev_in, self.h_in[i % len(self.h_in)]):
                    d[:h.shape[0]].copy_(h, non_blocking=True)
            with torch.cuda.stream(s_out):
                for k, v in sl.views.items():
                    v.copy_(outs[i % len(outs)][k], non_blocking=True)
        cur = torch.cuda.current_stream(self.dev)
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg3", choices=["cfg3", "cfg4", "cfg5"])
    ap.add_argument("--batch", type=int, default=0, help="scans per rank per step (default: the configuration's)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip what is reported beside the metric (tables-only step, voxeliser, the cfg4 / cfg5 "
                         "sub-records, the copy-only run): for profiler runs")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3

    if args.impl == "reference":
        run_reference(args)
        return

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    torch.cuda.set_per_process_memory_fraction(0.8, local_rank)   # stay well inside the device: a dead box helps nobody
    dev = torch.device("cuda", local_rank)
    dist = None
    numa_cpus = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        # one process per GPU: keep each rank's pinned host buffers in its GPU's NUMA node
        from sphconv_b200.pipeline import bind_host_to_device
        numa_cpus = bind_host_to_device(local_rank)

    import sphconv_b200 as sphconv
    from sphconv_b200 import _capi, profiling

    sphconv.config.fill_unused_rules = False   # entries of `rules` past rule_size are never read by the path
    lib = _capi.lib()
    flush = torch.empty(256 * 1024 * 1024 // 4, dtype=torch.float32, device=dev)   # > 126 MB L2

    def timed(fn, steps):
        evs = []
        for _ in range(steps):
            flush.fill_(1.0)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            evs.append((a, b))
        torch.cuda.synchronize()
        return [a.elapsed_time(b) for a, b in evs]

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce_ranks(x, op="max"):
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX if op == "max" else dist.ReduceOp.MIN)
        return float(t.item())

    def measure(wl, steps, warmup, full):
        """Resident-input and end-to-end timings of one workload; `full` adds the per-layer sections."""
        res = {}
        with torch.set_grad_enabled(wl.training):
            for _ in range(warmup):
                y = wl.step_resident()
            torch.cuda.synchronize()
            sphconv.check_status()
            res["out_rows"] = int(y.feature.shape[0])
            if full:
                # pairs per layer (for the algorithmic flop / byte counts), from one untimed step
                profiling.pair_counts = {}
                wl.step_resident()
                torch.cuda.synchronize()
                res["pairs_of"] = dict(profiling.pair_counts)
                profiling.pair_counts = None
                for _ in range(2):      # the counting pass left its temporaries in the allocator's cache
                    wl.step_resident()
                torch.cuda.synchronize()
            barrier()
            launches0 = lib.sph_kernel_launches()
            if full:
                profiling.enable(True)
            times = timed(wl.step_resident, steps)
            if full:
                res["sections"] = profiling.collect()
                profiling.enable(False)
            res["launches"] = (lib.sph_kernel_launches() - launches0) // steps
            barrier()
            own_ms = sum(times)
            res["total_ms"] = reduce_ranks(own_ms, "max")
            res["min_rank_ms"] = reduce_ranks(own_ms, "min")
            if full and not args.no_extras:
                # the same step when the module path keeps only the neighbour tables (what the convolution kernels
                # read) and skips the reference-format pair lists; reported beside `value`, never as it
                sphconv.config.materialize_rules = False
                for _ in range(2):
                    wl.step_resident()
                barrier()
                res["tables_ms"] = reduce_ranks(sum(timed(wl.step_resident, steps)), "max")
                sphconv.check_status()
                sphconv.config.materialize_rules = True
                for _ in range(2):
                    wl.step_resident()
                barrier()
            # ---- end to end from pinned host buffers
            wl.run_e2e(3, flush)
            barrier()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
            wl.run_e2e(steps, flush)      # ends with the last result in host memory and the side streams joined
            ev1.record()
            barrier()
            res["e2e_ms"] = reduce_ranks(ev0.elapsed_time(ev1), "max")
            sphconv.check_status()
            if not args.no_extras:
                barrier()
                c = wl.copy_only_ms(steps)
                res["copy_only_ms"] = None if c is None else reduce_ranks(c, "max")
                barrier()
        return res

    wl = Workload(args.workload, args, world, rank, dev, dist)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    t_wall0 = time.time()
    res = measure(wl, args.steps, args.warmup, full=True)
    t_wall1 = time.time()
    clocks = sampler.stop(t_wall0, t_wall1) if sampler is not None else None

    # ---- the other two encoder configurations, compactly (same path, fewer steps): training with the wgrad
    # all-reduce inside the step (cfg4) and the int8 run of 64 wide scans sharded over the ranks (cfg5)
    subs = {}
    if not args.no_extras:
        keep = (wl.B, wl.chunks, wl.shape, wl.training, wl.feat_dtype, wl.dtype_name, wl.scaling, wl.cfg,
                dict(wl.copy_bytes))
        del wl
        torch.cuda.empty_cache()
        for other in ("cfg4", "cfg5"):
            if other == args.workload:
                continue
            try:
                w2 = Workload(other, args, world, rank, dev, dist)
                k2 = max(2, min(args.steps, 5 if other == "cfg4" else 3))
                r2 = measure(w2, k2, 3, full=False)
                scans2 = world * w2.B * w2.chunks * k2
                subs[other] = {
                    "value": round(scans2 / (r2["total_ms"] * 1e-3), 2), "unit": "scans/s",
                    "ms_per_step": round(r2["total_ms"] / k2, 4), "min_rank_ms_per_step": round(r2["min_rank_ms"] / k2, 4),
                    "e2e": round(scans2 / (r2["e2e_ms"] * 1e-3), 2), "e2e_ms_per_step": round(r2["e2e_ms"] / k2, 4),
                    "dtype": w2.dtype_name, "scaling": w2.scaling, "steps": k2, "scans_per_step": world * w2.B * w2.chunks,
                    "h2d_bytes_per_step": int(w2.copy_bytes["h2d"]), "d2h_bytes_per_step": int(w2.copy_bytes["d2h"]),
                    "gpu_launches_per_step": int(r2["launches"]),
                    "what": ("bf16 forward + dgrad + wgrad of all 8 layers, %d scans per GPU; ONE %s all-reduce of the "
                             "flat fp32 weight-gradient buffer (%d floats) inside every step"
                             % (w2.B, "NCCL" if world > 1 else "(skipped at 1 GPU)", w2.grads.flat.numel()))
                            if other == "cfg4" else
                            ("int8 inference, grid %s, 64 scans split over %d GPU(s), %d forward passes of %d scans each"
                             % ("x".join(map(str, w2.shape)), world, w2.chunks, w2.B))}
                del w2
            except Exception as e:      # a sub-record never takes the bench line down
                subs[other] = {"error": str(e)[:300]}
            torch.cuda.empty_cache()
        B, chunks, shape, training, feat_dtype, dtype_name, scaling, cfg, copy_bytes = keep
    else:
        B, chunks, shape, training, feat_dtype, dtype_name, scaling, cfg, copy_bytes = (
            wl.B, wl.chunks, wl.shape, wl.training, wl.feat_dtype, wl.dtype_name, wl.scaling, wl.cfg, dict(wl.copy_bytes))

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peaks = load_peaks()
    total_ms, e2e_total_ms, tables_ms = res["total_ms"], res["e2e_ms"], res.get("tables_ms")
    pairs_of, sections, launches, out_rows = res["pairs_of"], res["sections"], res["launches"], res["out_rows"]
    scans = world * B * chunks * args.steps
    value = scans / (total_ms * 1e-3)
    e2e_value = scans / (e2e_total_ms * 1e-3)

    # ---- per-layer accounting.  Convolution: algorithmic flops F = 2*pairs*iC*oC, bytes Q = e*(rows_in*iC +
    # rows_out*oC) + e*KV*iC*oC + 8*pairs (each row read / written once, each pair read once).  The bound that binds
    # is the larger of F / tensor peak and Q / HBM peak; frac_bound = that time / the measured time.
    # Rule generation (integer work, HBM): Q = 4*B*H*W + 4*NNZ_in + 8*pairs + 4*NTile*KV + 4*KV*rows_out (the
    # neighbour table) (+ 4*B*oH*oW + 4*rows_out for a strided set, whose output pattern is produced too).
    layers = {}
    for name, ms, meta in sections:
        ent = layers.setdefault(name, {"ms": 0.0, "meta": meta})
        ent["ms"] += ms
    conv_meta = {n.split(":", 1)[1]: e["meta"] for n, e in layers.items() if n.startswith("conv:")}
    layer_rows = []
    groups = {}
    tc_flops = tc_ms = 0.0
    conv_ms = rules_ms = lists_ms = 0.0
    dcode = _capi.DTYPE_CODE[feat_dtype]
    t_peak, h_peak = peaks["tflops"] * 1e12, peaks["hbm_gbs"] * 1e9
    for name, ent in layers.items():
        ms = ent["ms"] / args.steps            # per step (all forward passes of the step together)
        meta = ent["meta"]
        kind, tag = name.split(":", 1)
        if kind in ("conv", "dgrad", "wgrad"):
            pairs = pairs_of.get("conv:" + tag, 0)
            iC, oC, e = meta["iC"], meta["oC"], meta["esize"]
            flops = 2.0 * pairs * iC * oC
            byts = chunks * (e * (meta["n_in"] * iC + meta["n_out"] * oC) + e * 27 * iC * oC) + 8.0 * pairs
            tf = flops / (ms * 1e-3) / 1e12
            gbs = byts / (ms * 1e-3) / 1e9
            k_ch, n_ch = (oC, iC) if kind == "dgrad" else (meta.get("k_ch", iC), meta.get("n_ch", oC))
            kernel, uses_tc = kernel_of(lib, dcode, kind, k_ch, n_ch, e, dtype_name)
            t_f, t_q = flops / t_peak, byts / h_peak
            layer_rows.append({"layer": name if kind != "conv" else tag, "ms": round(ms, 4), "pairs": pairs,
                               "tflops": round(tf, 2), "gbs": round(gbs, 1), "frac_tensor": round(tf / peaks["tflops"], 4),
                               "frac_hbm": round(gbs / peaks["hbm_gbs"], 4), "bound": "tensor" if t_f >= t_q else "hbm",
                               "frac_bound": round(max(t_f, t_q) / (ms * 1e-3), 4), "kernel": kernel})
            conv_ms += ms
            g = groups.setdefault(kernel, {"ms": 0.0, "flops": 0.0, "bytes": 0.0, "launches": 0, "layers": [], "traffic": 0.0})
            g["ms"] += ms
            g["flops"] += flops
            g["bytes"] += byts
            g["launches"] += chunks
            per_row = TRAFFIC_BYTES_PER_OUT_ROW.get(dtype_name, {}).get(tag) if kind == "conv" else None
            g["traffic"] = None if (per_row is None or g["traffic"] is None) else g["traffic"] + per_row * chunks * meta["n_out"]
            g["layers"].append(name if kind != "conv" else tag)
            if uses_tc:
                tc_flops += flops
                tc_ms += ms
        elif kind == "rules":
            rules_ms += ms
            row = {"layer": name, "ms": round(ms, 4)}
            cm = conv_meta.get(tag)
            if cm is not None and "B" in meta:
                pairs = pairs_of.get("conv:" + tag, 0)
                Bn, (ih, iw, _), (oh, ow, _) = meta["B"], meta["in_shape"], meta["out_shape"]
                q = chunks * (4.0 * Bn * ih * iw + 4.0 * meta["n_in"] + 4.0 * meta["n_tile"] * meta["kv"]
                              + 4.0 * meta["kv"] * cm["n_out"]) + 8.0 * pairs
                if not meta["subm"]:
                    q += chunks * (4.0 * Bn * oh * ow + 4.0 * cm["n_out"])
                row.update({"bytes": int(q), "gbs": round(q / (ms * 1e-3) / 1e9, 1),
                            "frac_hbm": round(q / (ms * 1e-3) / h_peak, 4),
                            "what": "neighbour table" + ("" if meta["subm"] else " + output pattern (count, scan, fill)")})
            layer_rows.append(row)
        elif kind == "lists":
            lists_ms += ms
            pairs = pairs_of.get("conv:" + tag, 0)
            cm = conv_meta.get(tag)
            row = {"layer": name, "ms": round(ms, 4)}
            if cm is not None:
                q = chunks * 4.0 * 27 * cm["n_out"] + 8.0 * pairs          # table read, pairs written
                row.update({"bytes": int(q), "gbs": round(q / (ms * 1e-3) / 1e9, 1),
                            "frac_hbm": round(q / (ms * 1e-3) / h_peak, 4),
                            "what": "reference-format pair lists from the table, on a side stream beside the convolution"})
            layer_rows.append(row)
        else:
            layer_rows.append({"layer": name, "ms": round(ms, 4)})
    all_tc = tc_flops / (tc_ms * 1e-3) / 1e12 if tc_ms > 0 else 0.0

    # ---- roofline: one object per kernel instantiation, on the bound that binds it; the line's `roofline` is the
    # instantiation that takes the most time in the step
    by_kernel = []
    for kernel, g in groups.items():
        t = g["ms"] * 1e-3
        t_f, t_q = g["flops"] / t_peak, g["bytes"] / h_peak
        bound = "tensor" if t_f >= t_q else "hbm"
        achieved = g["flops"] / t / 1e12 if bound == "tensor" else g["bytes"] / t / 1e9
        by_kernel.append({
            "kernel": kernel, "layers": g["layers"], "launches_per_step": g["launches"],
            "ms_per_step": round(g["ms"], 4), "share_of_conv_time": round(g["ms"] / conv_ms, 4) if conv_ms else None,
            "launch_ms": round(g["ms"] / g["launches"], 4), "bound": bound, "achieved": round(achieved, 2),
            "peak": peaks["tflops"] if bound == "tensor" else peaks["hbm_gbs"],
            "unit": "TFLOP/s" if bound == "tensor" else "GB/s",
            "frac": round(max(t_f, t_q) / t, 4),
            "frac_tensor": round(t_f / t, 4), "frac_hbm": round(t_q / t, 4),
            "flops_per_launch": g["flops"] / g["launches"], "bytes_per_launch": g["bytes"] / g["launches"],
            "traffic": None if g["traffic"] is None else int(g["traffic"] / g["launches"]),
            "traffic_source": None if g["traffic"] is None else TRAFFIC_SOURCE,
            "busiest_unit_ncu": BUSIEST_UNIT.get(kernel)})
    by_kernel.sort(key=lambda r: -r["ms_per_step"])
    dom = by_kernel[0] if by_kernel else {}
    roofline = dict(dom)
    roofline.update({"peak_source": "of " + peaks["source"] + (" (burst bf16)" if dom.get("bound") == "tensor" else " (copy)"),
                     "what": "the kernel instantiation with the largest share of the step's convolution time; achieved = "
                             "algorithmic work of its launches / their CUDA-event time inside the timed steps",
                     "all_tensor_core_layers_tflops": round(all_tc, 2), "conv_ms_per_step": round(conv_ms, 4),
                     "rules_ms_per_step": round(rules_ms, 4), "lists_ms_per_step_side_stream": round(lists_ms, 4),
                     "by_kernel": by_kernel})

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        w_div = 4 if args.workload == "cfg5" else 1        # cfg5 scans are 4x wider: time a quarter-azimuth strip
        dt, _ = cpu_dense_scan(cfg, 0, threads, w_div)    # warm-up (thread pool, allocator)
        dts = [cpu_dense_scan(cfg, 0, threads, w_div)[0] for _ in range(2)]
        cpu = {"value": 1.0 / w_div / (sum(dts) / len(dts)), "unit": "scans/s", "cores": threads, "kind": "port",
               "sample": "%s of one %s scan through all 8 layers (forward) as dense fp32 conv3d on the densified grid, "
                         "mean of 2" % ("a 1/%d azimuth strip" % w_div if w_div > 1 else "the whole", args.workload)}

    vox = None
    if world == 1 and not args.no_extras:
        try:
            vox = voxelize_section(cfg, B, dev, not args.no_cpu_baseline)
        except Exception as e:          # an extra: never takes the bench line down
            vox = {"error": str(e)[:200]}

    h2d, d2h = copy_bytes["h2d"], copy_bytes["d2h"]
    copy_ms = res.get("copy_only_ms")
    line = {
        "metric": "backbone scans/sec", "value": round(value, 2), "unit": "scans/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(total_ms / args.steps, 4),
        "min_rank_ms_per_step": round(res["min_rank_ms"] / args.steps, 4),
        "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": dtype_name, "data": "synthetic",
        "config": {"workload": "%s: SECOND-style 8-layer encoder, %s %s, grid %s, %d scans per GPU per step"
                               % (args.workload, dtype_name, "forward+backward+wgrad all-reduce" if training else "inference",
                                  "x".join(map(str, shape)), B * chunks),
                   "scans_per_step": world * B * chunks, "scans_per_forward_pass": B, "out_rows_rank0": out_rows,
                   "l2": "256 MB flush write between steps", "rule_sets_per_step": 5 * chunks,
                   "conv_layers_per_step": 8 * chunks},
        "e2e": {"value": round(e2e_value, 2), "unit": "scans/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h), "ms_per_step": round(e2e_total_ms / args.steps, 4),
                "copy_only_ms": None if copy_ms is None else round(copy_ms, 4),
                "copy_only_what": "the same H2D + D2H bytes per step through the same pinned buffers with nothing "
                                  "computed, all ranks at once: the floor the host side sets for ms_per_step",
                "host_binding": None if numa_cpus is None else "rank 0 bound to %d CPUs next to its GPU" % len(numa_cpus),
                "how": "sphconv_b200.ScanPipeline: copies on two side streams, two batches in flight; "
                       "the region times all steps at once, L2 flushes included"},
        "gpu_launches": int(launches) * args.steps,
        "gpu_launches_per_step": int(launches),
        "roofline": roofline,
        "cpu_baseline": cpu,
        "clocks": clocks,
        "tables_only": None if tables_ms is None else {
                        "value": round(scans / (tables_ms * 1e-3), 2), "unit": "scans/s",
                        "ms_per_step": round(tables_ms / args.steps, 4),
                        "what": "sphconv_b200.config.materialize_rules = False: the layers keep the neighbour tables "
                                "and do not write the reference-format rules / rule_size tensors (same outputs)"},
        "cfg4": subs.get("cfg4"),
        "cfg5": subs.get("cfg5"),
        "voxelize": vox,
        "layers": layer_rows,
    }
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per OUTPUT ROW of one launch of each convolution layer,
# from one ncu capture of the kernels of this tree on a 4-scan batch (ncu replays a launch once per pass, so the
# capture uses a smaller batch than the timed run; every output row is gathered, accumulated and written independently,
# so a launch's traffic is proportional to its rows).  Part of a launch's output is still in L2 when the kernel ends,
# so the write half undercounts.  A layer that is not listed has no captured figure (traffic: null).
TRAFFIC_SOURCE = ("ncu dram__bytes_read.sum + dram__bytes_write.sum per output row, 4-scan fp16 capture of these kernels, "
                  "scaled by the rows of the timed launches")
# What limits each instantiation according to the same capture (neither HBM nor the tensor pipe: the bench line's `bound`
# is the roofline the work is reported against, this is the unit that was busiest).
BUSIEST_UNIT = {
    "conv_gather_rows_kernel<4,f16>": "shared-memory data pipe 92 % busy (gather writes 64 % + tensor-core operand reads 28 %); DRAM 12 %, tensor pipe 11 %",
    "conv_gather_tc_kernel<8,f16>": "shared-memory data pipe 88 % busy (gather writes 58 % + operand reads 30 %); tensor pipe 47 %, DRAM 8 %",
    "conv_gather_tc_kernel<2,f16>": "shared-memory data pipe 69-93 % busy (gather writes 52-72 % + operand reads 17-22 %); DRAM 9-13 %",
    "conv_sparse_rows_kernel<4,16>": "instruction issue 68 % of the slots; DRAM 15 %",
}
TRAFFIC_BYTES_PER_OUT_ROW = {
    "fp16": {"L0": 116.2, "L1": 141.3, "L2": 146.5, "L3": 211.3, "L4": 208.9, "L5": 288.9, "L6": 280.6, "L7": 281.1},
}

if __name__ == "__main__":
    main()
