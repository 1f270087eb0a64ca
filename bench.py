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
    CUDA kernels; its tests check them against dense torch conv3d, which is what is timed here)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = dict(synthetic.CONFIGS[args.workload])
    threads = os.cpu_count() or 1
    w_div = 8                   # one step = a 1/8-azimuth strip of one scan: about a second of host work
    times = []
    for i in range(args.warmup + args.steps):
        dt, _ = cpu_dense_scan(cfg, i, threads, w_div)
        if i >= args.warmup:
            times.append(dt)
    total = sum(times)
    value = len(times) / w_div / total
    sample = ("each step = a 1/%d azimuth strip (%dx%dx%d) of one %s scan through all 8 layers as dense fp32 conv3d "
              "on the densified grid" % (w_div, cfg["shape"][0], cfg["shape"][1] // w_div, cfg["shape"][2], args.workload))
    line = {
        "impl": "reference", "metric": "backbone scans/sec", "value": value, "unit": "scans/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "%s: SECOND-style 8-layer encoder, dense fp32 on host cores" % args.workload,
                   "shape": cfg["shape"], "scans_per_step": 1.0 / w_div},
        "cpu_baseline": {"value": value, "unit": "scans/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "scans/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


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
                    help="skip the measurements reported beside the metric (tables-only step, voxeliser): for profiler runs")
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
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    import sphconv_b200 as sphconv
    from sphconv_b200 import _capi, profiling
    from sphconv_b200.encoder import build_encoder8

    from sphconv_b200 import quant, sharding
    cfg, B, chunks, scaling, first_scan = workload(args.workload, world, rank, args.batch)
    dtype_name = {"cfg3": "fp16", "cfg4": "bf16", "cfg5": "int8"}[args.workload]
    training = args.workload == "cfg4"
    shape = cfg["shape"]
    sphconv.config.fill_unused_rules = False   # entries of `rules` past rule_size are never read by the path
    lib = _capi.lib()
    h_in, d_in = [], []
    if args.workload == "cfg5":
        net32 = build_encoder8(dtype=torch.float32, device=dev, fused=True).eval()
        cb = synthetic.make_batch(cfg, batch=1, first_scan=10_000)
        with torch.no_grad():
            net = quant.quantize_encoder(net32, sphconv.SparseConvTensor(
                torch.as_tensor(cb["feature"], device=dev), shape, 1, z_idx=torch.as_tensor(cb["z_idx"], device=dev),
                z_ptr=torch.as_tensor(cb["z_ptr"], device=dev)))
        del net32
        torch.cuda.empty_cache()
        feat_dtype = torch.int8
    else:
        feat_dtype = DTYPES[dtype_name]
        net = build_encoder8(dtype=feat_dtype, device=dev, fused=True)
        net = net.train() if training else net.eval()
    for c in range(chunks):
        batch = synthetic.make_batch(cfg, batch=B, first_scan=first_scan + c * B)
        f = torch.as_tensor(batch["feature"])
        f = net.quantize_input(f.to(dev)).cpu() if args.workload == "cfg5" else f.to(feat_dtype)
        h = (f.pin_memory(), torch.as_tensor(batch["z_idx"]).pin_memory(), torch.as_tensor(batch["z_ptr"]).pin_memory())
        h_in.append(h)
        d_in.append(tuple(t.to(dev) for t in h))
    params = list(net.parameters()) if training else []
    grad_out = {}

    def run_pass(f, zi, zp):
        if not training:
            return net(sphconv.SparseConvTensor(f, shape, B, z_idx=zi, z_ptr=zp))
        # cfg4: forward + dgrad + wgrad of every layer, then ONE all-reduce of the flat fp32 weight gradient
        for p_ in params:
            p_.grad = None
        x = sphconv.SparseConvTensor(f.detach().requires_grad_(True), shape, B, z_idx=zi, z_ptr=zp)
        y = net(x)
        n = y.feature.shape[0]
        if grad_out.get("n") != n:
            g = torch.Generator(device=dev).manual_seed(4)
            grad_out["g"] = torch.randn(y.feature.shape, generator=g, device=dev).to(y.feature.dtype)
            grad_out["n"] = n
        y.feature.backward(grad_out["g"])
        flat, plist = sharding.flatten_grads(params)
        if dist is not None:
            dist.all_reduce(flat)
        grad_out["flat"] = flat
        return y

    def step_resident():
        for f, zi, zp in d_in:
            y = run_pass(f, zi, zp)
        return y

    # End to end through the public API: pinned host inputs -> ScanPipeline (copy-in, compute, copy-out on three
    # streams, two batches in flight) -> pinned host results.  Every batch's copies are inside the timed region.
    def run_to_outputs(f, zi, zp):
        y = run_pass(f, zi, zp)
        if training:
            return {"flat_grad": grad_out["flat"]}
        return {"feature": y.feature, "z_idx": y.z_idx, "z_ptr": y.z_ptr}

    from sphconv_b200 import ScanPipeline
    pipe = ScanPipeline(run_to_outputs, device=dev, depth=2)
    copy_bytes = {"h2d": 0, "d2h": 0}

    def run_e2e(steps, flush_buf):
        tickets = []
        h2d = d2h = 0
        for _ in range(steps):
            flush_buf.fill_(1.0)
            h2d = d2h = 0
            for host in h_in:
                tickets.append(pipe.submit(host))
                h2d += pipe.h2d_bytes
                d2h += pipe.d2h_bytes
                if len(tickets) > 1:
                    pipe.result(tickets.pop(0))     # the previous batch's result, while this one computes
        while tickets:
            pipe.result(tickets.pop(0))
        pipe.drain()
        copy_bytes["h2d"], copy_bytes["d2h"] = h2d, d2h

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

    def max_over_ranks(x):
        if dist is None:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    with torch.set_grad_enabled(training):
        sampler = ClockSampler(local_rank) if rank == 0 else None
        t_wall0 = time.time()
        for _ in range(args.warmup):
            y = step_resident()
        torch.cuda.synchronize()
        sphconv.check_status()
        out_rows = int(y.feature.shape[0])

        # pairs per layer (for the algorithmic flop / byte counts), from one untimed step
        profiling.pair_counts = {}
        step_resident()
        torch.cuda.synchronize()
        pairs_of = dict(profiling.pair_counts)
        profiling.pair_counts = None
        # the counting pass left its temporaries in the allocator's cache: settle it again before timing
        for _ in range(2):
            step_resident()
        torch.cuda.synchronize()

        # ---- resident-input timing (value), with per-layer sections for the roofline
        barrier()
        launches0 = lib.sph_kernel_launches()
        profiling.enable(True)
        times = timed(step_resident, args.steps)
        sections = profiling.collect()
        profiling.enable(False)
        launches = (lib.sph_kernel_launches() - launches0) // args.steps
        barrier()
        total_ms = max_over_ranks(sum(times))

        # ---- the same step when the module path keeps only the neighbour tables (what the convolution kernels read)
        # and skips the reference-format pair lists `rules` / `rule_size`; reported beside `value`, never as it
        tables_ms = None
        if not args.no_extras:
            sphconv.config.materialize_rules = False
            for _ in range(2):
                step_resident()
            barrier()
            tables_ms = max_over_ranks(sum(timed(step_resident, args.steps)))
            sphconv.check_status()
            sphconv.config.materialize_rules = True
            for _ in range(2):
                step_resident()
            barrier()

        # ---- end to end from pinned host buffers
        run_e2e(3, flush)
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        run_e2e(args.steps, flush)      # ends with the last result in host memory and the side streams joined
        ev1.record()
        barrier()
        e2e_total_ms = max_over_ranks(ev0.elapsed_time(ev1))
        t_wall1 = time.time()
        clocks = sampler.stop(t_wall0, t_wall1) if sampler is not None else None
        sphconv.check_status()

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peaks = load_peaks()
    scans = world * B * chunks * args.steps
    value = scans / (total_ms * 1e-3)
    e2e_value = scans / (e2e_total_ms * 1e-3)

    # ---- per-layer accounting: algorithmic flops = 2*pairs*iC*oC, bytes = e*(rows_in*iC + rows_out*oC) + e*KV*iC*oC + 8*pairs
    layers = {}
    for name, ms, meta in sections:
        ent = layers.setdefault(name, {"ms": 0.0, "meta": meta})
        ent["ms"] += ms
    layer_rows = []
    tc_flops = tc_ms = 0.0
    conv_ms = rules_ms = 0.0
    dcode = _capi.DTYPE_CODE[feat_dtype]
    for name, ent in layers.items():
        ms = ent["ms"] / args.steps            # per step (all forward passes of the step together)
        meta = ent["meta"]
        kind = name.split(":")[0]
        if kind in ("conv", "dgrad", "wgrad"):
            pairs = pairs_of.get("conv:" + name.split(":", 1)[1], 0)
            iC, oC, e = meta["iC"], meta["oC"], meta["esize"]
            flops = 2.0 * pairs * iC * oC
            byts = chunks * (e * (meta["n_in"] * iC + meta["n_out"] * oC) + e * 27 * iC * oC) + 8.0 * pairs
            tf = flops / (ms * 1e-3) / 1e12
            gbs = byts / (ms * 1e-3) / 1e9
            k_ch, n_ch = (oC, iC) if kind == "dgrad" else (meta.get("k_ch", iC), meta.get("n_ch", oC))
            # wgrad has its own tensor-core kernel for the 16-bit types, with the same row-width rule
            uses_tc = bool(lib.sph_conv_uses_tensor_cores(dcode, k_ch, n_ch)) and \
                (kind != "wgrad" or dtype_name in ("fp16", "bf16"))
            layer_rows.append({"layer": name if kind != "conv" else name[5:], "ms": round(ms, 4), "pairs": pairs,
                               "tflops": round(tf, 2), "gbs": round(gbs, 1), "frac_tensor": round(tf / peaks["tflops"], 4),
                               "frac_hbm": round(gbs / peaks["hbm_gbs"], 4), "tensor_cores": uses_tc})
            conv_ms += ms
            if uses_tc:
                tc_flops += flops
                tc_ms += ms
        else:
            rules_ms += ms
            layer_rows.append({"layer": name, "ms": round(ms, 4)})
    all_tc = tc_flops / (tc_ms * 1e-3) / 1e12 if tc_ms > 0 else 0.0
    # dominant kernel: the tensor-core convolution of the widest layers (L6 / L7: 64 -> 64), one launch per layer and
    # pass.  L6 is the first layer of its rule set: the pair-list kernel of that set runs beside its launch on a side
    # stream and its section ends with the join, so the kernel's own duration is taken from L7, the same launch alone.
    dom = [r for r in layer_rows if r.get("layer") in ("L7",)] or [r for r in layer_rows if r.get("layer") == "L6"]
    dom_ms = sum(r["ms"] for r in dom) / max(1, len(dom) * chunks)            # average launch duration
    dom_flops = sum(2.0 * r["pairs"] * 64 * 64 for r in dom) / max(1, len(dom) * chunks)
    achieved = dom_flops / (dom_ms * 1e-3) / 1e12 if dom_ms > 0 else 0.0
    traffic = TRAFFIC_BYTES_PER_OUT_ROW.get(dtype_name)
    roofline = {"kernel": "conv_gather_tc_kernel<8> on a 64->64 layer (L7; L6 is the same launch sharing the SMs with "
                          "the pair-list kernel of its rule set), per launch", "bound": "tensor",
                "achieved": round(achieved, 2), "peak": peaks["tflops"], "unit": "TFLOP/s",
                "frac": round(achieved / peaks["tflops"], 4), "peak_source": "of " + peaks["source"] + " (burst bf16)",
                "launch_ms": round(dom_ms, 4), "flops_per_launch": dom_flops,
                "traffic": None if traffic is None else int(traffic * out_rows),
                "all_tensor_core_layers_tflops": round(all_tc, 2),
                "conv_ms_per_step": round(conv_ms, 4), "rules_ms_per_step": round(rules_ms, 4)}

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
    line = {
        "metric": "backbone scans/sec", "value": round(value, 2), "unit": "scans/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(total_ms / args.steps, 4),
        "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": dtype_name, "data": "synthetic",
        "config": {"workload": "%s: SECOND-style 8-layer encoder, %s %s, grid %s, %d scans per GPU per step"
                               % (args.workload, dtype_name, "forward+backward+wgrad all-reduce" if training else "inference",
                                  "x".join(map(str, shape)), B * chunks),
                   "scans_per_step": world * B * chunks, "scans_per_forward_pass": B, "out_rows_rank0": out_rows,
                   "l2": "256 MB flush write between steps", "rule_sets_per_step": 5 * chunks,
                   "conv_layers_per_step": 8 * chunks},
        "e2e": {"value": round(e2e_value, 2), "unit": "scans/s", "h2d_bytes_per_step": int(h2d),
                "d2h_bytes_per_step": int(d2h), "ms_per_step": round(e2e_total_ms / args.steps, 4),
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
        "voxelize": vox,
        "layers": layer_rows,
    }
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


# DRAM bytes (read + write) per output row of one launch of the dominant kernel, from the ncu capture summarised in
# profiles/conv_gather_tc_64to64_fp16_b4_full.md (97.9 MB for 346.8 k rows); traffic grows in proportion to rows.
TRAFFIC_BYTES_PER_OUT_ROW = {"fp16": 282.0}

if __name__ == "__main__":
    main()
