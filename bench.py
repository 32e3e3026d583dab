#!/usr/bin/env python
"""Benchmark of the INPC hot path (sample -> project/bin -> sort -> blend, forward + backward).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One *step* is one batch of 64 camera views on a radius-3 orbit, every view being the single-view
training workload (2^18-leaf octree, 2^23 sampled points, 36 fp16 SH coefficients + fp32 opacity per
point, 1237x822, forward and backward).  The batch is sharded by view over the ranks (one process
per GPU, torchrun); per step the ranks exchange two fp32 buffers with NCCL all-reduce.  Rank 0
prints ONE JSON line.

  value  fwd+bwd Mpoints/s of the whole job, inputs resident in HBM, CUDA events, max over ranks
  e2e    the same through the public Python API with, per view, the camera and the upstream image
         gradient copied from pinned host memory and the loss read back
  roofline      dominant kernel's algorithmic bytes / measured launch time against the measured HBM peak
  cpu_baseline  the CPU restatement (oracle/, all host cores) on a bounded sample; reported only

`--impl reference` runs the reference's own CUDA backend (oracle/_ref, compiled unmodified from the
reference tree) on the same workload on one GPU; without that library it times the CPU restatement
on a bounded sample instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "fwd+bwd Mpoints/s at 2^23 points per view, 1237x822"
UNIT = "Mpoints/s"
N_VIEWS = 64
N_POINTS = 1 << 23
N_LEAVES = 1 << 18
N_APPEARANCE = 1 << 22
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per (point, tile) instance of the kernels of a
# stage, from an ncu capture of the warp blend kernels on the small case of this workload (2^22 points,
# 5,274,412 instances, 8x8 tiles: forward passes 453.9 MB, backward 328.1 MB); the traffic of these kernels grows in
# proportion to the instances.
TRAFFIC_BYTES_PER_INSTANCE = {"blend_fwd": 453.9e6 / 5274412, "blend_bwd": 328.1e6 / 5274412}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--views", type=int, default=N_VIEWS)
    ap.add_argument("--points", type=int, default=N_POINTS)
    ap.add_argument("--tile", type=int, default=8)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-side", action="store_true", help="skip the side workloads (configs 2 and 4, feature rows) at the end of a 1-GPU run")
    ap.add_argument("--streams", type=int, default=4, help="CUDA streams a rank pipelines its views over (1 = one view at a time)")
    ap.add_argument("--workload", default="config1", choices=["config1", "config2", "config4", "config4_rows32", "rows16", "rows32", "multisample4", "multisample4_batched"],
                    help="config1 is the headline (default); the others are single-GPU side measurements, one JSON line each")
    return ap.parse_args()


# ---------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.lines: list[str] = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower() == "active":
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def dist_setup(args):
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
        torch.cuda.set_device(0)
        local = 0
    return rank, local, world


def barrier(world):
    import torch
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(value: float, world: int, device) -> float:
    import torch
    if world == 1:
        return value
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def config_dict(args) -> dict:
    """The workload description both arms print (same keys, same values: the arms differ in `impl` only)."""
    return {"workload": f"config 1 single-view training step x {args.views} orbit views (config 3 batch), sharded by view",
            "points_per_view": args.points, "views_per_step": args.views, "leaves": N_LEAVES, "image": [1237, 822],
            "features": "36 x fp16 SH -> 4 channels", "tile": 8,
            "l2": "inputs (604 MB of features per view) exceed the 126 MB L2; no flush needed",
            "allreduce_floats": N_LEAVES + N_APPEARANCE}


def build_workload(args, device):
    import torch
    import synthetic_workloads as syn
    cfg = syn.config1(n_samples=args.points, n_leaves=N_LEAVES)
    views = syn.config3_views(args.views)
    g = torch.Generator().manual_seed(5)
    H, W = views[0].camera.height, views[0].camera.width
    grad_image = torch.randn((4, H, W), generator=g) * 1e-3
    grad_alpha = torch.randn((1, H, W), generator=g) * 1e-3
    return dict(tree=cfg["tree"].to(device), features=cfg["features"].to(device), opacities=cfg["opacities"].to(device),
                views_host=views, views=[v.to(device) for v in views], grad_image=grad_image, grad_alpha=grad_alpha, H=H, W=W)


# ---------------------------------------------------------------------------------------------------
def cpu_pipeline_points_per_s(n_points: int, threads: int, n_views: int = 1) -> tuple[float, str]:
    """The CPU restatement of the whole path on a bounded sample of the workload: `n_views` orbit views,
    forward and backward, `n_points` samples per view of the same octree."""
    import numpy as np
    import torch
    sys.path.insert(0, str(ROOT / "oracle"))
    import oracle as O
    import synthetic_workloads as syn
    os.environ["OMP_NUM_THREADS"] = str(threads)
    cfg = syn.config1(n_samples=n_points, n_leaves=N_LEAVES)
    tree = cfg["tree"]
    views = syn.config3_views(max(n_views, 1))
    c = views[0].camera
    g = torch.Generator().manual_seed(5)
    gi = (torch.randn((4, c.height, c.width), generator=g) * 1e-3).numpy()
    ga = (torch.randn((1, c.height, c.width), generator=g) * 1e-3).numpy()
    feats, opac = cfg["features"].numpy(), cfg["opacities"].numpy()
    centers, levels, weights = tree.centers.numpy(), tree.levels.numpy(), tree.weights.numpy()
    O.lib()
    t0 = time.perf_counter()
    for vi, view in enumerate(views[:max(n_views, 1)]):
        cam = O.Camera(view.w2c.numpy(), view.position.numpy(), c.width, c.height, c.focal_x, c.focal_y, c.center_x, c.center_y,
                       c.near_plane, c.far_plane)
        vw = O.viewpoint_weights(cam, centers, levels, weights, tree.initial_size)
        cdf, _ = O.build_cdf(vw)
        pos, idx, _ = O.training_samples(cam, 0, vi, cdf, centers, levels, tree.initial_size, n_points)
        st = O.rasterize_forward(O.BILINEAR, cam, pos, feats, opac, tile=16)
        O.rasterize_backward(st, gi, ga)
    dt = time.perf_counter() - t0
    return n_views * n_points / dt, f"{n_views} view(s) of the bench workload at {n_points} points per view (of {N_POINTS}), fwd+bwd, {dt:.1f} s"


def cpu_baseline(args) -> dict:
    threads = os.cpu_count() or 1
    pps, _ = cpu_pipeline_points_per_s(1 << 17, threads)            # calibration run
    budget_points = pps * 15.0                                      # about 15 s of CPU work
    if budget_points >= 1.5 * N_POINTS:
        pps, sample = cpu_pipeline_points_per_s(N_POINTS, threads, n_views=int(min(8, max(1, round(budget_points / N_POINTS)))))
    else:
        pps, sample = cpu_pipeline_points_per_s(int(min(max(budget_points, 1 << 17), N_POINTS)), threads)
    return {"value": pps / 1e6, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample}


# ---------------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    from inpc_b200 import _cabi
    from inpc_b200.batch import ViewShardedTrainer, partition_views

    rank, local, world = dist_setup(args)
    device = torch.device("cuda", local)
    wl = build_workload(args, device)
    trainer = ViewShardedTrainer(wl["tree"], wl["features"], wl["opacities"], args.points, seed=0, n_appearance=N_APPEARANCE,
                                 tile_size=args.tile, n_streams=args.streams)
    gi_dev, ga_dev = wl["grad_image"].to(device), wl["grad_alpha"].to(device)
    my_views = partition_views(args.views, rank, world)

    def step():
        trainer.run_batch(wl["views"], (gi_dev, ga_dev), rank, world)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier(world)
    launches0 = _cabi.launch_count()
    clocks = ClockSampler(local) if rank == 0 else None
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        step()
    stop.record()
    barrier(world)
    elapsed_ms = max_over_ranks(start.elapsed_time(stop), world, device)
    clock_info = clocks.stop() if clocks else None
    launches = _cabi.launch_count() - launches0

    # Per-stage CUDA-event times: a pass over (up to) 8 of this rank's views on ONE stream, right after the
    # timed region, so that a stage's time is that of its kernels running alone (in the timed region
    # the views of a rank overlap on several streams, which stretches every kernel).
    stage_views = my_views[:8]
    n_streams = trainer.n_streams
    trainer.n_streams = 1
    # first the same pass without the stage timers: the workload with ONE view in flight, as the reference's trainer
    # runs it (one view per optimizer step)
    trainer.buffers.zero_()
    for vi in stage_views[:2]:
        trainer.run_view(wl["views"][vi], gi_dev, ga_dev, view_index=vi)
    torch.cuda.synchronize()
    sv_start, sv_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sv_clocks = ClockSampler(local) if rank == 0 else None
    sv_reps = 3
    sv_start.record()
    for _ in range(sv_reps):
        for vi in stage_views:
            trainer.run_view(wl["views"][vi], gi_dev, ga_dev, view_index=vi)
    sv_stop.record()
    torch.cuda.synchronize()
    sv_ms = sv_start.elapsed_time(sv_stop) / max(len(stage_views) * sv_reps, 1)
    sv_clock_info = sv_clocks.stop() if sv_clocks else None
    _cabi.profile_read(reset=True)
    _cabi.profile_enable(True)
    trainer.buffers.zero_()
    for vi in stage_views:
        trainer.run_view(wl["views"][vi], gi_dev, ga_dev, view_index=vi)
    torch.cuda.synchronize()
    _cabi.profile_enable(False)
    stages = _cabi.profile_read(reset=True)
    trainer.n_streams = n_streams

    # instance / visible counts of this rank's views, for the algorithmic-byte model
    from inpc_b200 import rasterization as R
    n_inst, n_vis = [], []
    for vi in my_views[:4]:
        trainer.sampler.set_rng_state(vi)
        t = wl["tree"]
        pos, _ = trainer.sampler.generate_training_samples(t.centers, t.levels, t.weights, wl["views"][vi], args.points, t.initial_size)
        st = R.forward_with_state(pos, wl["features"], wl["opacities"], R.INPCRasterizer.extract_settings(wl["views"][vi], 0), args.tile)[3]
        n_inst.append(int(st.n_instances))
        n_vis.append(int(st.n_visible))
    torch.cuda.synchronize()

    # ---- end to end through the public API: host camera + host upstream gradient in, loss out
    pinned_gi = wl["grad_image"].pin_memory()
    pinned_ga = wl["grad_alpha"].pin_memory()
    pinned_views = [(v.w2c.pin_memory(), v.position.pin_memory()) for v in wl["views_host"]]
    loss_host = torch.zeros(max(args.views, 2), dtype=torch.float32).pin_memory()
    from inpc_b200.views import View
    copy_stream = torch.cuda.Stream(device=device)

    def host_inputs(vi, stream):
        # this view's inputs come from pinned host memory on a copy stream of their own, so that the copies run
        # ahead of, and under, the kernels of the views in flight
        # (the camera first: sampling and the forward pass wait for it alone, the backward pass for the gradients)
        with torch.cuda.stream(copy_stream):
            w2c, cpos = pinned_views[vi]
            w2c_d, cpos_d = w2c.to(device, non_blocking=True), cpos.to(device, non_blocking=True)
            camera_copied = torch.cuda.Event()
            camera_copied.record(copy_stream)
            gi = pinned_gi.to(device, non_blocking=True)
            ga = pinned_ga.to(device, non_blocking=True)
            grads_copied = torch.cuda.Event()
            grads_copied.record(copy_stream)
        stream.wait_event(camera_copied)
        for tensor in (gi, ga, w2c_d, cpos_d):
            tensor.record_stream(stream)
        return View(wl["views_host"][vi].camera, w2c_d, cpos_d), gi, ga, grads_copied

    # The step's result (the loss of the shard's last view) is read back every step, one step late: the copy into
    # pinned memory is enqueued behind the step and waited for while the next step's kernels are already queued, the
    # way a trainer logs its loss.  Every read-back lies inside the timed region; the last one is waited for before
    # the clock stops.
    loss_ready = [torch.cuda.Event(), torch.cuda.Event()]
    losses = []

    def e2e_enqueue(k):
        copy_stream.wait_stream(torch.cuda.current_stream())
        out = trainer.run_batch(wl["views"], None, rank, world, inputs=host_inputs)
        if out is not None:
            loss = (out[0].detach() * gi_dev).sum() + (out[1].detach() * ga_dev).sum()
            loss_host[k % 2: k % 2 + 1].copy_(loss.reshape(1), non_blocking=True)
        loss_ready[k % 2].record()

    def e2e_collect(k):
        loss_ready[k % 2].synchronize()
        losses.append(float(loss_host[k % 2].item()))

    # warm-up: as many steps as the device-resident leg gets, so that the caching allocator has reached its steady state
    # (every view brings fresh device tensors for its inputs, released only when the view's stream is through with them)
    for k in range(max(args.warmup, 3)):
        e2e_enqueue(k)
        e2e_collect(k)
    torch.cuda.synchronize()
    barrier(world)
    t0 = time.perf_counter()
    e2e_marks = [t0]
    for k in range(args.steps):
        e2e_enqueue(k)
        if k > 0:
            e2e_collect(k - 1)
            e2e_marks.append(time.perf_counter())   # step k - 1 has delivered its result
    e2e_collect(args.steps - 1)
    torch.cuda.synchronize()
    e2e_marks.append(time.perf_counter())
    barrier(world)
    e2e_s = max_over_ranks(time.perf_counter() - t0, world, device)
    e2e_step_ms = [round((b - a) * 1e3, 2) for a, b in zip(e2e_marks[:-1], e2e_marks[1:])]

    # values every rank count must reproduce: the reduced buffers of the last step (identical views, identical
    # per-view random streams, so only the order of floating-point sums differs between N = 1, 2, 4, 8)
    app = trainer.buffers.appearance.double()
    check = {"leaf_max": float(trainer.buffers.leaf.max_sampled.max().item()),
             "leaf_max_sum": float(trainer.buffers.leaf.max_sampled.double().sum().item()),
             "appearance_sum": float(app.sum().item()), "appearance_abs_sum": float(app.abs().sum().item())}

    if world > 1:
        import torch.distributed as dist
        gathered = [None] * world
        dist.all_gather_object(gathered, (n_inst, n_vis))
        n_inst = [x for g in gathered for x in g[0]]
        n_vis = [x for g in gathered for x in g[1]]
    if rank != 0:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()
        return

    total_points = args.steps * args.views * args.points
    value = total_points / (elapsed_ms * 1e-3) / 1e6
    e2e_value = total_points / e2e_s / 1e6
    peaks = {}
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    if peaks_path.exists():
        peaks = json.loads(peaks_path.read_text())
    peak_gbs = float(peaks.get("hbm_gbs", 6650.0))
    peak_kind = "measured" if "hbm_gbs" in peaks else "fallback"

    mean_i = statistics.mean(n_inst) if n_inst else 0.0
    mean_v = statistics.mean(n_vis) if n_vis else 0.0
    P = wl["H"] * wl["W"]
    c = 4
    alg = {   # algorithmic bytes per launch
        "blend_fwd": mean_i * (4 + 4 + 8 + 4 * c) + P * 4 * (c + 1) + mean_v * 8,
        "blend_bwd": mean_i * (16 + 4 * c) + P * 4 * (2 * c + 2) + mean_v * 8 * (c + 1),
        "sort_depth": mean_v * (4 + 4 * 16),
        "preprocess": args.points * (12 + 12 + 72) + mean_v * (32 + 4 * c + 4 + 8),
    }
    views_timed = max(len(stage_views), 1)
    per_stage = {k: {"ms_per_view": ms / views_timed, "scopes": n} for k, (ms, n) in stages.items()}
    dominant = max(alg, key=lambda k: stages[k][0])
    dom_ms = stages[dominant][0] / views_timed
    achieved = alg[dominant] / (dom_ms * 1e-3) / 1e9 if dom_ms > 0 else 0.0
    roofline = {"bound": "hbm", "kernel": dominant, "achieved": achieved, "peak": peak_gbs, "unit": "GB/s",
                "frac": achieved / peak_gbs if peak_gbs else None, "peak_source": peak_kind,
                "traffic": TRAFFIC_BYTES_PER_INSTANCE[dominant] * mean_i if dominant in TRAFFIC_BYTES_PER_INSTANCE and args.tile == 8 else None,
                "traffic_source": "ncu capture at 2^22 points scaled by the instance count",
                "algorithmic_bytes_per_launch": alg[dominant], "launch_ms": dom_ms}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": config_dict(args),
        "parallelism": f"view-dp{world}", "streams_per_rank": args.streams, "tile": args.tile,
        "frames_per_s": args.steps * args.views / (elapsed_ms * 1e-3),
        "ms_per_view": elapsed_ms / args.steps / max(len(my_views), 1),
        "e2e": {"value": e2e_value, "unit": UNIT,
                "h2d_bytes_per_step": args.views * (5 * P * 4 + 16 * 4 + 3 * 4), "d2h_bytes_per_step": 4 * world,
                "readback": "loss of every step copied to pinned memory behind the step and waited for one step later",
                "step_ms": e2e_step_ms},
        "gpu_launches": launches,
        "clocks": clock_info,
        "roofline": roofline,
        "stages": per_stage,
        "stage_timing": "CUDA events around each stage, one-stream pass over 8 views directly after the timed region",
        "single_view": {"value": args.points / (sv_ms * 1e-3) / 1e6, "unit": UNIT, "ms_per_view": sv_ms, "frames_per_s": 1e3 / sv_ms,
                        "views": len(stage_views) * sv_reps, "clocks": sv_clock_info,
                        "what": "the same workload with one view in flight (one stream, as the reference's trainer runs it), CUDA events"},
        "check": check,
        "instances_per_view": mean_i, "visible_per_view": mean_v,
    }
    if world == 1 and not args.no_side:
        side = {}
        for name in ("config2", "config4", "config4_rows32", "rows16", "rows32", "multisample4", "multisample4_batched"):
            try:
                torch.cuda.empty_cache()
                side[name] = side_workload(name, args.tile, warmup=3, reps=6, points=args.points)
            except Exception as e:   # side numbers never cost the bench line
                side[name] = {"failed": repr(e)}
        line["side"] = side
    if world == 1 and not args.no_cpu_baseline:
        try:
            line["cpu_baseline"] = cpu_baseline(args)
        except Exception as e:   # the baseline is a side number: never lose the bench line over it
            line["cpu_baseline"] = {"value": None, "unit": UNIT, "cores": os.cpu_count(), "kind": "port", "sample": f"failed: {e!r}"}
    print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------------
def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return                                   # the reference is single-GPU: rank 0 alone runs it
    sys.path.insert(0, str(ROOT / "oracle"))
    import ref_backend as RB
    base = {"impl": "reference", "metric": METRIC, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": max(args.warmup, 3),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config_dict(args),
            "parallelism": "single GPU, one view at a time on the legacy default stream (the reference has no multi-GPU path and no streams)",
            "tile": 8}
    import torch
    if not RB.available() or not torch.cuda.is_available():
        # no compiled reference backend (or no GPU): time the CPU restatement on a bounded sample
        cb = cpu_baseline(args)
        base.update(value=cb["value"], ms_per_step=args.views * args.points / (cb["value"] * 1e6) * 1e3, cpu_baseline=cb,
                    e2e={"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
        print(json.dumps(base))
        return

    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    wl = build_workload(args, device)
    t = wl["tree"]
    gi_dev, ga_dev = wl["grad_image"].to(device), wl["grad_alpha"].to(device)
    opac_flat = wl["opacities"].reshape(-1).contiguous()
    RB.sampler_seed(0)

    def view_step(view, gi, ga):
        pos, idx, _ = RB.training_samples(view, t.centers, t.levels, t.weights, args.points, t.initial_size, sync=False)
        img, alpha, bw = RB.forward(view, 0, pos, wl["features"], opac_flat, sync=False)
        RB.backward(view, 0, gi, ga, img, alpha, pos, opac_flat, sync=False)
        return img, alpha

    def step():
        for v in wl["views"]:
            view_step(v, gi_dev, ga_dev)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    clocks = ClockSampler(0)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    clock_info = clocks.stop()

    pinned_gi, pinned_ga = wl["grad_image"].pin_memory(), wl["grad_alpha"].pin_memory()
    pinned_views = [(v.w2c.pin_memory(), v.position.pin_memory()) for v in wl["views_host"]]
    loss_host = torch.zeros(1, dtype=torch.float32).pin_memory()
    from inpc_b200.views import View

    def e2e_step():
        for vi in range(args.views):
            gi = pinned_gi.to(device, non_blocking=True)
            ga = pinned_ga.to(device, non_blocking=True)
            w2c, cpos = pinned_views[vi]
            view = View(wl["views_host"][vi].camera, w2c.to(device, non_blocking=True), cpos.to(device, non_blocking=True))
            img, alpha = view_step(view, gi, ga)
            loss = (img * gi).sum() + (alpha * ga).sum()
            loss_host.copy_(loss.reshape(1), non_blocking=True)
        torch.cuda.synchronize()

    e2e_step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    e2e_s = time.perf_counter() - t0

    total_points = args.steps * args.views * args.points
    P = wl["H"] * wl["W"]
    base.update(value=total_points / elapsed / 1e6, ms_per_step=elapsed / args.steps * 1e3,
                frames_per_s=args.steps * args.views / elapsed, ms_per_view=elapsed / args.steps / args.views * 1e3,
                clocks=clock_info,
                cpu_baseline={"value": total_points / elapsed / 1e6, "unit": UNIT, "cores": 0, "kind": "reference",
                              "sample": "the reference's own CUDA backend (it has no CPU implementation of this path), "
                                        "compiled unmodified for sm_100a, full workload on one B200"},
                e2e={"value": total_points / e2e_s / 1e6, "unit": UNIT,
                     "h2d_bytes_per_step": args.views * (5 * P * 4 + 16 * 4 + 3 * 4), "d2h_bytes_per_step": args.views * 4},
                single_view={"value": total_points / elapsed / 1e6, "unit": UNIT, "ms_per_view": elapsed / args.steps / args.views * 1e3,
                             "frames_per_s": args.steps * args.views / elapsed, "views": args.views, "clocks": clock_info,
                             "what": "the reference always has one view in flight: this is its timed region"})
    if not args.no_side:
        side = {}
        del wl
        for name in ("config2", "config4", "config4_rows32", "rows16", "rows32", "multisample4", "multisample4_batched"):
            try:
                torch.cuda.empty_cache()
                side[name] = side_workload(name, 8, warmup=3, reps=6, points=args.points, impl="reference")
            except Exception as e:
                side[name] = {"failed": repr(e)}
        base["side"] = side
    print(json.dumps(base))


# ---------------------------------------------------------------------------------------------------
SIDE_METRICS = {
    "config2": ("frames/s", "render_preextracted frames/s at 2^25 points, 1920x1080 (config 2)"),
    "multisample4": ("frames/s", "multisampled inference frames/s, 4 sets of 2^23 expected samples of config 1, one stream per set"),
    "multisample4_batched": ("frames/s", "multisampled inference frames/s, 4 sets of 2^23 expected samples of config 1, two batched renders of two sets on two streams"),
    "config4": (UNIT, "fwd+bwd Mpoints/s at 2^24 skewed points, 3840x2160, 36 x fp16 SH -> 4 channels (config 4 in the reference's layout)"),
    "config4_rows32": (UNIT, "fwd+bwd Mpoints/s at 2^24 skewed points, 3840x2160, 32 fp32 channels (config 4 as stated)"),
    "rows16": (UNIT, "fwd+bwd Mpoints/s at 2^23 points per view, 1237x822, 16 fp32 channels, incl. sampling"),
    "rows32": (UNIT, "fwd+bwd Mpoints/s at 2^23 points per view, 1237x822, 32 fp32 channels, incl. sampling"),
}


def side_workload(name: str, tile: int, warmup: int, reps: int, points: int = N_POINTS, impl: str = "ours") -> dict:
    """One single-GPU side measurement (device-timed with CUDA events, inputs resident in HBM, one call in flight):
    config2         pre-extracted inference, 2^25 points, 1920x1080                      -> frames/s
    config4         skewed stress case, 2^24 points, 3840x2160, fwd+bwd, SH layout       -> Mpoints/s
    config4_rows32  the same with 32 fp32 feature channels                               -> Mpoints/s
    rows16 / rows32 config 1 with (N,C) fp32 feature rows, fwd+bwd incl. sampling        -> Mpoints/s
    multisample4 / multisample4_batched   inference over 4 sample sets of config 1's octree (raw 37-half features,
                    accumulate + background compose): one render per set on 4 streams / two batched renders on 2 streams -> frames/s
    impl = "reference" runs the reference's own CUDA backend where it can (config 2)."""
    import torch
    import synthetic_workloads as syn
    unit, metric = SIDE_METRICS[name]
    device = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator().manual_seed(5)
    if impl == "reference":
        if name not in ("config2", "multisample4"):
            why = ("the reference's 16-bit tile key overflows at 3840x2160 (129,600 tiles of 8x8 pixels)" if name.startswith("config4")
                   else "the reference has no batched multi-set render" if name.startswith("multisample")
                   else "the reference has no fp32 feature-row layout")
            return {"metric": metric, "unavailable": why}
        sys.path.insert(0, str(ROOT / "oracle"))
        import ref_backend as RB
        if name == "config2":
            c = syn.config2()
            view, pos, feats = c["view"].to(device), c["positions"].to(device), c["features"].to(device)
            opac = c["opacities"].to(device).reshape(-1).contiguous()
            n_points = pos.shape[0]

            def step():
                RB.render_preextracted(view, 0, pos, feats, opac, None, 1.0, 3.0, sync=False)
        else:
            # the reference's own loop (Renderer.py:99-125): one render per set on the default stream, then accumulate
            # and compose; the sets are the ones this library's sampler draws for the other arm
            from inpc_b200.compose import MultisampleAccumulator
            from inpc_b200.sampling import ProbabilityFieldSampler
            c = syn.config1(n_samples=points, n_leaves=N_LEAVES)
            view, tree = c["view"].to(device), c["tree"].to(device)
            del c
            sampler = ProbabilityFieldSampler(0)
            gd = torch.Generator(device=device).manual_seed(3)
            sets = []
            for _ in range(4):
                pos = sampler.generate_expected_samples(tree.centers, tree.levels, tree.weights, view, points, 1, tree.initial_size)
                sets.append((pos, (torch.randn((pos.shape[0], 37), generator=gd, device=device) * 0.5).to(torch.float16)))
            n_points = sum(p.shape[0] for p, _ in sets)
            bg = torch.zeros((4, view.camera.height, view.camera.width), device=device)

            def step():
                acc = MultisampleAccumulator(len(sets), True)
                for p, raw in sets:
                    acc.add(*RB.render(view, 0, p, raw, 1.0, 3.0))
                acc.resolve(bg)
    else:
        import inpc_b200
        from inpc_b200.sampling import ProbabilityFieldSampler
        rast = inpc_b200.INPCRasterizer(tile_size=tile)
        if name == "config2":
            c = syn.config2()
            view, pos, feats, opac = c["view"].to(device), c["positions"].to(device), c["features"].to(device), c["opacities"].to(device)
            n_points = pos.shape[0]

            def step():
                rast.render_preextracted(view, 0, pos, feats, opac)
        elif name in ("multisample4", "multisample4_batched"):
            from inpc_b200.compose import render_multisampled
            c = syn.config1(n_samples=points, n_leaves=N_LEAVES)
            view, tree = c["view"].to(device), c["tree"].to(device)
            del c
            sampler = ProbabilityFieldSampler(0)
            gd = torch.Generator(device=device).manual_seed(3)
            sets = []
            for _ in range(4):
                pos = sampler.generate_expected_samples(tree.centers, tree.levels, tree.weights, view, points, 1, tree.initial_size)
                sets.append((pos, (torch.randn((pos.shape[0], 37), generator=gd, device=device) * 0.5).to(torch.float16)))
            n_points = sum(p.shape[0] for p, _ in sets)
            bg = torch.zeros((4, view.camera.height, view.camera.width), device=device)
            batched = name.endswith("batched")

            def step():
                render_multisampled(rast, view, 0, sets, bg, n_streams=2 if batched else 4, batched=batched)
        elif name in ("config4", "config4_rows32"):
            c = syn.config4()
            view, pos, opac = c["view"].to(device), c["positions"].to(device), c["opacities"].to(device)
            H, W = view.camera.height, view.camera.width
            n_points = pos.shape[0]
            ga = (torch.randn((1, H, W), generator=g) * 1e-3).to(device)
            if name == "config4":
                feats = c["features"].to(device)
                gi = (torch.randn((4, H, W), generator=g) * 1e-3).to(device)

                def step():
                    f, o = feats.detach().requires_grad_(True), opac.detach().requires_grad_(True)
                    im, al, _ = rast(view, 0, pos, f, o)
                    torch.autograd.backward([im, al], [gi, ga])
            else:
                del c
                feats = (torch.randn((n_points, 32), generator=g) * 0.5).to(device)
                gi = (torch.randn((32, H, W), generator=g) * 1e-3).to(device)

                def step():
                    f, o = feats.detach().requires_grad_(True), opac.detach().requires_grad_(True)
                    im, al, _ = rast.forward_rows(view, pos, f, o)
                    torch.autograd.backward([im, al], [gi, ga])
        else:
            channels = 16 if name == "rows16" else 32
            c = syn.config1(n_samples=points, n_leaves=N_LEAVES)
            view, tree, opac = c["view"].to(device), c["tree"].to(device), c["opacities"].to(device)
            del c
            feats = (torch.randn((points, channels), generator=g) * 0.5).to(device)
            H, W = view.camera.height, view.camera.width
            gi, ga = (torch.randn((channels, H, W), generator=g) * 1e-3).to(device), (torch.randn((1, H, W), generator=g) * 1e-3).to(device)
            sampler = ProbabilityFieldSampler(0)
            n_points = points

            def step():
                pos, _ = sampler.generate_training_samples(tree.centers, tree.levels, tree.weights, view, points, tree.initial_size)
                f, o = feats.detach().requires_grad_(True), opac.detach().requires_grad_(True)
                im, al, _ = rast.forward_rows(view, pos, f, o)
                torch.autograd.backward([im, al], [gi, ga])

    for _ in range(max(warmup, 3)):
        step()
    torch.cuda.synchronize()
    clocks = ClockSampler(device.index or 0)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        step()
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / reps
    clock_info = clocks.stop()
    value = 1e3 / ms if unit == "frames/s" else n_points / (ms * 1e-3) / 1e6
    return {"metric": metric, "value": value, "unit": unit, "ms": ms, "reps": reps, "points": n_points, "clocks": clock_info}


def run_side_workload(args):
    """`--workload X`: one side measurement as a JSON line of its own."""
    import torch
    if int(os.environ.get("RANK", "0")) != 0:
        return
    torch.cuda.set_device(0)
    r = side_workload(args.workload, args.tile, warmup=args.warmup, reps=max(args.steps, 1) * 8, points=args.points, impl=args.impl)
    line = {"metric": r["metric"], "n_gpus": 1, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": {"workload": args.workload, "tile": args.tile, "l2": "inputs exceed the 126 MB L2; no flush needed"}}
    if args.impl == "reference":
        line["impl"] = "reference"
    line.update({k: v for k, v in r.items() if k != "metric"})
    if "ms" in r:
        line.update(steps=r["reps"], warmup=max(args.warmup, 3), ms_per_step=r["ms"])
    print(json.dumps(line))


def main():
    args = parse_args()
    if args.workload != "config1":
        run_side_workload(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
