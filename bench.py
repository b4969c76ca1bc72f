#!/usr/bin/env python3
"""Benchmark of the splat rasterizer hot path: forward + backward of one 1920x1080 view of 1M degree-3
splats (config 1 of BASELINE.json), reported as whole-job views/s (``fwd_bwd_ms_per_view`` is fwd+bwd ms/iter).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c1]

One process per GPU (torchrun for N > 1).  Each step every rank renders ``--views-per-rank`` views of
the replicated cloud (forward, backward with gradient accumulation into one flat 59-float-per-splat
buffer) and, for N > 1, all ranks sum that buffer with one NCCL all-reduce: weak scaling, per-GPU work
fixed.  Rank 0 prints ONE JSON line.

  value      device-timed throughput (CUDA events, barrier + synchronize on both sides, max over ranks)
             of the fused C-ABI calls with all inputs resident in HBM;
  e2e        the same step through the public Python operator (GaussianRasterizer + autograd) with the
             step's inputs (camera, upstream image gradient) copied from pinned host memory and the
             rendered image + radii copied back inside the timed region;
  roofline   the dominant kernel (backward blend), timed live with cudaEvent pairs the library records
             around each stage while the same steps run again;
  cpu_baseline  the C++/OpenMP restatement of the reference's algorithm (oracle/), one full view, all
             host threads -- a reported baseline, not the target;
  --impl reference  times that CPU restatement as the reference arm (the reference ships no CPU path
             and cannot be pip-installed here; its own CUDA kernels, built under oracle/_ref, are
             reported beside it as ``reference_cuda`` when that library is present).
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

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "training views/s (fwd+bwd), 1M splats SH-3 @1920x1080 (fwd_bwd_ms_per_view = fwd+bwd ms/iter)"
UNIT = "views/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c1", choices=["c0", "c1", "c2", "c3", "c4"])
    ap.add_argument("--views-per-rank", type=int, default=8,
                    help="views each rank renders per step before the gradient all-reduce (64-view batch on 8 GPUs)")
    ap.add_argument("--view-streams", type=int, default=2,
                    help="streams the per-view stages of a step's views are dealt over (1 = one after the other)")
    ap.add_argument("--splats", type=int, default=0, help="override the workload's splat count (debugging)")
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-reference-cuda", action="store_true")
    ap.add_argument("--skip-optimizer", action="store_true")
    return ap.parse_args()


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons every 100 ms while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu_index)], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, sm_max, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); sm_max.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(sm_max) if sm_max else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def load_scene(args):
    from ds_splat_b200 import scenes
    kw = {}
    if args.splats:
        kw["n"] = args.splats
    return scenes.CONFIGS[args.workload](**kw)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json, copy bandwidth)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


def oracle_one_view(scene, view, v_image):
    """One forward+backward of the CPU restatement; returns (seconds, forward dict, backward dict)."""
    from oracle import oracle as O
    cam = O.Camera(view=view.view, proj=view.proj, campos=view.campos, tanfovx=view.tanfovx, tanfovy=view.tanfovy,
                   H=view.H, W=view.W, sh_degree=scene.sh_degree)
    t0 = time.perf_counter()
    fwd = O.forward(cam, scene.means, scene.shs, scene.opacities, scene.scales, scene.rotations)
    bwd = O.backward(cam, fwd, scene.means, scene.shs, scene.opacities, scene.scales, scene.rotations, v_image)
    return time.perf_counter() - t0, fwd, bwd


def reference_cuda_numbers(scene, view, v_image):
    """Per-stage milliseconds of the reference's own CUDA kernels (oracle/_ref), or None when not built."""
    try:
        from oracle import ref_cuda
        if not ref_cuda.available():
            return None
        r = ref_cuda.run(view, scene.means, scene.shs, scene.opacities, scene.scales, scene.rotations, v_image=v_image,
                         iters=20, warmup=5, outputs=False)
        return {"fwd_ms": round(r["ms_forward"], 4), "bwd_ms": round(r["ms_backward"], 4),
                "fwd_bwd_ms": round(r["ms_forward"] + r["ms_backward"], 4), "K": r["K"],
                "stages_ms": {k: round(v, 4) for k, v in r["ms"].items()},
                "note": "reference kernels + thrust, -O3 --use_fast_math, sm_100a, buffers preallocated, device-timed"}
    except Exception as e:  # the checker must never take the benchmark down
        return {"unavailable": f"{type(e).__name__}: {e}"}


def run_reference_arm(args):
    """CPU restatement of the reference's algorithm, all host threads, one full view per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as O
    scene = load_scene(args)
    view = scene.views[0]
    v_image = scene.image_grad()
    steps, warmup = max(1, min(args.steps, 5)), max(0, min(args.warmup, 1))
    for _ in range(warmup):
        oracle_one_view(scene, view, v_image)
    times = [oracle_one_view(scene, view, v_image)[0] for _ in range(steps)]
    sec = sum(times) / len(times)
    value = 1.0 / sec
    cores = O.num_threads()
    line = {"impl": "reference", "metric": METRIC, "value": round(value, 5), "unit": UNIT, "n_gpus": args.gpus,
            "steps": steps, "warmup": warmup, "ms_per_step": round(sec * 1e3, 2), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{scene.name}: {scene.n} splats SH-3, {view.W}x{view.H}, one view fwd+bwd",
                       "note": "the reference has no CPU path; this is the C++/OpenMP restatement of its algorithm (oracle/)"},
            "cpu_baseline": {"value": round(value, 5), "unit": UNIT, "cores": cores, "kind": "port",
                             "sample": f"{steps} full views of the workload (steps clamped to 5)"},
            "e2e": {"value": round(value, 5), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    try:
        import torch
        if torch.cuda.is_available():
            line["reference_cuda"] = reference_cuda_numbers(scene, view, v_image)
    except Exception:
        pass
    print(json.dumps(line), flush=True)


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    from ds_splat_b200 import GaussianRasterizationSettings, GaussianRasterizer, _capi
    from ds_splat_b200.dp import CameraTensors, GradientBuffer, ViewRenderer, data_parallel_step

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the rasterizer has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    json_out = sys.stdout
    if world > 1:
        # Libraries below write to file descriptor 1 (NCCL prints its version there): keep a private copy of it
        # for the one JSON line and point descriptor 1 at stderr for everything else.
        sys.stdout.flush()
        json_out = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)
        dist.init_process_group("nccl", device_id=dev)
    _capi.lib()  # fail loudly if the library is missing

    scene = load_scene(args)
    view = scene.views[0]
    H, W = view.H, view.W
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    params = dict(means3d=t(scene.means), shs=t(scene.shs), opacities=t(scene.opacities), scales=t(scene.scales),
                  rotations=t(scene.rotations))
    vpr = max(1, args.views_per_rank)
    # Cameras are dealt to ranks in blocks of vpr; a scene with a single camera (config 1) gives every rank that one.
    view_ids = [(rank * vpr + j) % len(scene.views) for j in range(vpr)]
    cams = [CameraTensors.from_view(scene.views[v], dev) for v in view_ids]
    v_images_host = [scene.image_grad(v, seed=7 + rank * vpr + j) for j, v in enumerate(view_ids)]
    view = scene.views[view_ids[0]]
    v_images = [t(v) for v in v_images_host]
    renderer = ViewRenderer(**params, sh_degree=scene.sh_degree, view_streams=args.view_streams)
    grads = GradientBuffer(scene.n, dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step():
        data_parallel_step(renderer, cams, v_images, grads)

    # ---- device-timed throughput ------------------------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = _capi.launch_count()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    elapsed_ms = ev0.elapsed_time(ev1)
    launches = _capi.launch_count() - launches0
    clocks = sampler.stop()
    tmax = torch.tensor([elapsed_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    elapsed_ms = float(tmax.item())
    ms_per_step = elapsed_ms / args.steps
    views_per_s = world * vpr * args.steps / (elapsed_ms * 1e-3)
    K_emitted = renderer.last_k
    # Pair count of the reference's own list for the same view (the renderer pairs a splat only with the tiles it can
    # contribute to, a subset with identical results): the algorithmic figures below are those of the reference's list.
    ref_lists = ViewRenderer(**params, sh_degree=scene.sh_degree, batch_views=1, tight_tiles=False)
    ref_lists.forward(cams[-1])
    torch.cuda.synchronize()
    K = ref_lists.last_k
    del ref_lists
    torch.cuda.empty_cache()

    # ---- per-stage timing of the same steps (events recorded by the library around each stage) ---------
    # The stages are timed with the views one after the other on one stream: with two views in flight the events
    # around one view's stage also cover the other view's kernels.
    lanes_used = renderer.view_streams
    renderer.view_streams = 1
    _capi.stage_timing(True)
    for _ in range(min(args.steps, 40)):
        step()
    torch.cuda.synchronize()
    stage_raw = _capi.read_stage_timings()
    _capi.stage_timing(False)
    renderer.view_streams = lanes_used
    # per view: the per-splat backward runs once for all views of a step, every other stage once per view
    timed_views = min(args.steps, 40) * vpr
    stages_ms = {name: round(ms / timed_views, 5) for name, (ms, calls) in stage_raw.items() if calls}

    # ---- the optimizer step that follows a training step (not part of the metric; reported beside it) ---------
    optimizer = None
    if world == 1 and not args.skip_optimizer:
        from ds_splat_b200.dp import FlatAdam
        scratch = {k: v.clone() for k, v in renderer.p.items()}   # the timed steps must not move the benchmark's scene
        opt = FlatAdam(scratch, dict(means3d=1.6e-4, shs=2.5e-3, opacities=5e-2, scales=5e-3, rotations=1e-3))
        for _ in range(3):
            opt.step(grads, grad_scale=1.0 / vpr)
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        ev0.record()
        for _ in range(20):
            opt.step(grads, grad_scale=1.0 / vpr)
        ev1.record()
        torch.cuda.synchronize()
        adam_ms = ev0.elapsed_time(ev1) / 20
        adam_bytes = 28 * grads.flat.numel()   # read p, g, m, v; write p, m, v
        optimizer = {"kernel": "adam_kernel (5 launches, one per parameter tensor)", "ms_per_step": round(adam_ms, 4),
                     "achieved_GBps": round(adam_bytes / (adam_ms * 1e-3) / 1e9, 1), "algorithmic_bytes": int(adam_bytes)}
        del scratch, opt
        # ... and the photometric loss between forward and backward (L1 + D-SSIM and its gradient, two launches)
        from ds_splat_b200.dp import ImageLoss
        loss_fn = ImageLoss(lambda_dssim=0.2)
        img = renderer.forward(cams[-1]).clone()
        tgt = torch.rand_like(img)
        for _ in range(3):
            loss_fn.gradient(img, tgt)
        torch.cuda.synchronize()
        ev0.record()
        for _ in range(20):
            loss_fn.gradient(img, tgt)
        ev1.record()
        torch.cuda.synchronize()
        loss_ms = ev0.elapsed_time(ev1) / 20
        loss_bytes = 4 * 3 * H * W * (2 + 3 + 3 + 2 + 1)   # read x, y; write 3 maps; read 3 maps, x, y; write dL/dx
        optimizer["image_loss"] = {"kernels": "ssim_moments_kernel + ssim_gradient_kernel", "ms_per_view": round(loss_ms, 4),
                                   "achieved_GBps": round(loss_bytes / (loss_ms * 1e-3) / 1e9, 1),
                                   "algorithmic_bytes": int(loss_bytes)}
        del loss_fn, img, tgt
        torch.cuda.empty_cache()

    # ---- end to end through the public operator, host buffers -----------------------------------------
    e2e = None
    if not args.skip_e2e:
        pinned_grad = torch.from_numpy(v_images_host[0]).pin_memory()
        pinned_view = torch.from_numpy(view.viewmatrix_t).pin_memory()
        pinned_proj = torch.from_numpy(view.projmatrix_t).pin_memory()
        pinned_pos = torch.from_numpy(np.ascontiguousarray(view.campos)).pin_memory()
        out_image = torch.empty((H, W, 3), dtype=torch.float32).pin_memory()
        out_radii = torch.empty(scene.n, dtype=torch.int32).pin_memory()
        leaves = {k: v.clone().requires_grad_(True) for k, v in params.items()}
        means2d = torch.zeros_like(leaves["means3d"], requires_grad=True)
        bg = torch.zeros(3, device=dev)
        h2d = pinned_grad.numel() * 4 + (16 + 16 + 3) * 4
        d2h = out_image.numel() * 4 + out_radii.numel() * 4

        copy_stream = torch.cuda.Stream(device=dev)

        def e2e_step():
            # A training loop's usual overlap: the image gradient travels to the device while the forward
            # runs, the rendered image travels back while the backward runs (second stream, events).
            main = torch.cuda.current_stream()
            vm = pinned_view.to(dev, non_blocking=True)
            pm = pinned_proj.to(dev, non_blocking=True)
            cp = pinned_pos.to(dev, non_blocking=True)
            with torch.cuda.stream(copy_stream):
                vg = pinned_grad.to(dev, non_blocking=True)
                grad_ready = torch.cuda.Event()
                grad_ready.record(copy_stream)
            settings = GaussianRasterizationSettings(H, W, view.tanfovx, view.tanfovy, bg, 1.0, vm, pm, scene.sh_degree, 3,
                                                     cp, False, False)
            for leaf in list(leaves.values()) + [means2d]:
                leaf.grad = None
            image, radii = GaussianRasterizer(settings)(leaves["means3d"], means2d, leaves["shs"], None, leaves["opacities"],
                                                        leaves["scales"], leaves["rotations"], None)
            rendered = torch.cuda.Event()
            rendered.record(main)
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(rendered)
                out_image.copy_(image.detach(), non_blocking=True)
                out_radii.copy_(radii, non_blocking=True)
            image.record_stream(copy_stream)
            radii.record_stream(copy_stream)
            main.wait_event(grad_ready)
            vg.record_stream(main)
            image.backward(vg)
            torch.cuda.synchronize()  # the caller reads the result on the host every step

        for _ in range(max(args.warmup, 3)):
            e2e_step()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        wall0 = time.perf_counter()
        a.record()
        for _ in range(args.steps):
            e2e_step()
        b.record()
        barrier()
        wall = time.perf_counter() - wall0
        e_ms = max(a.elapsed_time(b), wall * 1e3)  # host work between kernels counts: take the slower clock
        tm = torch.tensor([e_ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        e2e = {"value": round(world * args.steps / (float(tm.item()) * 1e-3), 3), "unit": UNIT,
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
               "ms_per_step": round(float(tm.item()) / args.steps, 4),
               "note": "GaussianRasterizer + autograd; per step H2D camera + dL/dimage from pinned memory, D2H image + radii; "
                       "splat parameters are model state resident on the device"}
        del leaves, means2d

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- CPU baseline + roofline (rank 0) -----------------------------------------------------------
    cpu_baseline, pairs_bwd, pairs_fwd = None, None, None
    if world == 1 and not args.skip_cpu_baseline:
        from oracle import oracle as O
        sec, fwd_o, bwd_o = oracle_one_view(scene, view, v_images_host[0])
        pairs_fwd, pairs_bwd = fwd_o["pairs_fwd"], bwd_o["pairs_bwd"]
        cpu_baseline = {"value": round(1.0 / sec, 5), "unit": UNIT, "cores": O.num_threads(), "kind": "port",
                        "sample": "one full view of the workload (forward + backward), C++/OpenMP restatement in oracle/",
                        "ms_per_view": round(sec * 1e3, 1)}
    reference_cuda = reference_cuda_numbers(scene, view, v_images_host[0]) if world == 1 and not args.skip_reference_cuda else None

    peak, peak_src = measured_peaks()
    if optimizer:
        optimizer["frac_of_hbm_peak"] = round(optimizer["achieved_GBps"] / peak, 4)
    dom = "blend_backward"
    dom_ms = stages_ms.get(dom)
    roofline, roofline_fp32 = None, None
    if dom_ms:
        # algorithmic bytes of one backward-blend launch: 8 B pair + 48 B record gathered per list entry,
        # 36 B of per-splat sums added per list entry, 20 B per pixel read (dL/dimage 12, final_T 4, final_idx 4),
        # plus the 48 B/splat zero fill of the accumulator that the stage includes.
        alg_bytes = K * (8 + 48 + 36) + 20 * H * W + 48 * scene.n
        achieved = alg_bytes / (dom_ms * 1e-3) / 1e9
        # DRAM bytes of one blend_backward_kernel launch from the ncu capture summarised in
        # profiles/blend_backward_c1.md (83,103,232 read + 4,211,712 written at config 1); it is dominated
        # by the pair list and the gathered records, so other workloads scale it by their pair count.
        traffic = int(87_314_944 * (K / 10_957_444))
        roofline = {"kernel": dom, "bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": "GB/s",
                    "frac": round(achieved / peak, 4), "traffic": traffic,
                    "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch on config 1, scaled by pairs",
                    "peak_source": peak_src,
                    "algorithmic_bytes": int(alg_bytes), "ms": dom_ms,
                    "note": "this kernel is bound by FP32/SHFL issue, not HBM; see roofline_fp32"}
        if pairs_bwd and clocks.get("sm_mhz"):
            flops = 74.0 * pairs_bwd
            fp32_peak = 148 * 128 * 2 * clocks["sm_mhz"] * 1e6 / 1e12
            roofline_fp32 = {"kernel": dom, "achieved": round(flops / (dom_ms * 1e-3) / 1e12, 3), "peak": round(fp32_peak, 2),
                             "unit": "TFLOP/s", "frac": round(flops / (dom_ms * 1e-3) / 1e12 / fp32_peak, 4),
                             "pairs": int(pairs_bwd), "flop_per_pair": 74,
                             "peak_source": "148 SMs x 128 FP32 lanes x 2 flop x median SM clock sampled during the run"}

    line = {"metric": METRIC, "value": round(views_per_s, 3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 4),
            "fwd_bwd_ms_per_view": round(ms_per_step / vpr, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{scene.name}: {scene.n} splats SH-3, {W}x{H}, {vpr} view(s) per rank per step, fwd+bwd"
                                   + (", gradient all-reduce of 59 floats/splat" if world > 1 else ""),
                       "pairs_K": int(K), "pairs_emitted": int(K_emitted), "tiles": view.num_tiles, "view_streams": int(min(args.view_streams, vpr)), "l2": "inputs larger than L2 (236 MB of parameters + "
                       "88 MB pair list per view; no explicit flush)", "parallelism": f"dp{world} (cameras sharded, splats replicated)"},
            "clocks": clocks, "gpu_launches": int(launches), "stages_ms": stages_ms, "roofline": roofline,
            "roofline_fp32": roofline_fp32, "cpu_baseline": cpu_baseline, "e2e": e2e, "reference_cuda": reference_cuda,
            "optimizer": optimizer,
            "pairs_evaluated": {"forward_per_pixel": pairs_fwd, "backward_per_pixel": pairs_bwd}}
    print(json.dumps(line), file=json_out, flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
