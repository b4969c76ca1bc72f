#!/usr/bin/env python3
"""Benchmark of the splat rasterizer hot path: training steps over 1920x1080 views of 1M degree-3 splats
(config 1 of BASELINE.json), reported as whole-job views/s, with the literal "fwd+bwd ms/iter" beside it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c1]

One process per GPU (torchrun for N > 1).  A step on every rank: forward + backward of ``--views-per-rank``
distinct cameras of the replicated cloud (gradients summed into one flat 59-float-per-splat block), then the
optimizer step with the gradient sum folded in -- reduce-scatter of the block over NCCL, Adam on the rank's 1/N
slice, all-gather of the parameters (plain Adam in a single process).  Weak scaling: per-GPU work is fixed.
Rank 0 prints ONE JSON line.

  value            device-timed throughput of those steps (CUDA events, barrier + synchronize on both sides, max
                   over ranks), all inputs resident in HBM; ``step_breakdown_ms`` splits a step into render,
                   gradient reduce-scatter, Adam and parameter all-gather;
  single_view_ms   the literal metric "fwd+bwd ms/iter @1M": ONE view per iteration through the fused single-view
                   calls (dsb_forward / dsb_backward), median over the iterations, for the default pair lists and
                   for ``strict_lists`` (tiles-touched counts, pair list and tile ranges bit-identical to the
                   reference's; the default pairs a splat only with tiles it can contribute to, a subset with
                   identical image, radii and gradients);
  strict_lists     the multi-view step again with the reference-identical lists;
  e2e              one training iteration per step through the public Python operator (GaussianRasterizer +
                   autograd): camera and 8-bit target image copied from pinned host memory, L1 loss (dp.ImageLoss), backward,
                   and the loss value read on the host, all inside the timed region;
  roofline         the dominant kernel (backward blend) on the configuration's own camera against the FP32 pipe
                   (148 SMs x 128 lanes x 2 flop x sampled SM clock), timed live with the cudaEvent pairs the
                   library records around each stage; ``roofline_hbm`` is the same launch against the measured
                   copy bandwidth;
  c3               config 3 (6M splats, 8 of its 64 ring cameras per rank and step, 1.416 GB of gradients) for a
                   few steps, so that the scaling curve of the configuration the multi-GPU metric names is on record;
  cpu_baseline     the C++/OpenMP restatement of the reference's algorithm (oracle/), one full view, all host
                   threads -- a reported baseline, not the target;
  --impl reference times that CPU restatement as the reference arm (the reference ships no CPU path and cannot be
                   pip-installed here; its own CUDA kernels, built under oracle/_ref, are reported beside it as
                   ``reference_cuda`` when that library is present).
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

METRIC = "training views/s (fwd+bwd+optimizer step), 1M splats SH-3 @1920x1080 (single_view_ms = fwd+bwd ms/iter)"
UNIT = "views/s"
LRS = dict(means3d=1.6e-4, shs=2.5e-3, opacities=5e-2, scales=5e-3, rotations=1e-3)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c1", choices=["c0", "c1", "c2", "c3", "c4", "flythrough"])
    ap.add_argument("--views-per-rank", type=int, default=8,
                    help="views each rank renders per step before the gradient reduction (64-view batch on 8 GPUs)")
    ap.add_argument("--view-streams", type=int, default=2,
                    help="streams the per-view stages of a step's views are dealt over (1 = one after the other)")
    ap.add_argument("--splats", type=int, default=0, help="override the workload's splat count (debugging)")
    ap.add_argument("--reduce", default="sharded", choices=["sharded", "allreduce"],
                    help="sharded: reduce-scatter + Adam on 1/N + all-gather; allreduce: all-reduce + Adam over everything")
    ap.add_argument("--no-nccl-registration", action="store_true")
    ap.add_argument("--row-binning", action="store_true",
                    help="build the pair lists by row binning (DSB_FLAG_ROW_BINNING) instead of writing and sorting the pairs")
    ap.add_argument("--skip-cpu-baseline", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-reference-cuda", action="store_true")
    ap.add_argument("--skip-optimizer", action="store_true", help="skip the separate Adam / image-loss kernel timings")
    ap.add_argument("--skip-c3", action="store_true")
    ap.add_argument("--skip-strict", action="store_true")
    ap.add_argument("--optimizer-chunks", type=int, default=1,
                    help="N > 1: cut the gradient/parameter blocks into this many chunks and pipeline reduce-scatter, Adam and "
                         "all-gather over two communicators (1: one reduce-scatter, one update, one all-gather)")
    ap.add_argument("--frames", type=int, default=120, help="frames of the fly-through workload")
    ap.add_argument("--image", default="", help="fly-through only: WIDTHxHEIGHT instead of 1920x1080 (same field of view)")
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


def load_scene(args, views: int = 1):
    from ds_splat_b200 import scenes
    kw = {}
    if args.splats:
        kw["n"] = args.splats
    name = "c1" if args.workload == "flythrough" else args.workload
    if args.workload == "flythrough" and args.image:
        w, h = (int(x) for x in args.image.lower().split("x"))
        kw.update(W=w, H=h, focal=1100.0 * w / 1920.0)
    if name == "c1":
        kw["views"] = views   # view 0 is the configuration's camera, the others are turned +-5 degrees away from it
    return scenes.CONFIGS[name](**kw)


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
    cores = O.use_all_host_threads()   # torchrun exports OMP_NUM_THREADS=1 to its workers
    scene = load_scene(args)
    view = scene.views[0]
    v_image = scene.image_grad()
    steps, warmup = max(1, min(args.steps, 5)), max(0, min(args.warmup, 1))
    for _ in range(warmup):
        oracle_one_view(scene, view, v_image)
    times = [oracle_one_view(scene, view, v_image)[0] for _ in range(steps)]
    sec = sum(times) / len(times)
    value = 1.0 / sec
    line = {"impl": "reference", "metric": METRIC, "value": round(value, 5), "unit": UNIT, "n_gpus": args.gpus,
            "steps": steps, "warmup": warmup, "ms_per_step": round(sec * 1e3, 2), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{scene.name}: {scene.n} splats SH-3, {view.W}x{view.H}, one view fwd+bwd",
                       "note": "the reference has no CPU path; this is the C++/OpenMP restatement of its algorithm (oracle/), "
                               "which has no optimizer step"},
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


def views_of_rank(num_views: int, rank: int, world: int, vpr: int):
    """The cameras of one step: world * vpr of the scene's views, evenly spaced over the whole set, dealt to the ranks
    round-robin (the library's dp.shard_views).  Every rank's batch spans the whole camera set at every world size, so
    the ranks' batches cost about the same and a rank's work does not depend on how many ranks there are."""
    from ds_splat_b200.dp import shard_views
    batch = world * vpr
    picked = [(g * num_views) // batch % num_views for g in range(batch)] if num_views >= batch else [g % num_views for g in range(batch)]
    return [picked[i] for i in shard_views(batch, rank, world)]


_AFFINITY_AT_START = None
GATHER_GROUP = [None]   # second communicator over all ranks, made once in main() when the optimizer step is pipelined


def bind_to_gpu_numa_node(dev_index: int):
    """Best effort: keeps this process (and so the pinned host buffers it allocates afterwards, which are placed on
    the allocating thread's node) on the host cores of the NUMA node the GPU hangs off.  Reads sysfs only; returns
    what it did for the bench line."""
    try:
        import torch
        props = torch.cuda.get_device_properties(dev_index)
        bus = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return {"node": None, "bound": False, "why": "the GPU reports no NUMA node"}
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        global _AFFINITY_AT_START
        allowed = os.sched_getaffinity(0)
        _AFFINITY_AT_START = set(allowed)
        local = sorted(cpus & allowed)
        if not local:
            return {"node": node, "bound": False, "why": "none of the node's cores is in this process's affinity set"}
        if len(local) < len(allowed):
            os.sched_setaffinity(0, local)
        return {"node": node, "bound": True, "cores": len(local)}
    except Exception as e:   # no sysfs entry, no permission: run unbound
        return {"node": None, "bound": False, "why": type(e).__name__}


def check_sharded_optimizer(dev, world, rank, chunks, gather_group):
    """N > 1, a few milliseconds: the forms of the optimizer step must agree on the device they will be timed on.  A small
    cloud, learning rates that move every parameter, three steps with gradients that differ per rank and step; compared
    are (a) all-reduce + Adam over everything, (b) ShardedAdam in one piece, (c) ShardedAdam in `chunks` pipelined chunks
    over the second communicator.  Returns the largest absolute parameter difference of (b) and of (c) against (a)."""
    import torch
    from ds_splat_b200.dp import FlatAdam, GradientBuffer, ParameterBuffer, ShardedAdam, allreduce_gradients
    n = 4099
    lrs = {"means3d": 1e-3, "shs": 2e-3, "opacities": 5e-2, "scales": 5e-3, "rotations": 1e-3}
    gen = torch.Generator(device="cpu").manual_seed(5)
    init = torch.randn(n * 59, generator=gen)

    def fresh(shards):
        p, g = ParameterBuffer(n, dev, shards=shards), GradientBuffer(n, dev, shards=shards)
        p.flat.copy_(init.to(dev)[:p.flat.numel()])
        return p, g

    def gradients(step):
        gg = torch.Generator(device="cpu").manual_seed(1000 * step + rank)
        return torch.randn(n * 59, generator=gg).to(dev)

    forms = {}
    pa, ga = fresh(1)
    oa = FlatAdam(pa.views, lrs, eps=1e-8)
    pb, gb = fresh(world)
    ob = ShardedAdam(pb, lrs, eps=1e-8)
    pc, gc = fresh(world * chunks)
    oc = ShardedAdam(pc, lrs, eps=1e-8, chunks=chunks, gather_group=gather_group)
    for step in range(1, 4):
        g = gradients(step)
        ga.flat.copy_(g[:ga.flat.numel()]); gb.flat.copy_(g[:gb.flat.numel()]); gc.flat.copy_(g[:gc.flat.numel()])
        allreduce_gradients(ga)
        oa.step(ga, grad_scale=1.0 / world)
        ob.step(gb, grad_scale=1.0 / world)
        oc.step(gc, grad_scale=1.0 / world)
    torch.cuda.synchronize()
    forms["sharded"] = float((pb.flat - pa.flat).abs().max())
    forms["sharded_pipelined" if oc.pipelined() else "sharded_chunked"] = float((pc.flat - pa.flat).abs().max())
    return forms


class Timed:
    """CUDA-event timing of a callable on the current stream: barrier + synchronize on both sides, max over ranks."""

    def __init__(self, world, dev):
        self.world, self.dev = world, dev

    def barrier(self):
        import torch
        import torch.distributed as dist
        if self.world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, ms: float) -> float:
        import torch
        import torch.distributed as dist
        if self.world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=self.dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def run(self, fn, steps, warmup):
        import torch
        from ds_splat_b200 import _capi
        for _ in range(warmup):
            fn()
        self.barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = _capi.launch_count()
        ev0.record()
        for _ in range(steps):
            fn()
        ev1.record()
        self.launches = _capi.launch_count() - launches0   # kernels of this library launched inside the timed region
        self.barrier()
        return self.max_over_ranks(ev0.elapsed_time(ev1))


def build_training(scene, cams, v_images, dev, args, world, tight_tiles=True):
    """Parameter block, renderer on its views, gradient block and optimizer of one training configuration."""
    import numpy as np
    import torch
    from ds_splat_b200.dp import GradientBuffer, ParameterBuffer, ShardedAdam, ViewRenderer, register_with_nccl
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    host = dict(means3d=scene.means, shs=scene.shs, opacities=scene.opacities, scales=scene.scales, rotations=scene.rotations)

    chunks = max(1, args.optimizer_chunks) if world > 1 else 1
    gather_group = GATHER_GROUP[0] if (world > 1 and chunks > 1) else None

    def make():
        return (ParameterBuffer(scene.n, dev, shards=world * chunks), GradientBuffer(scene.n, dev, shards=world * chunks))

    if world > 1 and not args.no_nccl_registration:
        (params, grads), pool = register_with_nccl(make, more_groups=[gather_group] if gather_group is not None else ())
    else:
        (params, grads), pool = make(), None
    for name, arr in host.items():
        params.views[name].copy_(t(arr).reshape(params.views[name].shape))
    renderer = ViewRenderer(**params.views, sh_degree=scene.sh_degree, view_streams=args.view_streams, tight_tiles=tight_tiles,
                            row_binning=args.row_binning)
    # Learning rate zero: the kernel reads and writes exactly what it does in training (parameters, gradients, both
    # moments), but the cloud stays the configuration's cloud over hundreds of timed steps.  (Adam's normalised
    # update would otherwise move every scale by lr per step whatever the gradient, and 300 steps destroy the scene.)
    opt = ShardedAdam(params, {k: 0.0 for k in LRS}, chunks=chunks, gather_group=gather_group)
    return params, grads, renderer, opt, pool


def timed_training(timer, renderer, cams, v_images, grads, opt, args, world, steps, warmup):
    """Times `steps` training steps; returns (ms per step, per-phase ms)."""
    import torch
    import torch.distributed as dist
    vpr = len(cams)
    marks = []

    pipelined = opt.pipelined()

    def step(record=False):
        # the library's own training step: render the rank's cameras, then ShardedAdam.step
        ev = []
        mark = None
        if record:
            def mark():
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                ev.append(e)
            mark()
        renderer.render_views(cams, v_images, grads, accumulate=False)
        if record:
            mark()
        opt.step(grads, grad_scale=1.0 / (vpr * world), marks=None if pipelined else mark)
        if record:
            if pipelined:
                mark()
            marks.append(ev)

    ms = timer.run(step, steps, warmup) / steps
    launches = timer.launches
    # the phases of a step, from a few extra steps with events between them (not part of the timed region above)
    for _ in range(min(steps, 10)):
        step(record=True)
    torch.cuda.synchronize()

    def mean_ms(pairs):   # pairs of event indices whose intervals are added up
        return round(timer.max_over_ranks(sum(sum(e[i].elapsed_time(e[j]) for i, j in pairs) for e in marks) / len(marks)), 4)
    if pipelined:   # reduce-scatter, update and all-gather of the chunks overlap: one figure
        phases = {"render": mean_ms([(0, 1)]), "sharded_step_pipelined": mean_ms([(1, 2)])}
    else:           # per chunk: reduce-scatter, update, all-gather
        c = opt.chunks
        phases = {"render": mean_ms([(0, 1)]),
                  "reduce_scatter": mean_ms([(1 + 3 * k, 2 + 3 * k) for k in range(c)]),
                  "adam": mean_ms([(2 + 3 * k, 3 + 3 * k) for k in range(c)]),
                  "all_gather": mean_ms([(3 + 3 * k, 4 + 3 * k) for k in range(c)])}
    timer.launches = launches
    return ms, phases


def timed_allreduce_form(timer, renderer, cams, v_images, grads, params, args, world, steps, warmup):
    """The replicated form for comparison: all-reduce of the gradient block, Adam over everything on every rank."""
    import torch
    from ds_splat_b200.dp import FlatAdam, allreduce_gradients
    opt = FlatAdam(params.views, {k: 0.0 for k in LRS})
    vpr = len(cams)

    def step():
        renderer.render_views(cams, v_images, grads, accumulate=False)
        allreduce_gradients(grads)
        opt.step(grads, grad_scale=1.0 / (vpr * world))

    ms = timer.run(step, steps, warmup) / steps
    del opt
    torch.cuda.empty_cache()
    return ms


def single_view_timing(renderer_cls, params_views, scene, cam, v_image, grads, tight_tiles, iters, warmup, capi, row_binning=False):
    """Median device time of ONE forward+backward through the fused single-view calls, and the stage times of it."""
    import torch
    r = renderer_cls(**params_views, sh_degree=scene.sh_degree, batch_views=1, tight_tiles=tight_tiles, view_streams=1,
                     row_binning=row_binning)
    for _ in range(warmup):
        r.forward(cam)
        r.backward(v_image, grads, accumulate=False)
    torch.cuda.synchronize()
    evs = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        r.forward(cam)
        r.backward(v_image, grads, accumulate=False)
        b.record()
        evs.append((a, b))
    torch.cuda.synchronize()
    times = sorted(a.elapsed_time(b) for a, b in evs)
    k, r_rows = r.last_k, r.last_k_rows
    capi.stage_timing(True)
    for _ in range(min(iters, 20)):
        r.forward(cam)
        r.backward(v_image, grads, accumulate=False)
    torch.cuda.synchronize()
    raw = capi.read_stage_timings()
    capi.stage_timing(False)
    stages = {name: round(ms / calls, 5) for name, (ms, calls) in raw.items() if calls}
    del r
    return {"median_ms": round(statistics.median(times), 4), "min_ms": round(times[0], 4), "iters": iters,
            "pairs": int(k), "row_items": int(r_rows), "stages_ms": stages}


def run_flythrough(args):
    """The reference README's protocol on a synthetic cloud: 120 frames of a camera that backs away from the scene,
    forward only, milliseconds per frame (README.md:199-204 of the reference plots such series for trained scenes)."""
    import numpy as np
    import torch
    from ds_splat_b200 import _capi, scene_io
    from ds_splat_b200.dp import CameraTensors, ViewRenderer
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    _capi.lib()
    scene = load_scene(args)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    r = ViewRenderer(t(scene.means), t(scene.shs), t(scene.opacities), t(scene.scales), t(scene.rotations),
                     sh_degree=scene.sh_degree, batch_views=1, view_streams=1)
    v0 = scene.views[0]
    views = scene_io.zoom_out_path(args.frames, start_distance=3.0, end_distance=12.0, W=v0.W, H=v0.H,
                                   focal=v0.W / (2.0 * v0.tanfovx))
    cams = [CameraTensors.from_view(v, dev) for v in views]
    for c in cams[:3]:
        r.forward(c)
    torch.cuda.synchronize()
    ms, pairs = [], []
    for c in cams:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        r.forward(c)
        b.record()
        b.synchronize()
        ms.append(round(a.elapsed_time(b), 4))
        pairs.append(int(r.last_k))
    line = {"metric": "forward ms per frame, 120-frame zoom-out fly-through", "value": round(statistics.mean(ms), 4), "unit": "ms",
            "n_gpus": 1, "steps": len(ms), "warmup": 3, "higher_is_better": False, "data": "synthetic", "dtype": "f32",
            "config": {"workload": f"flythrough over {scene.name}: {scene.n} splats, {v0.W}x{v0.H}, camera distance 3 -> 12"},
            "frame_ms": ms, "frame_pairs": pairs, "median_ms": round(statistics.median(ms), 4), "max_ms": max(ms)}
    print(json.dumps(line), flush=True)


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return
    if args.workload == "flythrough":
        run_flythrough(args)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    from ds_splat_b200 import GaussianRasterizationSettings, GaussianRasterizer, _capi
    from ds_splat_b200.dp import CameraTensors, ViewRenderer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the rasterizer has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    numa = bind_to_gpu_numa_node(local_rank)   # before the first pinned allocation
    json_out = sys.stdout
    if world > 1:
        # Libraries below write to file descriptor 1 (NCCL prints its version there): keep a private copy of it
        # for the one JSON line and point descriptor 1 at stderr for everything else.
        sys.stdout.flush()
        json_out = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)
        dist.init_process_group("nccl", device_id=dev)
        if args.optimizer_chunks > 1:
            try:
                GATHER_GROUP[0] = dist.new_group(backend="nccl", device_id=dev)
            except TypeError:   # a torch whose new_group takes no device
                GATHER_GROUP[0] = dist.new_group(backend="nccl")
    _capi.lib()  # fail loudly if the library is missing
    timer = Timed(world, dev)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    optimizer_check = None
    if world > 1:
        optimizer_check = check_sharded_optimizer(dev, world, rank, max(2, args.optimizer_chunks), GATHER_GROUP[0])
        optimizer_check = {k: timer.max_over_ranks(v) for k, v in optimizer_check.items()}
        optimizer_check["agree"] = all(v < 1e-5 for v in optimizer_check.values())   # reported, not fatal: the timings stand

    vpr = max(1, args.views_per_rank)
    scene = load_scene(args, views=world * vpr)
    H, W = scene.views[0].H, scene.views[0].W
    # Every view of a step, on every rank, is a different camera (views_of_rank).
    view_ids = views_of_rank(len(scene.views), rank, world, vpr)
    cams = [CameraTensors.from_view(scene.views[v], dev) for v in view_ids]
    v_images_host = [scene.image_grad(v, seed=7 + v) for v in view_ids]
    v_images = [t(v) for v in v_images_host]
    params, grads, renderer, opt, pool = build_training(scene, cams, v_images, dev, args, world)
    opt_chunks, opt_pipelined = int(opt.chunks), bool(opt.pipelined())
    warmup = max(args.warmup, 3)

    # ---- device-timed training steps ------------------------------------------------------------------
    for _ in range(warmup):   # allocator and pair buffers reach their steady state before the clocks are sampled
        renderer.render_views(cams, v_images, grads, accumulate=False)
    timer.barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms_per_step, phases = timed_training(timer, renderer, cams, v_images, grads, opt, args, world, args.steps, warmup)
    launches = timer.launches
    clocks = sampler.stop()
    if world > 1 and args.reduce == "allreduce":
        ms_per_step = timed_allreduce_form(timer, renderer, cams, v_images, grads, params, args, world, args.steps, 3)
        launches = timer.launches
    views_per_s = world * vpr / (ms_per_step * 1e-3)
    ks = [int(k) for k in renderer.last_ks]
    kt = torch.tensor([min(ks), max(ks), sum(ks)], dtype=torch.float64, device=dev)
    if world > 1:
        kmin, kmax, ksum = kt[0:1].clone(), kt[1:2].clone(), kt[2:3].clone()
        dist.all_reduce(kmin, op=dist.ReduceOp.MIN); dist.all_reduce(kmax, op=dist.ReduceOp.MAX); dist.all_reduce(ksum)
        kt = torch.cat([kmin, kmax, ksum])
    pairs_emitted = {"min": int(kt[0].item()), "max": int(kt[1].item()), "mean": int(kt[2].item() / (world * vpr))}
    allreduce_form_ms = None
    if world > 1 and args.reduce == "sharded":
        allreduce_form_ms = timed_allreduce_form(timer, renderer, cams, v_images, grads, params, args, world,
                                                 min(args.steps, 40), 3)

    # ---- the same step with the reference-identical pair lists ------------------------------------------
    strict = None
    if not args.skip_strict:
        renderer.tight_tiles = False
        s_steps = min(args.steps, 60)
        s_ms, _ = timed_training(timer, renderer, cams, v_images, grads, opt, args, world, s_steps, 3)
        strict = {"ms_per_view": round(s_ms / vpr, 4), "views_per_s": round(world * vpr / (s_ms * 1e-3), 3), "steps": s_steps,
                  "pairs_mean": int(sum(renderer.last_ks) / vpr),
                  "note": "tight_tiles off: tiles-touched counts, pair list and tile ranges are bit-identical to the reference's"}
        renderer.tight_tiles = True

    # ---- per-stage timing of the same steps (events recorded by the library around each stage) ---------
    # The stages are timed with the views one after the other on one stream: with two views in flight the events
    # around one view's stage also cover the other view's kernels.
    lanes_used = renderer.view_streams
    renderer.view_streams = 1
    _capi.stage_timing(True)
    stage_steps = min(args.steps, 40)
    for _ in range(stage_steps):
        renderer.render_views(cams, v_images, grads, accumulate=False)
    torch.cuda.synchronize()
    stage_raw = _capi.read_stage_timings()
    _capi.stage_timing(False)
    renderer.view_streams = lanes_used
    # per view: the per-splat backward runs once for all views of a step, every other stage once per view
    stages_ms = {name: round(ms / (stage_steps * vpr), 5) for name, (ms, calls) in stage_raw.items() if calls}

    # ---- the literal metric: one view per iteration through the fused single-view calls, configuration's camera ----
    single = None
    if world == 1 or rank == 0:
        cam0 = CameraTensors.from_view(scene.views[0], dev)
        v0 = t(scene.image_grad(0, seed=7))
        iters = max(20, min(args.steps, 100))
        single = {"tight_tiles": single_view_timing(ViewRenderer, params.views, scene, cam0, v0, grads, True, iters, 5, _capi),
                  "strict_lists": single_view_timing(ViewRenderer, params.views, scene, cam0, v0, grads, False, iters, 5, _capi),
                  # the other way to the same list (DSB_FLAG_ROW_BINNING), for the record: emit_pairs = row items,
                  # tile_sort = their sort, the width scan and the one pass over the pairs
                  "strict_lists_row_binning": single_view_timing(ViewRenderer, params.views, scene, cam0, v0, grads, False,
                                                                 iters, 5, _capi, row_binning=True)}
        del cam0, v0
    timer.barrier()

    # ---- the kernels either side of the operator in a training loop (reported beside the metric) ---------
    optimizer = None
    if world == 1 and not args.skip_optimizer:
        adam_ms = phases["adam"]
        adam_bytes = 28 * grads.flat.numel()   # read p, g, m, v; write p, m, v
        optimizer = {"kernel": "adam_kernel (one launch per parameter tensor)", "ms_per_step": round(adam_ms, 4),
                     "achieved_GBps": round(adam_bytes / (adam_ms * 1e-3) / 1e9, 1), "algorithmic_bytes": int(adam_bytes)}
        from ds_splat_b200.dp import ImageLoss
        loss_fn = ImageLoss(lambda_dssim=0.2)
        img = renderer.forward(cams[-1]).clone()
        tgt = torch.rand_like(img)
        loss_ms = timer.run(lambda: loss_fn.gradient(img, tgt), 20, 3) / 20
        loss_bytes = 4 * 3 * H * W * (2 + 3 + 3 + 2 + 1)   # read x, y; write 3 maps; read 3 maps, x, y; write dL/dx
        optimizer["image_loss"] = {"kernels": "ssim_moments_kernel + ssim_gradient_kernel", "ms_per_view": round(loss_ms, 4),
                                   "achieved_GBps": round(loss_bytes / (loss_ms * 1e-3) / 1e9, 1),
                                   "algorithmic_bytes": int(loss_bytes)}
        del loss_fn, img, tgt

    # ---- end to end through the public operator, host buffers -----------------------------------------
    e2e = None
    if not args.skip_e2e:
        # One training iteration the way a user of the operator writes it: the camera and the step's target image (8-bit
        # RGB, the form datasets hold) come from pinned host memory, the loss is L1 on the rendered image (dp.ImageLoss
        # with lambda_dssim = 0: one kernel for the loss value and dL/dimage), autograd drives the operator's backward, and
        # the loss value is read on the host.
        view = scene.views[view_ids[0]]
        rng = np.random.default_rng(11)
        pinned_target = torch.from_numpy(rng.integers(0, 256, size=(H, W, 3), dtype=np.uint8)).pin_memory()
        pinned_view = torch.from_numpy(view.viewmatrix_t).pin_memory()
        pinned_proj = torch.from_numpy(view.projmatrix_t).pin_memory()
        pinned_pos = torch.from_numpy(np.ascontiguousarray(view.campos)).pin_memory()
        # two sets of buffers: step i's loss is read on the host while step i + 1 is already enqueued (a training loop
        # logs the loss of the step before the one in flight)
        loss_host = [torch.empty((), dtype=torch.float32).pin_memory() for _ in range(2)]
        target_dev = [torch.empty((H, W, 3), dtype=torch.uint8, device=dev) for _ in range(2)]
        leaves = {k: v.detach().clone().requires_grad_(True) for k, v in params.views.items()}
        means2d = torch.zeros_like(leaves["means3d"], requires_grad=True)
        bg = torch.zeros(3, device=dev)
        vm, pm, cp = (torch.empty_like(x, device=dev) for x in (pinned_view, pinned_proj, pinned_pos))
        settings = GaussianRasterizationSettings(H, W, view.tanfovx, view.tanfovy, bg, 1.0, vm, pm, scene.sh_degree, 3, cp,
                                                 False, False)
        rasterizer = GaussianRasterizer(settings)
        from ds_splat_b200.dp import ImageLoss
        loss_fn = ImageLoss(lambda_dssim=0.0)
        h2d = pinned_target.numel() + (16 + 16 + 3) * 4
        d2h = 4
        upload_stream = torch.cuda.Stream(device=dev)    # the target image travels while the forward runs
        main_stream = torch.cuda.current_stream()
        target_ready = torch.cuda.Event()
        backward_done = [torch.cuda.Event(), torch.cuda.Event()]
        result_on_host = [torch.cuda.Event(), torch.cuda.Event()]
        checksum = [0.0]

        def e2e_step(i):
            s = i & 1
            vm.copy_(pinned_view, non_blocking=True)
            pm.copy_(pinned_proj, non_blocking=True)
            cp.copy_(pinned_pos, non_blocking=True)
            with torch.cuda.stream(upload_stream):
                upload_stream.wait_event(backward_done[s])   # the loss that last read target_dev[s] (two steps ago)
                target_dev[s].copy_(pinned_target, non_blocking=True)
                target_ready.record(upload_stream)
            for leaf in leaves.values():
                leaf.grad = None
            means2d.grad = None
            image, radii = rasterizer(leaves["means3d"], means2d, leaves["shs"], None, leaves["opacities"],
                                      leaves["scales"], leaves["rotations"], None)
            main_stream.wait_event(target_ready)
            v_image, loss = loss_fn.gradient(image.detach(), target_dev[s])   # the library's one-pass L1 loss, 8-bit target
            image.backward(v_image)
            backward_done[s].record(main_stream)
            loss_host[s].copy_(loss[0], non_blocking=True)
            result_on_host[s].record(main_stream)
            if i > 0:   # the previous step's loss, on the host
                result_on_host[s ^ 1].synchronize()
                checksum[0] += float(loss_host[s ^ 1])

        def e2e_drain(i):   # the last step's loss
            result_on_host[(i - 1) & 1].synchronize()
            checksum[0] += float(loss_host[(i - 1) & 1])
            torch.cuda.synchronize()

        for ev in backward_done:
            ev.record(main_stream)
        for i in range(warmup):
            e2e_step(i)
        e2e_drain(warmup)
        timer.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        wall0 = time.perf_counter()
        a.record()
        for i in range(args.steps):
            e2e_step(i)
        e2e_drain(args.steps)
        b.record()
        timer.barrier()
        wall = time.perf_counter() - wall0
        e_ms = timer.max_over_ranks(max(a.elapsed_time(b), wall * 1e3))  # host work between kernels counts: the slower clock
        e2e = {"value": round(world * args.steps / (e_ms * 1e-3), 3), "unit": UNIT,
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
               "ms_per_step": round(e_ms / args.steps, 4),
               "note": "one training iteration per step through GaussianRasterizer + autograd: camera and the 8-bit target "
                       "image from pinned host memory (second stream), L1 loss on the rendered image (dp.ImageLoss), backward, the loss "
                       "value read on the host one step behind the step being enqueued; splat parameters are model state "
                       "resident on the device"
                       + ("; per-rank iterations with no collective in them (N independent loops)" if world > 1 else "")}
        del leaves, means2d, rasterizer, loss_fn

    nccl_registered = pool is not None
    # ---- config 3 beside it: 6M splats, 8 of the 64 ring cameras per rank and step, 1.416 GB of gradients ----------
    c3 = None
    if not args.skip_c3 and args.workload == "c1" and not args.splats:
        del renderer, opt, params, grads, cams, v_images, pool
        torch.cuda.empty_cache()
        from ds_splat_b200 import scenes
        sc3 = scenes.multiview()
        ids3 = views_of_rank(len(sc3.views), rank, world, vpr)
        cams3 = [CameraTensors.from_view(sc3.views[v], dev) for v in ids3]
        vim3 = [t(sc3.image_grad(v, seed=7 + v)) for v in ids3]
        params3, grads3, renderer3, opt3, pool3 = build_training(sc3, cams3, vim3, dev, args, world)
        ms3, phases3 = timed_training(timer, renderer3, cams3, vim3, grads3, opt3, args, world, 8, 3)
        c3 = {"workload": f"{sc3.name}: {sc3.n} splats SH-3, {W}x{H}, {vpr} of {len(sc3.views)} ring cameras per rank per step, spaced evenly around the ring",
              "views_per_s": round(world * vpr / (ms3 * 1e-3), 3), "ms_per_step": round(ms3, 4), "steps": 8, "warmup": 3,
              "step_breakdown_ms": phases3, "gradient_bytes": int(grads3.nbytes()),
              "pairs_emitted_mean": int(sum(renderer3.last_ks) / vpr), "nccl_registered_buffers": pool3 is not None}
        del renderer3, opt3, params3, grads3, cams3, vim3, sc3, pool3
        torch.cuda.empty_cache()

    # ---- CPU baseline (rank 0; the other ranks wait at the barrier below) -------------------------------
    view0 = scene.views[0]
    v_image0 = scene.image_grad(0, seed=7)
    cpu_baseline, pairs_bwd, pairs_fwd, K_ref = None, None, None, None
    if rank == 0 and not args.skip_cpu_baseline:
        from oracle import oracle as O
        if _AFFINITY_AT_START:   # the CPU baseline gets every core the process started with, not only the GPU's node
            os.sched_setaffinity(0, _AFFINITY_AT_START)
        cores = O.use_all_host_threads()   # torchrun exports OMP_NUM_THREADS=1 to its workers
        sec, fwd_o, bwd_o = oracle_one_view(scene, view0, v_image0)
        pairs_fwd, pairs_bwd, K_ref = fwd_o["pairs_fwd"], bwd_o["pairs_bwd"], fwd_o["K"]
        # timed at every N (it also counts the pairs the roofline needs), reported as the baseline at N = 1 only
        if world == 1:
            cpu_baseline = {"value": round(1.0 / sec, 5), "unit": UNIT, "cores": cores, "kind": "port",
                            "sample": "one full view of the workload (forward + backward, no optimizer step), C++/OpenMP "
                                      "restatement in oracle/", "ms_per_view": round(sec * 1e3, 1)}
    timer.barrier()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    reference_cuda = reference_cuda_numbers(scene, view0, v_image0) if world == 1 and not args.skip_reference_cuda else None

    peak, peak_src = measured_peaks()
    if optimizer:
        optimizer["frac_of_hbm_peak"] = round(optimizer["achieved_GBps"] / peak, 4)
    roofline, roofline_hbm, stage_achieved = None, None, None
    if single:
        # The dominant kernel, on the configuration's own camera, strict lists (the pairs it walks are the reference's).
        sv = single["strict_lists"]
        dom_ms, K = sv["stages_ms"].get("blend_backward"), sv["pairs"]
        if dom_ms and pairs_bwd and clocks.get("sm_mhz"):
            flops = 74.0 * pairs_bwd
            fp32_peak = 148 * 128 * 2 * clocks["sm_mhz"] * 1e6 / 1e12
            # DRAM bytes of one blend_backward_kernel launch from the ncu capture summarised in
            # profiles/blend_backward_c1.md (83,856,640 read + 3,512,064 written for 7,710,065 pairs); it is dominated by
            # the first touch of the pair list and the gathered records, so it is scaled by the pairs of this launch.
            traffic = int(87_368_704 * (K / 7_710_065))
            roofline = {"kernel": "blend_backward_kernel", "bound": "fp32", "achieved": round(flops / (dom_ms * 1e-3) / 1e12, 3),
                        "peak": round(fp32_peak, 2), "unit": "TFLOP/s", "frac": round(flops / (dom_ms * 1e-3) / 1e12 / fp32_peak, 4),
                        "traffic": traffic, "ms": dom_ms, "pairs_visited": int(pairs_bwd), "flop_per_pair": 74,
                        # what the kernel itself executes per visited pair after its regrouping (one running dot product
                        # per pixel instead of three colour buffers, moments instead of per-pixel gradients): 37 flop of
                        # blending arithmetic + 14 adds of the warp reduction shared by a lane's four pixels
                        "executed": {"flop_per_pair": 40.5, "achieved": round(40.5 * pairs_bwd / (dom_ms * 1e-3) / 1e12, 3),
                                     "frac": round(40.5 * pairs_bwd / (dom_ms * 1e-3) / 1e12 / fp32_peak, 4)},
                        "peak_source": "148 SMs x 128 FP32 lanes x 2 flop x median SM clock sampled during the run (not in "
                                       "MEASURED_PEAKS.json, which holds HBM and bf16 tensor peaks only)",
                        "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch on config 1, scaled by pairs",
                        "note": "single-view call on the configuration's camera with the reference-identical pair list; 'achieved' "
                                "counts the reference algorithm's 74 flop per visited (pixel, splat) pair as written in its "
                                "kernel; this kernel reaches the same sums with fewer operations, so 'executed' is the figure "
                                "that describes the FP32 pipes (issue-slot and pipe counters in profiles/)"}
            # 8 B pair + 48 B record gathered per list entry, 36 B of per-splat sums added per list entry, 20 B per pixel
            # read (dL/dimage 12, final_T 4, final_idx 4), plus the 48 B/splat zero fill of the accumulator in the stage.
            alg_bytes = K * (8 + 48 + 36) + 20 * H * W + 48 * scene.n
            roofline_hbm = {"kernel": "blend_backward_kernel", "bound": "hbm", "achieved": round(alg_bytes / (dom_ms * 1e-3) / 1e9, 2),
                            "peak": peak, "unit": "GB/s", "frac": round(alg_bytes / (dom_ms * 1e-3) / 1e9 / peak, 4),
                            "algorithmic_bytes": int(alg_bytes), "peak_source": peak_src,
                            "note": "secondary: the kernel is bound by FP32/SHFL issue, its working set is L2-resident"}
        # K-sized stages on the pairs they actually move (strict: the reference's count; tight: the emitted subset)
        stage_achieved = {}
        for mode, sv_ in single.items():
            if sv_["row_items"]:
                continue   # row-binned: its stages move row items, not pairs
            k_, st = sv_["pairs"], sv_["stages_ms"]
            rec = {}
            if st.get("emit_pairs"):
                rec["emit_pairs_GBps"] = round((8 * k_ + 36 * scene.n) / (st["emit_pairs"] * 1e-3) / 1e9, 1)
            if st.get("tile_sort"):
                rec["tile_sort_GBps"] = round(2 * 16 * k_ / (st["tile_sort"] * 1e-3) / 1e9, 1)
            rec["frac_of_hbm_peak"] = {k2[:-5]: round(v / peak, 3) for k2, v in rec.items()}
            stage_achieved[mode] = rec

    line = {"metric": METRIC, "value": round(views_per_s, 3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": round(ms_per_step, 4),
            "fwd_bwd_ms_per_view": round(phases["render"] / vpr, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{scene.name}: {scene.n} splats SH-3, {W}x{H}, {vpr} distinct cameras per rank per step "
                                   f"(camera 0 is the configuration's, the others turned +-5 degrees from it), fwd+bwd of each, "
                                   + ("gradient reduce-scatter, Adam on 1/N of the parameters, parameter all-gather"
                                      if world > 1 else "Adam step"),
                       "pairs_reference_list_view0": K_ref, "pairs_emitted": pairs_emitted, "tiles": scene.views[0].num_tiles,
                       "view_streams": int(min(args.view_streams, vpr)), "row_binning": bool(args.row_binning), "optimizer": "Adam, learning rate 0 (same reads and "
                       "writes; the cloud stays the configuration's)", "reduce": args.reduce if world > 1 else "none",
                       "nccl_registered_buffers": bool(nccl_registered), "host_numa": numa,
                       "optimizer_chunks": opt_chunks, "optimizer_pipelined": opt_pipelined,
                       "optimizer_forms_max_abs_difference": optimizer_check,
                       "l2": "inputs larger than L2 (236 MB of parameters + 62-88 MB pair list per view; no explicit flush)",
                       "parallelism": f"dp{world} (cameras sharded, splats replicated)"},
            "clocks": clocks, "gpu_launches": int(launches), "step_breakdown_ms": phases,
            "single_view_ms": single["tight_tiles"]["median_ms"] if single else None, "single_view": single,
            "strict_lists": strict, "allreduce_form_ms_per_step": round(allreduce_form_ms, 4) if allreduce_form_ms else None,
            "stages_ms": stages_ms, "stages_note": "per view, from a rerun of the same steps with the views on ONE stream",
            "stage_achieved": stage_achieved, "roofline": roofline, "roofline_hbm": roofline_hbm,
            "cpu_baseline": cpu_baseline, "e2e": e2e, "reference_cuda": reference_cuda, "optimizer": optimizer, "c3": c3,
            "pairs_evaluated": {"forward_per_pixel": pairs_fwd, "backward_per_pixel": pairs_bwd}}
    print(json.dumps(line), file=json_out, flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
