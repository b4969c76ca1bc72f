"""Multi-view data-parallel rendering step: cameras sharded over ranks, splats replicated, one
gradient all-reduce per step.

The reference has no multi-GPU code; this module is the camera-sharded training step the benchmark's
multi-GPU configuration describes: every rank (one process per GPU) renders its share of the batch's
cameras against the full replicated splat cloud, accumulates the parameter gradients of its views, and
the ranks sum them with one NCCL all-reduce over NVLink.

Layout choices:
  * ``GradientBuffer`` is ONE flat fp32 allocation holding the five gradient tensors back to back
    (means 3 | sh 48 | opacity 1 | scale 3 | rotation 4 = 59 floats per splat).  The fused backward
    kernel adds each view's gradients straight into these views (``accumulate`` flag of
    ``dsb_backward``), so the buffer that is all-reduced is the buffer the kernels write -- no copy,
    no per-tensor collectives.
  * ``ViewRenderer`` bypasses autograd and calls the fused C-ABI entry points with buffers that are
    allocated once and reused across views and steps (only the pair list grows with the largest K seen).
  * A step deals its views over two streams (forward, then the backward blend, per view; one view's pair sort,
    which waits on memory, runs beside another view's blend, which waits on instruction issue) but runs the
    per-splat part of the backward ONCE for up to eight views (``dsb_geometry_backward_views``): the splat
    parameters are read once and the 236 bytes of gradients per splat are written once per step instead of
    being read and rewritten for every view.  Each view of a batch keeps its own records, radii and
    accumulator rows (100 bytes per splat and view) until that call.

Everything that is not a kernel launch (sharding, buffer layout, the collective) works on CPU tensors
too, which is how the world_size-2 gloo tests exercise it.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

def _on_own_device(method):
    """Runs a method with the object's device (``self.dev``) current: the library launches on the current device and
    stream, so a renderer whose tensors live on another GPU than the current one must switch first."""
    import functools

    @functools.wraps(method)
    def wrapped(self, *args, **kwargs):
        dev = torch.device(self.dev)
        if dev.type != "cuda":
            raise RuntimeError(f"{type(self).__name__} launches CUDA kernels; its tensors are on {dev}")
        with torch.cuda.device(dev):
            return method(self, *args, **kwargs)
    return wrapped


SEGMENTS = (("means3d", 3), ("shs", 48), ("opacities", 1), ("scales", 3), ("rotations", 4))
FLOATS_PER_SPLAT = sum(w for _, w in SEGMENTS)  # 59


def shard_views(num_views: int, rank: int, world_size: int) -> List[int]:
    """Round-robin assignment of view indices to ranks; every view lands on exactly one rank."""
    if not (0 <= rank < world_size):
        raise ValueError(f"rank {rank} outside world of {world_size}")
    return list(range(rank, num_views, world_size))


class GradientBuffer:
    """Flat fp32 gradient block with per-tensor views (see module docstring).  ``shards`` > 1 pads the allocation to
    ``shards`` equal slices of whole 16-byte lanes, the form reduce-scatter and all-gather take (``ShardedAdam``)."""

    def __init__(self, n: int, device, sh_coeffs: int = 16, shards: int = 1):
        self.n = n
        self.sh_coeffs = sh_coeffs
        widths = dict(SEGMENTS)
        widths["shs"] = 3 * sh_coeffs
        self.length = n * sum(widths.values())            # elements that carry gradients
        quantum = 4 * max(1, int(shards))
        padded = (self.length + quantum - 1) // quantum * quantum
        self.storage = torch.zeros(padded, dtype=torch.float32, device=device)   # the padded allocation
        self.flat = self.storage[:self.length]
        self.views: Dict[str, torch.Tensor] = {}
        self.segments: Dict[str, tuple] = {}              # name -> (first element, one past the last) in the flat block
        off = 0
        for name, _ in SEGMENTS:
            w = widths[name]
            v = self.flat[off:off + n * w]
            self.views[name] = v.view(n, sh_coeffs, 3) if name == "shs" else v.view(n, w)
            self.segments[name] = (off, off + n * w)
            off += n * w

    def zero_(self):
        self.flat.zero_()

    def nbytes(self) -> int:
        return self.flat.numel() * 4


class ParameterBuffer(GradientBuffer):
    """The five parameter tensors of a splat cloud in ONE allocation laid out like the gradient block, so that a
    rank's slice of the gradients lines up with the same slice of the parameters (``ShardedAdam``).  ``views`` are
    what ``ViewRenderer`` takes as its tensors."""

    @staticmethod
    def from_tensors(params: Dict[str, torch.Tensor], shards: int = 1) -> "ParameterBuffer":
        means = params["means3d"]
        buf = ParameterBuffer(means.shape[0], means.device, sh_coeffs=params["shs"].shape[1], shards=shards)
        for name, _ in SEGMENTS:
            buf.views[name].copy_(params[name].reshape(buf.views[name].shape))
        return buf


def allreduce_gradients(buf: GradientBuffer, group=None) -> None:
    """Sum the flat gradient block over all ranks (no-op in a single-process run)."""
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(buf.flat, op=dist.ReduceOp.SUM, group=group)


@dataclass
class CameraTensors:
    """Device-resident camera in the layout GaussianRasterizationSettings carries (transposed matrices)."""
    H: int
    W: int
    tanfovx: float
    tanfovy: float
    viewmatrix: torch.Tensor
    projmatrix: torch.Tensor
    campos: torch.Tensor
    bg: Optional[torch.Tensor] = None

    @staticmethod
    def from_view(view, device) -> "CameraTensors":
        t = lambda a: torch.from_numpy(a).to(device)
        import numpy as np
        return CameraTensors(view.H, view.W, view.tanfovx, view.tanfovy, t(view.viewmatrix_t), t(view.projmatrix_t),
                             t(np.ascontiguousarray(view.campos)), torch.zeros(3, device=device))


class _Slot:
    """Per-view buffers that must survive until the batch's per-splat backward: 128 bytes per splat.  tiles,
    depth_keys and offsets are rows of tensors shared by the slots, because the batch's plan takes them as rows."""

    def __init__(self, n, dev, capi, tiles, depth_keys, offsets):
        f32 = dict(dtype=torch.float32, device=dev)
        self.records = torch.empty((n, capi.RECORD_FLOATS), **f32)
        self.radii = torch.empty(n, dtype=torch.int32, device=dev)
        self.tiles, self.depth_keys, self.offsets = tiles, depth_keys, offsets
        self.grad_acc = torch.empty((n, capi.GRAD_FLOATS), **f32)
        self.marks = {}     # (H, W) -> tile-mark grid, later the tile order
        self.ranges = {}    # (H, W) -> tile ranges of the view
        self.layout = torch.empty(capi.LAYOUT_WORDS, dtype=torch.int32, device=dev)   # layout block of the fused render
        self.cam = None     # (DsbCamera, keep-alive) of the view the slot holds


class DensifyStats:
    """The per-splat statistics a 3-D Gaussian Splatting training loop consults when it densifies, kept by the
    per-splat backward itself (``dsb_geometry_backward_views_stats``): for every view in which a splat is visible
    (radius > 0) ``grad_norm_sum`` grows by the norm of that view's pixel-mean gradient, ``visible_count`` by one,
    and ``max_radius`` becomes the larger of itself and the view's radius.  ``ndc_units`` scales the gradient by
    (W/2, H/2) first, the units of loops written for the original 3DGS rasterizer; otherwise pixel units, as the
    reference's v_means2d.  The caller clears them with ``zero_()`` when it has densified."""

    def __init__(self, n: int, device, ndc_units: bool = False):
        self.flat = torch.zeros((3, n), dtype=torch.float32, device=device)
        self.grad_norm_sum, self.visible_count, self.max_radius = self.flat[0], self.flat[1], self.flat[2]
        self.ndc_units = ndc_units

    def zero_(self):
        self.flat.zero_()

    def add_view(self, v_means2d: torch.Tensor, radii: torch.Tensor, height: int, width: int) -> None:
        """The same update from one view's v_means2d and radii as tensors (what a loop around the single-view
        operator has in hand)."""
        sx, sy = (0.5 * width, 0.5 * height) if self.ndc_units else (1.0, 1.0)
        seen = radii > 0
        norm = torch.sqrt((sx * v_means2d[:, 0]) ** 2 + (sy * v_means2d[:, 1]) ** 2)
        self.grad_norm_sum += torch.where(seen, norm, torch.zeros_like(norm))
        self.visible_count += seen.to(torch.float32)
        torch.maximum(self.max_radius, torch.where(seen, radii.to(torch.float32), self.max_radius), out=self.max_radius)

    def allreduce(self, group=None) -> None:
        """Combines the ranks' statistics (sums of the first two, maximum of the third).  Called once, just before
        the ranks densify: each rank's arrays only cover the views it rendered itself."""
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(self.flat[:2], op=dist.ReduceOp.SUM, group=group)
            dist.all_reduce(self.flat[2], op=dist.ReduceOp.MAX, group=group)

    def mean_grad_norm(self) -> torch.Tensor:
        """grad_norm_sum / visible_count, zero where a splat was never visible."""
        return torch.where(self.visible_count > 0, self.grad_norm_sum / self.visible_count.clamp(min=1),
                           torch.zeros_like(self.grad_norm_sum))


class _Lane:
    """Buffers of the per-view stages (pair list and its sort, image, transmittance, last contributor) and the stream
    they run on.  Lane 0 runs on the caller's stream; ``render_views`` adds lanes with streams of their own so that
    one view's latency-bound pair sort runs beside another view's issue-bound blend."""

    def __init__(self, stream=None):
        self.stream = stream    # None: whatever stream is current
        self.pairs = None       # sorted (tile, splat) pairs of the lane's view
        self.cap = 0            # pairs the list holds
        self.render_ws = None   # row items, their sort and scan, the scatter's look-back words
        self.render_bytes = 0
        self.cap_rows = 0       # row items the workspace was sized for
        self.img = {}


class ViewRenderer:
    """Forward + backward of views of one splat cloud through the fused C-ABI calls, with reusable buffers.

    ``forward`` / ``backward`` handle one view at a time; ``render_views`` handles a whole step (see the module
    docstring) and is what ``data_parallel_step`` uses."""

    def __init__(self, means3d, shs, opacities, scales, rotations, sh_degree: int = 3, strict_reference: bool = True,
                 batch_views: int = 8, tight_tiles: bool = True, view_streams: int = 2, row_binning: bool = False):
        from . import _capi
        self._capi = _capi
        self.lib = _capi.lib()
        self.p = dict(means3d=means3d.contiguous(), shs=shs.contiguous(), opacities=opacities.contiguous(),
                      scales=scales.contiguous(), rotations=rotations.contiguous())
        self.n = means3d.shape[0]
        self.dev = means3d.device
        self.sh_degree = sh_degree
        self.coeffs = shs.shape[1]
        self.strict = strict_reference
        self.tight_tiles = tight_tiles   # pairs only for tiles a splat can contribute to: same results, shorter lists
        # row binning (DSB_FLAG_ROW_BINNING): one pass over the pairs instead of writing them and sorting them in two;
        # the same list, faster when splats are wide (many tiles per tile row), slower on the benchmark clouds
        self.row_binning = row_binning
        n, dev = self.n, self.dev
        self.batch_views = max(1, min(int(batch_views), _capi.MAX_BATCH_VIEWS))
        bv = self.batch_views
        self.tiles_rows = torch.empty((bv, n), dtype=torch.int32, device=dev)
        self.depth_rows = torch.empty((2, bv, n), dtype=torch.int64, device=dev)   # [1] is the sort's other buffer
        self.offset_rows = torch.empty((bv, n), dtype=torch.int32, device=dev)
        self.slots = []                      # the slots' large buffers are allocated when a step first needs them
        self.cur = self._slot(0)
        self.cov3d = torch.empty((n, 6), dtype=torch.float32, device=dev)
        self.plan_bytes = int(self.lib.dsb_plan_workspace_bytes_views(n, bv))
        self.plan_ws = torch.empty(self.plan_bytes, dtype=torch.uint8, device=dev)
        self.view_streams = max(1, int(view_streams))   # lanes render_views spreads a batch's views over
        self.lanes = [_Lane()]
        self.last_k = 0
        self.last_k_rows = 0
        self.last_ks = []

    # buffers of the view rendered last (kept as attributes for callers that inspect them)
    records = property(lambda self: self.cur.records)
    radii = property(lambda self: self.cur.radii)
    grad_acc = property(lambda self: self.cur.grad_acc)
    pairs = property(lambda self: self.lanes[0].pairs)

    def _image_buffers(self, h, w, lane: int = 0):
        img = self.lanes[lane].img
        key = (h, w)
        if key not in img:
            f32 = dict(dtype=torch.float32, device=self.dev)
            img[key] = (torch.empty((h, w, 3), **f32), torch.empty((h, w), **f32),
                        torch.empty((h, w), dtype=torch.int32, device=self.dev))
        return img[key]

    def _lane(self, i: int) -> _Lane:
        while len(self.lanes) <= i:
            self.lanes.append(_Lane(torch.cuda.Stream(device=self.dev)))
        return self.lanes[i]

    def _ranges(self, slot: _Slot, h, w):
        key = (h, w)
        if key not in slot.ranges:
            slot.ranges[key] = torch.empty(self._capi.num_tiles(h, w) + 1, dtype=torch.int32, device=self.dev)
        return slot.ranges[key]

    def _marks(self, slot: _Slot, h, w):
        key = (h, w)
        if key not in slot.marks:
            slot.marks[key] = torch.empty(int(self.lib.dsb_tile_marks_bytes(h, w)), dtype=torch.uint8, device=self.dev)
        return slot.marks[key]

    def _camera(self, cam: CameraTensors):
        max_deg = {1: 0, 4: 1, 9: 2, 16: 3}[self.coeffs]
        return self._capi.make_camera(cam.H, cam.W, cam.tanfovx, cam.tanfovy, cam.viewmatrix, cam.projmatrix, cam.campos,
                                      cam.bg, self.sh_degree, max_deg, 1.0, transposed=True, drop_last=self.strict,
                                      tight_tiles=self.tight_tiles, row_binning=self.row_binning)

    def _slot(self, j: int) -> _Slot:
        while len(self.slots) <= j:
            i = len(self.slots)
            self.slots.append(_Slot(self.n, self.dev, self._capi, self.tiles_rows[i], self.depth_rows[0, i],
                                    self.offset_rows[i]))
        return self.slots[j]

    def _pair_buffers(self, k: int, k_rows: int, h: int, w: int, lane: int = 0) -> _Lane:
        """Pair list and render workspace of a lane, grown (with 25% slack) when a view needs more than they hold."""
        ln = self.lanes[lane]
        need = int(self.lib.dsb_render_workspace_bytes(h, w, k, k_rows))
        if ln.pairs is None or ln.cap < k or ln.render_bytes < need:
            if ln.pairs is not None and ln.stream is not None:
                ln.stream.synchronize()   # the old buffers go back to the allocator of another stream
            ln.cap = max(int(k * 1.25), 1024, ln.cap)
            ln.cap_rows = max(int(k_rows * 1.25), ln.cap_rows) if k_rows else ln.cap_rows   # only row-binned views have any
            ln.pairs = torch.empty(ln.cap, dtype=torch.int64, device=self.dev)
            ln.render_bytes = int(self.lib.dsb_render_workspace_bytes(h, w, ln.cap, ln.cap_rows))
            ln.render_ws = torch.empty(ln.render_bytes, dtype=torch.uint8, device=self.dev)
        return ln

    def _render(self, slot: _Slot, cam: CameraTensors, k: int, k_rows: int, lane: int = 0):
        """Second half of a forward: from the depth-ordered splats to the sorted pair list and the blended image, on the
        current stream with the buffers of ``lane``.  Returns the image buffer."""
        capi, lib = self._capi, self.lib
        c, _keep = slot.cam
        image, final_t, final_idx = self._image_buffers(cam.H, cam.W, lane)
        ranges = self._ranges(slot, cam.H, cam.W)
        ln = self._pair_buffers(k, k_rows, cam.H, cam.W, lane)
        capi.check(lib.dsb_forward_render(
            C.byref(c), self.n, k, k_rows, slot.records.data_ptr(), slot.tiles.data_ptr(), slot.depth_keys.data_ptr(),
            slot.offsets.data_ptr(), ln.pairs.data_ptr(), self._marks(slot, cam.H, cam.W).data_ptr(), ranges.data_ptr(),
            slot.layout.data_ptr(), ln.render_ws.data_ptr(), ln.render_bytes, image.data_ptr(), final_t.data_ptr(),
            final_idx.data_ptr(), None, capi.stream_ptr()))
        self.last_k, self.last_k_rows = k, k_rows
        self.cur = slot
        self._last_cam = cam
        return image

    @_on_own_device
    def forward(self, cam: CameraTensors, slot: int = 0):
        """Returns the image tensor (owned by the renderer, overwritten by the next call of the same size)."""
        capi, lib, p = self._capi, self.lib, self.p
        sl = self._slot(slot)
        sl.cam = self._camera(cam)
        # plan and render in one library call when the pair buffers of the previous view are large enough (they are
        # kept with 25% slack), so that no host work sits between the pair-count read-back and the render
        ln = self.lanes[0]
        image, final_t, final_idx = self._image_buffers(cam.H, cam.W, 0)
        ranges = self._ranges(sl, cam.H, cam.W)
        k, k_rows, rendered = C.c_int64(0), C.c_int64(0), C.c_int32(0)
        capi.check(lib.dsb_forward(
            C.byref(sl.cam[0]), self.n, p["means3d"].data_ptr(), p["shs"].data_ptr(), None, p["opacities"].data_ptr(),
            p["scales"].data_ptr(), p["rotations"].data_ptr(), None, sl.records.data_ptr(), sl.radii.data_ptr(),
            sl.tiles.data_ptr(), self.cov3d.data_ptr(), sl.depth_keys.data_ptr(), self.depth_rows[1, slot].data_ptr(),
            sl.offsets.data_ptr(), self._marks(sl, cam.H, cam.W).data_ptr(), ranges.data_ptr(), sl.layout.data_ptr(),
            self.plan_ws.data_ptr(), self.plan_bytes, ln.pairs.data_ptr() if ln.cap else None, ln.cap,
            ln.render_ws.data_ptr() if ln.cap else None, ln.render_bytes, image.data_ptr(), final_t.data_ptr(),
            final_idx.data_ptr(), None, C.byref(k), C.byref(k_rows), C.byref(rendered), capi.stream_ptr()))
        if not rendered.value:
            return self._render(sl, cam, int(k.value), int(k_rows.value))
        self.last_k, self.last_k_rows = int(k.value), int(k_rows.value)
        self.cur = sl
        self._last_cam = cam
        return image

    @_on_own_device
    def backward(self, v_image: torch.Tensor, grads: GradientBuffer, accumulate: bool = True):
        """Backward of the view rendered by the last forward(); adds into (or overwrites) ``grads``."""
        capi, lib, p = self._capi, self.lib, self.p
        sl, cam = self.cur, self._last_cam
        image, final_t, final_idx = self._image_buffers(cam.H, cam.W)
        ranges = self._ranges(sl, cam.H, cam.W)
        g = grads.views
        capi.check(lib.dsb_backward(
            C.byref(sl.cam[0]), self.n, p["means3d"].data_ptr(), p["scales"].data_ptr(), p["rotations"].data_ptr(),
            sl.records.data_ptr(), self.cov3d.data_ptr(), sl.radii.data_ptr(), self.pairs.data_ptr(),
            ranges.data_ptr(), final_t.data_ptr(), final_idx.data_ptr(), v_image.data_ptr(), None,
            self._marks(sl, cam.H, cam.W).data_ptr(), sl.grad_acc.data_ptr(),
            g["means3d"].data_ptr(), None, g["shs"].data_ptr(), None, g["opacities"].data_ptr(), g["scales"].data_ptr(),
            g["rotations"].data_ptr(), None, 1 if accumulate else 0, capi.stream_ptr()))

    # ---- views with more pairs than one list may hold: rendered in bands of tile rows --------------------------------
    def _plan_band(self, sl: _Slot, cam: CameraTensors, band):
        """Preprocess + plan of one band of tile rows (None: the whole image).  Returns (pairs, row items, status):
        the exact pair count also when it is beyond what one list may hold (status DSB_ERR_TOO_MANY_PAIRS)."""
        capi, lib, p = self._capi, self.lib, self.p
        sl.cam = self._camera(cam)
        sl.cam[0].tile_row_band = 0 if band is None else (band[0] | (band[1] << 16))
        k, k_rows = C.c_int64(0), C.c_int64(0)
        rc = lib.dsb_forward_plan(
            C.byref(sl.cam[0]), self.n, p["means3d"].data_ptr(), p["shs"].data_ptr(), None, p["opacities"].data_ptr(),
            p["scales"].data_ptr(), p["rotations"].data_ptr(), None, sl.records.data_ptr(), sl.radii.data_ptr(),
            sl.tiles.data_ptr(), self.cov3d.data_ptr(), sl.depth_keys.data_ptr(), self.depth_rows[1, 0].data_ptr(),
            sl.offsets.data_ptr(), self._marks(sl, cam.H, cam.W).data_ptr(), self._ranges(sl, cam.H, cam.W).data_ptr(),
            sl.layout.data_ptr(), self.plan_ws.data_ptr(), self.plan_bytes, C.byref(k), C.byref(k_rows), capi.stream_ptr())
        if rc not in (0, capi.DSB_ERR_TOO_MANY_PAIRS):
            capi.check(rc)
        return int(k.value), int(k_rows.value), rc

    @_on_own_device
    def forward_banded(self, cam: CameraTensors, max_pairs: Optional[int] = None):
        """Forward of a view whose pair list may exceed what one list holds (DSB_MAX_PAIRS - 1; ``max_pairs`` lowers the
        limit, which is how the tests exercise this path at small sizes): the image is rendered in bands of tile rows,
        each with its own plan, pair list and ranges, all writing into the same image.  The bands are found by halving:
        a band whose exact pair count is over the limit is split in two.  Returns the image; ``backward_banded`` follows.
        The image is bit for bit the unbanded one; ``self.bands`` lists (first row, one past the last, pairs)."""
        capi = self._capi
        limit = min(int(max_pairs), capi.MAX_PAIRS - 1) if max_pairs else capi.MAX_PAIRS - 1
        tiles_y = (cam.H + 15) // 16
        sl = self._slot(0)
        image, final_t, final_idx = self._image_buffers(cam.H, cam.W, 0)
        todo, done = [(0, tiles_y)], []
        while todo:
            y0, y1 = todo.pop(0)
            whole = (y0, y1) == (0, tiles_y)
            k, k_rows, rc = self._plan_band(sl, cam, None if whole else (y0, y1))
            if k > limit or rc != 0:
                if y1 - y0 == 1:
                    raise capi.DsbError(capi.DSB_ERR_TOO_MANY_PAIRS, f"tile row {y0} alone holds {k} pairs, more than one list may hold")
                mid = (y0 + y1) // 2
                todo[:0] = [(y0, mid), (mid, y1)]
                continue
            # this band fits: render it into the shared image with buffers of its own, kept for the backward
            band = _Lane()
            band.img = self.lanes[0].img      # every band writes into the one image
            self.lanes.append(band)
            try:
                self._render(sl, cam, k, k_rows, lane=len(self.lanes) - 1)
            finally:
                self.lanes.pop()
            done.append(dict(rows=(y0, y1), k=k, pairs=band.pairs, cam=sl.cam, ranges=self._ranges(sl, cam.H, cam.W).clone(),
                             order=self._marks(sl, cam.H, cam.W).clone()))
            band.render_ws = None   # only the list survives
        self._banded = (cam, done)
        self.bands = [(b["rows"][0], b["rows"][1], b["k"]) for b in done]
        self.cur, self._last_cam = sl, cam
        return image

    @_on_own_device
    def backward_banded(self, v_image: torch.Tensor, grads: GradientBuffer, accumulate: bool = True):
        """Backward of the view ``forward_banded`` rendered: every band's backward blend adds into the one accumulator
        (the records differ between bands only in their tile rectangles, which the backward does not read), then the
        per-splat backward runs once."""
        capi, lib, p = self._capi, self.lib, self.p
        cam, bands = self._banded
        sl = self.cur
        _image, final_t, final_idx = self._image_buffers(cam.H, cam.W, 0)
        for i, b in enumerate(bands):
            capi.check(lib.dsb_backward_blend(
                C.byref(b["cam"][0]), self.n, sl.records.data_ptr(), b["pairs"].data_ptr(), b["ranges"].data_ptr(),
                final_t.data_ptr(), final_idx.data_ptr(), v_image.data_ptr(), None, b["order"].data_ptr(),
                sl.grad_acc.data_ptr(), 1 if i else 0, capi.stream_ptr()))
        g = grads.views
        cams = (capi.DsbCamera * 1)(bands[0]["cam"][0])
        ptrs = lambda ts: (C.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
        capi.check(lib.dsb_geometry_backward_views(
            cams, 1, self.n, p["means3d"].data_ptr(), p["scales"].data_ptr(), p["rotations"].data_ptr(), self.cov3d.data_ptr(),
            ptrs([sl.records]), ptrs([sl.radii]), ptrs([sl.grad_acc]), g["means3d"].data_ptr(), None, g["shs"].data_ptr(), None,
            g["opacities"].data_ptr(), g["scales"].data_ptr(), g["rotations"].data_ptr(), None, 1 if accumulate else 0,
            capi.stream_ptr()))

    @_on_own_device
    def render_views(self, cameras, image_grads, grads: GradientBuffer, accumulate: bool = False,
                     stats: Optional[DensifyStats] = None):
        """Forward + backward of ``cameras`` with the gradients of all of them summed into ``grads`` (added to its
        contents when ``accumulate``).  ``image_grads`` is a sequence of dL/dimage tensors or a callable
        ``(index, image) -> dL/dimage``; it is called under the stream its view runs on (``view_streams`` of them
        take turns), so buffers it reuses from call to call must be per stream, as ``ImageLoss`` keeps them.  Views are
        taken in batches of up to ``batch_views`` of one image size:
        one preprocess launch (with the tile layout of every view) and one plan (depth sorts, offset scans, a
        single read-back of the pair counts) for the batch, then per view the rest of the forward and the backward blend, then one per-splat backward for
        the batch, which also updates ``stats`` (a ``DensifyStats``) when given."""
        capi, lib, p = self._capi, self.lib, self.p
        g = grads.views
        b0, first = 0, True
        self.last_ks = []          # pair count of every view of this call
        while b0 < len(cameras):
            size = (cameras[b0].H, cameras[b0].W)
            b1 = b0 + 1
            while b1 < len(cameras) and b1 - b0 < self.batch_views and (cameras[b1].H, cameras[b1].W) == size:
                b1 += 1
            nv = b1 - b0
            slots = [self._slot(j) for j in range(nv)]
            for j, sl in enumerate(slots):
                sl.cam = self._camera(cameras[b0 + j])
            cams = (capi.DsbCamera * nv)(*[sl.cam[0] for sl in slots])
            ptrs = lambda ts: (C.c_void_p * len(ts))(*[t.data_ptr() for t in ts])
            main = torch.cuda.current_stream(self.dev)
            nl = min(self.view_streams, nv)
            lanes = [self._lane(i) for i in range(nl)]
            capi.check(lib.dsb_preprocess_views(
                cams, nv, self.n, p["means3d"].data_ptr(), p["shs"].data_ptr(), None, p["opacities"].data_ptr(),
                p["scales"].data_ptr(), p["rotations"].data_ptr(), None, ptrs([sl.records for sl in slots]),
                ptrs([sl.radii for sl in slots]), ptrs([sl.tiles for sl in slots]), self.cov3d.data_ptr(),
                ptrs([sl.depth_keys for sl in slots]), ptrs([self._marks(sl, *size) for sl in slots]),
                ptrs([self._ranges(sl, *size) for sl in slots]), ptrs([sl.layout for sl in slots]), capi.stream_ptr()))
            # depth order and row-item offsets of all views: launched without a host wait, then ONE read-back of the totals
            capi.check(lib.dsb_plan_views(
                C.byref(slots[0].cam[0]), nv, self.n, self.n, ptrs([sl.records for sl in slots]), self.tiles_rows.data_ptr(),
                self.depth_rows[0].data_ptr(), self.depth_rows[1].data_ptr(), self.offset_rows.data_ptr(),
                ptrs([sl.layout for sl in slots]), self.plan_ws.data_ptr(), self.plan_bytes, None, None, capi.stream_ptr()))
            ks, krs = (C.c_int64 * nv)(), (C.c_int64 * nv)()
            capi.check(lib.dsb_plan_totals_views(nv, self.n, self.plan_ws.data_ptr(), self.plan_bytes, ks, krs,
                                                 capi.stream_ptr()))
            self.last_ks.extend(int(k) for k in ks)
            # The K-sized stages of the views, dealt over the lanes: lane 0 is the caller's stream, the others wait for
            # the batch's plan, and the caller's stream waits for them before the per-splat backward.
            planned = torch.cuda.Event()
            planned.record(main)
            for ln in lanes[1:]:
                ln.stream.wait_event(planned)
            for j, sl in enumerate(slots):
                cam, li = cameras[b0 + j], j % nl
                with torch.cuda.stream(lanes[li].stream if li else main):
                    image = self._render(sl, cam, int(ks[j]), int(krs[j]), lane=li)
                    v_image = image_grads(b0 + j, image) if callable(image_grads) else image_grads[b0 + j]
                    _img, final_t, final_idx = self._image_buffers(cam.H, cam.W, li)
                    ranges = self._ranges(sl, cam.H, cam.W)
                    capi.check(lib.dsb_backward_blend(
                        C.byref(sl.cam[0]), self.n, sl.records.data_ptr(), lanes[li].pairs.data_ptr(),
                        ranges.data_ptr(), final_t.data_ptr(), final_idx.data_ptr(), v_image.data_ptr(), None,
                        self._marks(sl, cam.H, cam.W).data_ptr(), sl.grad_acc.data_ptr(), 0, capi.stream_ptr()))
            for ln in lanes[1:]:
                done = torch.cuda.Event()
                done.record(ln.stream)
                main.wait_event(done)
            geo_args = (
                cams, nv, self.n, p["means3d"].data_ptr(), p["scales"].data_ptr(), p["rotations"].data_ptr(),
                self.cov3d.data_ptr(), ptrs([sl.records for sl in slots]), ptrs([sl.radii for sl in slots]),
                ptrs([sl.grad_acc for sl in slots]), g["means3d"].data_ptr(), None, g["shs"].data_ptr(), None,
                g["opacities"].data_ptr(), g["scales"].data_ptr(), g["rotations"].data_ptr(), None,
                1 if (accumulate or not first) else 0)
            if stats is None:
                capi.check(lib.dsb_geometry_backward_views(*geo_args, capi.stream_ptr()))
            else:
                sx, sy = (0.5 * size[1], 0.5 * size[0]) if stats.ndc_units else (1.0, 1.0)
                capi.check(lib.dsb_geometry_backward_views_stats(
                    *geo_args, sx, sy, stats.grad_norm_sum.data_ptr(), stats.visible_count.data_ptr(),
                    stats.max_radius.data_ptr(), capi.stream_ptr()))
            first = False
            b0 = b1


class ImageLoss:
    """L = (1 - lambda) * mean|image - target| + lambda * (1 - mean SSIM(image, target)) and dL/dimage in two kernel
    launches (``dsb_image_loss_backward``; one launch when lambda is 0), with buffers that are reused from call to call.
    Targets are float images or 8-bit ones (value / 255).  ``__call__`` returns
    (dL/dimage [H, W, 3], loss as a one-element device tensor -- reading it is the caller's synchronisation);
    it has the ``(index, image)`` form ``ViewRenderer.render_views`` expects of its ``image_grads`` argument when
    built with a list of target images."""

    def __init__(self, targets=None, lambda_dssim: float = 0.2):
        from . import _capi
        self._capi, self.lib = _capi, _capi.lib()
        self.targets, self.lam = targets, float(lambda_dssim)
        self.buf = {}
        self.losses = []

    def gradient(self, image: torch.Tensor, target: torch.Tensor):
        if not image.is_cuda or target.device != image.device:
            raise RuntimeError(f"ImageLoss launches CUDA kernels: image is on {image.device}, target on {target.device}")
        with torch.cuda.device(image.device):
            return self._gradient(image, target)

    def _gradient(self, image: torch.Tensor, target: torch.Tensor):
        h, w = image.shape[0], image.shape[1]
        # one set of buffers per stream: render_views calls this under the stream of the view's lane, and a buffer
        # shared by two lanes would be rewritten while the other lane's backward still reads it
        stream = self._capi.stream_ptr(image.device)
        key = (h, w, image.device, stream)
        if key not in self.buf:
            nbytes = int(self.lib.dsb_image_loss_workspace_bytes(h, w))
            self.buf[key] = (torch.empty(nbytes, dtype=torch.uint8, device=image.device), torch.empty_like(image))
        ws, v_image = self.buf[key]
        loss = torch.empty(1, dtype=torch.float32, device=image.device)
        image, target = image.contiguous(), target.contiguous()
        if target.dtype == torch.uint8:   # 8-bit targets stand for value / 255
            if self.lam == 0.0:
                self._capi.check(self.lib.dsb_l1_loss_backward_u8(image.data_ptr(), target.data_ptr(), h, w, v_image.data_ptr(),
                                                                  loss.data_ptr(), stream))
                return v_image, loss
            target = target.to(torch.float32).mul_(1.0 / 255.0)
        self._capi.check(self.lib.dsb_image_loss_backward(image.data_ptr(), target.data_ptr(), h, w, self.lam, ws.data_ptr(),
                                                          ws.numel(), v_image.data_ptr(), loss.data_ptr(), stream))
        return v_image, loss

    def __call__(self, index: int, image: torch.Tensor):
        v_image, loss = self.gradient(image, self.targets[index])
        self.losses.append(loss)
        return v_image


class FlatAdam:
    """Adam over the five parameter tensors of a splat cloud, fed from a ``GradientBuffer``: one fused kernel launch
    per tensor (``dsb_adam_step``), each with its own learning rate as 3DGS training uses them, moments kept in one
    flat allocation laid out like the gradient block.  The update is torch.optim.Adam's (no weight decay, no
    amsgrad); ``grad_scale`` turns the summed gradient of a multi-view, multi-rank step into a mean on the fly."""

    def __init__(self, params: Dict[str, torch.Tensor], lrs: Dict[str, float], betas=(0.9, 0.999), eps: float = 1e-15):
        from . import _capi
        self._capi, self.lib = _capi, _capi.lib()
        self.params, self.lrs, self.betas, self.eps = params, dict(lrs), betas, eps
        self.step_count = 0
        n = params["means3d"].shape[0]
        dev = params["means3d"].device
        self.dev = dev
        self.m = GradientBuffer(n, dev, sh_coeffs=params["shs"].shape[1])
        self.v = GradientBuffer(n, dev, sh_coeffs=params["shs"].shape[1])

    @_on_own_device
    def step(self, grads: GradientBuffer, grad_scale: float = 1.0):
        self.step_count += 1
        for name, _ in SEGMENTS:
            p, g = self.params[name], grads.views[name]
            if not p.is_contiguous() or p.numel() != g.numel():
                raise ValueError(f"{name}: parameter and gradient layouts differ")
            self._capi.check(self.lib.dsb_adam_step(
                p.data_ptr(), g.data_ptr(), self.m.views[name].data_ptr(), self.v.views[name].data_ptr(), p.numel(),
                float(self.lrs[name]), float(self.betas[0]), float(self.betas[1]), float(self.eps), self.step_count,
                float(grad_scale), self._capi.stream_ptr()))


def _group_info(group=None):
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(group), dist.get_rank(group)
    return 1, 0


def _adam_kernel_update(capi):
    lib = capi.lib()

    def update(p, g, m, v, lr, beta1, beta2, eps, step, grad_scale):
        with torch.cuda.device(p.device):
            capi.check(lib.dsb_adam_step(p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), p.numel(), float(lr),
                                         float(beta1), float(beta2), float(eps), int(step), float(grad_scale),
                                         capi.stream_ptr(p.device)))
    return update


class ShardedAdam:
    """The optimizer step of a data-parallel training step with the gradient sum folded in:

        reduce-scatter of the flat gradient block  ->  Adam on this rank's 1/G slice  ->  all-gather of the parameters

    instead of all-reduce + Adam over everything on every rank.  The bytes that cross NVLink are those of the
    all-reduce (a ring all-reduce is this reduce-scatter followed by this all-gather), the optimizer pass and its
    moment buffers shrink to 1/G per rank, and the parameters every rank holds afterwards are identical to the
    replicated form's up to the order in which the ranks' gradients are summed.  Both collectives run in place on
    the two flat allocations (``GradientBuffer`` / ``ParameterBuffer`` built with ``shards=world_size * chunks``): the
    kernels' output buffer is the communication buffer.  In a single process it degenerates to plain Adam over
    everything.

    ``chunks`` > 1 cuts the block into that many contiguous chunks, each reduce-scattered, updated and all-gathered on
    its own; a rank then owns slice ``rank`` of every chunk.  With ``gather_group`` (a second process group over the
    same ranks, i.e. a second communicator) on CUDA devices the chunks are pipelined: the update and the all-gather of
    chunk c run on a second stream beside the reduce-scatter of chunk c + 1.  A reduce-scatter mostly sends and an
    all-gather mostly receives when the switch reduces and multicasts (NVLS), so the two directions of the links work
    at the same time; over rings or a single peer link the pipeline costs nothing and gains little.  Results do not
    depend on ``chunks`` beyond the order of the sums.

    ``update`` is the per-slice Adam update, ``update(p, g, m, v, lr, beta1, beta2, eps, step, grad_scale)`` in place on
    flat tensors; the default launches ``dsb_adam_step``.  (Tests on CPU ranks pass the checker's update.)"""

    def __init__(self, params: ParameterBuffer, lrs: Dict[str, float], betas=(0.9, 0.999), eps: float = 1e-15, group=None,
                 update=None, chunks: int = 1, gather_group=None):
        self.params, self.lrs, self.betas, self.eps, self.group = params, dict(lrs), betas, float(eps), group
        self.world, self.rank = _group_info(group)
        self.chunks = max(1, int(chunks))
        self.gather_group = gather_group
        total = params.storage.numel()
        if total % (4 * self.world * self.chunks) != 0:
            raise ValueError(f"the parameter block of {total} elements does not split into {self.world * self.chunks} "
                             f"slices of whole 16-byte lanes: build ParameterBuffer and GradientBuffer with "
                             f"shards={self.world * self.chunks}")
        self.span = total // self.chunks          # elements of one chunk
        self.piece = self.span // self.world      # this rank's slice of a chunk
        self.chunk = total // self.world          # elements this rank owns in all
        dev = params.storage.device
        self.m = torch.zeros(self.chunk, dtype=torch.float32, device=dev)
        self.v = torch.zeros(self.chunk, dtype=torch.float32, device=dev)
        # per chunk: this rank's slice [lo, hi) of the flat block and the parts of it that belong to each parameter
        # tensor (each has its own learning rate) with their place in the moment buffers
        self.slices = []
        for c in range(self.chunks):
            lo = c * self.span + self.rank * self.piece
            hi = lo + self.piece
            parts = []
            for name, _ in SEGMENTS:
                a, b = params.segments[name]
                a, b = max(a, lo), min(b, hi)
                if a < b:
                    parts.append((name, a, b, c * self.piece + (a - lo)))
            self.slices.append((lo, hi, parts))
        self.lo, self.hi = self.slices[0][0], self.slices[0][1]           # the one slice when chunks == 1
        self.pieces = [(name, a, b) for _, _, parts in self.slices for name, a, b, _ in parts]
        self.step_count = 0
        if update is None:
            from . import _capi
            update = _adam_kernel_update(_capi)
        self.update = update
        self._streams = None

    def _update_slice(self, grads: GradientBuffer, c: int, grad_scale: float):
        for name, a, b, mo in self.slices[c][2]:
            self.update(self.params.storage[a:b], grads.storage[a:b], self.m[mo:mo + (b - a)], self.v[mo:mo + (b - a)],
                        self.lrs[name], self.betas[0], self.betas[1], self.eps, self.step_count, grad_scale)

    def pipelined(self) -> bool:
        return (self.world > 1 and self.chunks > 1 and self.gather_group is not None
                and self.params.storage.device.type == "cuda")

    def step(self, grads: GradientBuffer, grad_scale: float = 1.0, marks=None):
        """``marks``: an optional callable invoked after each phase of an unpipelined step (reduce-scatter, update,
        all-gather, in that order, once per chunk), for callers that record events between the phases."""
        import torch.distributed as dist
        if grads.storage.numel() != self.params.storage.numel():
            raise ValueError("gradient and parameter blocks are laid out differently")
        self.step_count += 1
        P, G = self.params.storage, grads.storage
        if not self.pipelined():
            for c, (lo, hi, _) in enumerate(self.slices):
                first, last = c * self.span, (c + 1) * self.span
                if self.world > 1:
                    dist.reduce_scatter_tensor(G[lo:hi], G[first:last], op=dist.ReduceOp.SUM, group=self.group)
                if marks:
                    marks()
                self._update_slice(grads, c, grad_scale)
                if marks:
                    marks()
                if self.world > 1:
                    dist.all_gather_into_tensor(P[first:last], P[lo:hi], group=self.gather_group or self.group)
                if marks:
                    marks()
            return
        # Pipelined: reduce-scatters in order on one stream (first communicator), update + all-gather of every chunk on a
        # second stream (second communicator) as soon as that chunk's reduce-scatter is done.
        if self._streams is None:
            dev = P.device
            self._streams = (torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev),
                             [torch.cuda.Event() for _ in range(self.chunks)])
        reduce_stream, gather_stream, reduced = self._streams
        caller = torch.cuda.current_stream(P.device)
        reduce_stream.wait_stream(caller)
        gather_stream.wait_stream(caller)
        for c, (lo, hi, _) in enumerate(self.slices):
            first, last = c * self.span, (c + 1) * self.span
            with torch.cuda.stream(reduce_stream):
                dist.reduce_scatter_tensor(G[lo:hi], G[first:last], op=dist.ReduceOp.SUM, group=self.group)
                reduced[c].record(reduce_stream)
            with torch.cuda.stream(gather_stream):
                gather_stream.wait_event(reduced[c])
                self._update_slice(grads, c, grad_scale)
                dist.all_gather_into_tensor(P[first:last], P[lo:hi], group=self.gather_group)
        caller.wait_stream(reduce_stream)
        caller.wait_stream(gather_stream)


def register_with_nccl(make_buffers, group=None, more_groups=()):
    """Runs ``make_buffers()`` (a callable that allocates and returns the communication buffers) under a memory
    pool of NCCL's own allocator and registers that pool with the process group, so that the collectives on those
    buffers take NCCL's registered-buffer path (zero-copy, and in-switch reduction over NVSwitch where the
    communicator has it).  Returns (buffers, pool or None): when the backend has no such allocator (gloo, an older
    NCCL) or registration fails, the buffers come from torch's ordinary allocator and the second value is None --
    the collectives still run, through NCCL's staging buffers.  Keep the pool alive as long as the buffers.
    ``more_groups``: further process groups whose communicators should know the pool as well."""
    import torch.distributed as dist
    try:
        if not (dist.is_available() and dist.is_initialized()) or dist.get_backend(group) != "nccl":
            return make_buffers(), None
        backend = (group or dist.group.WORLD)._get_backend(torch.device("cuda"))
        if not getattr(backend, "supports_mem_allocator", True):
            return make_buffers(), None
        pool = torch.cuda.MemPool(backend.mem_allocator)
        with torch.cuda.use_mem_pool(pool):
            buffers = make_buffers()
        backend.register_mem_pool(pool)
        for g in more_groups:   # further communicators over the same ranks that will use the buffers (ShardedAdam's gather_group)
            try:
                g._get_backend(torch.device("cuda")).register_mem_pool(pool)
            except Exception:
                pass            # that communicator stages through its own buffers
        return buffers, pool
    except Exception:   # anything the running torch / NCCL pair does not offer: plain buffers
        return make_buffers(), None


def data_parallel_step(renderer: ViewRenderer, cameras: Sequence[CameraTensors], image_grads,
                       grads: GradientBuffer, group=None, stats: Optional[DensifyStats] = None) -> None:
    """One step of the multi-view batch on this rank: forward + backward of each local camera (gradients
    summed into ``grads``), then the all-reduce.  ``cameras`` is this rank's shard; ``image_grads`` is the
    matching sequence of dL/dimage tensors, or a callable ``(index, image) -> dL/dimage`` (the loss)."""
    if len(cameras) == 0:
        grads.zero_()  # a rank without views still takes part in the collective
    else:
        renderer.render_views(cameras, image_grads, grads, accumulate=False, stats=stats)
    allreduce_gradients(grads, group)


def training_step(renderer: ViewRenderer, cameras: Sequence[CameraTensors], image_grads, grads: GradientBuffer,
                  optimizer: ShardedAdam, grad_scale: float = 1.0, stats: Optional[DensifyStats] = None) -> None:
    """One whole training step on this rank: forward + backward of its cameras, then ``ShardedAdam.step`` (gradient
    reduce-scatter, Adam on the rank's slice, parameter all-gather).  The renderer must have been built on the views
    of the optimizer's ``ParameterBuffer`` so that the next step renders the updated cloud."""
    if len(cameras) == 0:
        grads.zero_()
    else:
        renderer.render_views(cameras, image_grads, grads, accumulate=False, stats=stats)
    optimizer.step(grads, grad_scale=grad_scale)
