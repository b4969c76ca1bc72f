"""Python operator: ``GaussianRasterizationSettings`` / ``GaussianRasterizer`` with the reference's
surface (ds_splat/rasterizer.py:115-194) over the sm_100a library.

Drop-in by import swap: ``from ds_splat_b200 import GaussianRasterizationSettings, GaussianRasterizer``.
The positional call of the reference ``rasterizer(means_3d, means_2d, shs, colors_precomp, opacities,
scales, rotations, cov_3d_precomp)`` works unchanged; graphdeco's keyword names (``means3D=...,
cov3D_precomp=...``) are accepted too.  The result is ``(image[H,W,3], radii[N])`` as in the reference
(``channels_first=True`` in the settings gives graphdeco's ``[3,H,W]``).  ``return_depth=True`` adds a third
result, the blended view-space depth map ``[H,W]`` (``sum z_i alpha_i T_i``; the reference has no depth
output), which is differentiable like the image.

Differences from the reference that a caller can observe, all deliberate:
  * work is enqueued on the *current* torch stream of the inputs' device (the reference uses the
    legacy default stream and the current device);
  * the camera matrices are read in the transposed form the settings carry them in, so the two
    per-call transposes of ``settings_for_cpp_code`` (:147-148) disappear;
  * tensors saved for backward are this library's own (packed records, sorted pairs), not the
    reference's nine-tensor list.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch

from . import _capi


@dataclass(init=False)
class GaussianRasterizationSettings:
    """Same thirteen fields, in the same order, as the reference's dataclass
    (ds_splat/rasterizer.py:115-129).  ``max_sh_degree`` defaults to 3 so that graphdeco-style keyword
    construction (which has no such field) works; ``channels_first``, ``strict_reference``, ``return_depth`` and
    ``tight_tiles`` are additions."""
    image_height: int
    image_width: int
    tanfovx: float
    tanfovy: float
    bg: torch.Tensor
    scale_modifier: float
    viewmatrix: torch.Tensor
    projmatrix: torch.Tensor
    sh_degree: int
    max_sh_degree: int
    campos: torch.Tensor
    prefiltered: bool
    debug: bool
    channels_first: bool
    strict_reference: bool
    return_depth: bool
    tight_tiles: bool

    def __init__(self, image_height, image_width, tanfovx, tanfovy, bg, scale_modifier, viewmatrix, projmatrix,
                 sh_degree, max_sh_degree=3, campos=None, prefiltered=False, debug=False, channels_first=False,
                 strict_reference=True, return_depth=False, tight_tiles=True):
        if campos is None:
            raise TypeError("GaussianRasterizationSettings: campos is required")
        self.image_height, self.image_width = int(image_height), int(image_width)
        self.tanfovx, self.tanfovy = float(tanfovx), float(tanfovy)
        self.bg, self.scale_modifier = bg, float(scale_modifier)
        self.viewmatrix, self.projmatrix = viewmatrix, projmatrix
        self.sh_degree, self.max_sh_degree = int(sh_degree), int(max_sh_degree)
        self.campos, self.prefiltered, self.debug = campos, bool(prefiltered), bool(debug)
        # strict_reference keeps the reference's habit of never drawing the splat with the highest index
        # (cpp/rasterizer_torch.cu:97-104), which bit-exact parity of the sorted lists requires.
        self.channels_first, self.strict_reference = bool(channels_first), bool(strict_reference)
        # return_depth makes the rasterizer return (image, radii, depth) instead of the reference's (image, radii).
        self.return_depth = bool(return_depth)
        # tight_tiles pairs a splat only with the tiles it can contribute to (a subset of the reference's pair list);
        # image, radii and gradients are the same either way, the pair list and its sort are a third to a half shorter.
        self.tight_tiles = bool(tight_tiles)


def _camera_for(settings: GaussianRasterizationSettings, device):
    """DsbCamera of the settings, rebuilt only when a field or a settings tensor changed since the last call (the
    reference rebuilds its settings struct and transposes both matrices on every call, ds_splat/rasterizer.py:137-155)."""
    tensors = (settings.viewmatrix, settings.projmatrix, settings.campos, settings.bg)
    # The camera block only holds device POINTERS, so it stays valid while the settings tensors stay where they are
    # (their contents may change in place).  Tensors that first have to be converted are not cached.
    direct = all(t is None or (isinstance(t, torch.Tensor) and t.device == device and t.dtype == torch.float32
                               and t.is_contiguous()) for t in tensors)
    key = None
    if direct:
        key = (device, settings.image_height, settings.image_width, settings.tanfovx, settings.tanfovy,
               settings.scale_modifier, settings.sh_degree, settings.max_sh_degree, settings.strict_reference,
               settings.tight_tiles, tuple(0 if t is None else t.data_ptr() for t in tensors))
        cached = getattr(settings, "_dsb_camera", None)
        if cached is not None and cached[0] == key:
            return cached[1], cached[2]

    def dev_f32(t, name, numel):
        if not isinstance(t, torch.Tensor):
            t = torch.as_tensor(t, dtype=torch.float32)
        if t.numel() != numel:
            raise ValueError(f"{name} must have {numel} elements, got {t.numel()}")
        return t.to(device=device, dtype=torch.float32).contiguous()

    view = dev_f32(settings.viewmatrix, "viewmatrix", 16)
    proj = dev_f32(settings.projmatrix, "projmatrix", 16)
    campos = dev_f32(settings.campos, "campos", 3)
    bg = dev_f32(settings.bg, "bg", 3) if settings.bg is not None else None
    if settings.max_sh_degree not in (0, 1, 2, 3):
        raise ValueError("max_sh_degree must be in 0..3")
    cam, keep = _capi.make_camera(settings.image_height, settings.image_width, settings.tanfovx, settings.tanfovy, view,
                                  proj, campos, bg, settings.sh_degree, settings.max_sh_degree, settings.scale_modifier,
                                  transposed=True, drop_last=settings.strict_reference, tight_tiles=settings.tight_tiles)
    if key is not None:
        settings._dsb_camera = (key, cam, keep)
    return cam, keep


def _up256(nbytes: int) -> int:
    return (nbytes + 255) & ~255


class _Layout:
    """Byte offsets of the operator's internal buffers inside ONE allocation per call (the reference allocates
    about twenty tensors per forward, cpp/rasterizer_torch.cu:139-157,52-53,90,106-107): everything whose size
    follows from N and the image size.  Pure arithmetic, cached per (N, H, W)."""
    _cache = {}

    def __init__(self, n, h, w, lib):
        off = 0

        def take(nbytes):
            nonlocal off
            at = off
            off += _up256(max(int(nbytes), 1))
            return at

        self.plan_bytes = int(lib.dsb_plan_workspace_bytes(n))
        self.records = take(n * _capi.RECORD_FLOATS * 4)
        self.tiles = take(n * 4)
        self.cov3d = take(n * 24)
        self.depth_keys = take(n * 8)
        self.depth_keys_alt = take(n * 8)
        self.offsets = take(n * 4)
        self.tile_marks = take(int(lib.dsb_tile_marks_bytes(h, w)))
        self.plan_ws = take(self.plan_bytes)
        self.ranges = take((_capi.num_tiles(h, w) + 1) * 4)
        self.layout = take(_capi.LAYOUT_WORDS * 4)
        self.final_t = take(h * w * 4)
        self.final_idx = take(h * w * 4)
        self.grad_acc = take(n * _capi.GRAD_FLOATS * 4)
        self.total = off

    @classmethod
    def of(cls, n, h, w, lib):
        key = (n, h, w)
        got = cls._cache.get(key)
        if got is None:
            if len(cls._cache) > 64:
                cls._cache.clear()
            got = cls._cache[key] = cls(n, h, w, lib)
        return got


# pair count of the last forward per (device, N, H, W): the next call of that shape brings buffers for 25% more, so
# that the render can follow the pair-count read-back inside one library call
_pair_hint = {}


class DsRasterizerFunction(torch.autograd.Function):
    """Counterpart of the reference's autograd Function (ds_splat/rasterizer.py:7-112): eight tensor inputs
    plus the settings; returns (image, radii) -- (image, radii, depth) with ``return_depth`` -- and backward returns
    one gradient per tensor input, shaped like that input."""

    @staticmethod
    def forward(ctx, means_3d, means_2d, shs, colors_precomp, opacities, scales, rotations, cov_3d_precomp,
                raster_settings):
        lib = _capi.lib()
        if not isinstance(means_3d, torch.Tensor) or not means_3d.is_cuda:
            raise RuntimeError("means_3d must be a CUDA tensor")
        dev = means_3d.device
        shapes = tuple(t.shape if isinstance(t, torch.Tensor) else None
                       for t in (means_3d, means_2d, shs, colors_precomp, opacities, scales, rotations, cov_3d_precomp))
        means_3d = _capi.as_f32(means_3d, dev, "means_3d")
        if means_3d is None:
            raise RuntimeError("means_3d is empty")
        opacities = _capi.as_f32(opacities, dev, "opacities")
        shs = _capi.as_f32(shs, dev, "shs")
        colors_precomp = _capi.as_f32(colors_precomp, dev, "colors_precomp")
        scales = _capi.as_f32(scales, dev, "scales")
        rotations = _capi.as_f32(rotations, dev, "rotations")
        cov_3d_precomp = _capi.as_f32(cov_3d_precomp, dev, "cov_3d_precomp")
        n = means_3d.shape[0]
        if opacities is None or opacities.numel() != n:
            raise RuntimeError("opacities must have one value per splat")
        if colors_precomp is None and shs is None:
            raise RuntimeError("SHS error: provide shs or colors_precomp")  # the reference's check, rasterizer_torch.cu:187-189
        if cov_3d_precomp is None and (scales is None or rotations is None or scales.shape[0] != rotations.shape[0]):
            raise RuntimeError("cov3D error: provide scales and rotations, or cov_3d_precomp")  # :184-186
        if shs is not None:
            coeffs = (raster_settings.max_sh_degree + 1) ** 2
            if shs.numel() != n * coeffs * 3:
                raise RuntimeError(f"shs must be [N, {coeffs}, 3] for max_sh_degree={raster_settings.max_sh_degree}")
        h, w = raster_settings.image_height, raster_settings.image_width

        with torch.cuda.device(dev):
            cam, keep = _camera_for(raster_settings, dev)
            stream = _capi.stream_ptr()
            lay = _Layout.of(n, h, w, lib)
            arena = torch.empty(lay.total, dtype=torch.uint8, device=dev)
            a = arena.data_ptr()
            radii = torch.empty(n, dtype=torch.int32, device=dev)
            image = torch.empty((h, w, 3), dtype=torch.float32, device=dev)
            depth = torch.empty((h, w), dtype=torch.float32, device=dev) if raster_settings.return_depth else None
            cov3d_ptr = cov_3d_precomp.data_ptr() if cov_3d_precomp is not None else a + lay.cov3d

            # Pair list and render workspace are sized from the counts of the previous call of this shape, with 25%
            # slack, so that plan and render run inside one library call; a view that needs more gets more.
            hint_key = (dev, n, h, w, raster_settings.tight_tiles)
            hint_k, hint_rows = _pair_hint.get(hint_key, (8 * n, 0))
            cap, cap_rows = max(int(hint_k * 1.25), 1024), int(hint_rows * 1.25)   # row items only when views are row-binned
            ws_bytes = int(lib.dsb_render_workspace_bytes(h, w, cap, cap_rows))
            pair_arena = torch.empty(_up256(cap * 8) + ws_bytes, dtype=torch.uint8, device=dev)
            b = pair_arena.data_ptr()
            k, k_rows, rendered = C.c_int64(0), C.c_int64(0), C.c_int32(0)
            _capi.check(lib.dsb_forward(
                C.byref(cam), n, _capi.ptr(means_3d), _capi.ptr(shs), _capi.ptr(colors_precomp), _capi.ptr(opacities),
                _capi.ptr(scales), _capi.ptr(rotations), _capi.ptr(cov_3d_precomp), a + lay.records, radii.data_ptr(),
                a + lay.tiles, cov3d_ptr, a + lay.depth_keys, a + lay.depth_keys_alt, a + lay.offsets, a + lay.tile_marks,
                a + lay.ranges, a + lay.layout, a + lay.plan_ws, lay.plan_bytes, b, cap, b + _up256(cap * 8), ws_bytes,
                image.data_ptr(), a + lay.final_t, a + lay.final_idx, _capi.ptr(depth),
                C.byref(k), C.byref(k_rows), C.byref(rendered), stream))
            k, k_rows = int(k.value), int(k_rows.value)
            _pair_hint[hint_key] = (k, k_rows)
            if not rendered.value:   # more pairs or row items than the buffers brought along hold: grow them and render
                cap = max(k, 1)
                ws_bytes = int(lib.dsb_render_workspace_bytes(h, w, k, k_rows))
                pair_arena = torch.empty(_up256(cap * 8) + ws_bytes, dtype=torch.uint8, device=dev)
                b = pair_arena.data_ptr()
                _capi.check(lib.dsb_forward_render(
                    C.byref(cam), n, k, k_rows, a + lay.records, a + lay.tiles, a + lay.depth_keys, a + lay.offsets, b,
                    a + lay.tile_marks, a + lay.ranges, a + lay.layout, b + _up256(cap * 8), ws_bytes,
                    image.data_ptr(), a + lay.final_t, a + lay.final_idx, _capi.ptr(depth), stream))

        ctx.raster_settings = raster_settings
        ctx.num_pairs = k
        ctx.layout = lay
        ctx.shapes = shapes
        ctx.had = (shs is not None, colors_precomp is not None, scales is not None, rotations is not None,
                   cov_3d_precomp is not None)
        empty = means_3d.new_empty(0)
        ctx.save_for_backward(means_3d, scales if scales is not None else empty, rotations if rotations is not None else empty,
                              cov_3d_precomp if cov_3d_precomp is not None else empty, arena, pair_arena, radii)
        ctx.mark_non_differentiable(radii)
        if raster_settings.channels_first:
            image = image.permute(2, 0, 1)
        if raster_settings.return_depth:
            return image, radii, depth
        return image, radii

    @staticmethod
    def backward(ctx, rendered_img_grad, _radii_grad, depth_grad=None):
        lib = _capi.lib()
        means_3d, scales, rotations, cov_3d_precomp, arena, pair_arena, radii = ctx.saved_tensors
        settings, lay = ctx.raster_settings, ctx.layout
        had_shs, had_colors, had_scales, had_rots, had_cov = ctx.had
        dev = means_3d.device
        n = means_3d.shape[0]
        h, w = settings.image_height, settings.image_width
        if rendered_img_grad is None:  # only the depth map took part in the loss
            rendered_img_grad = means_3d.new_zeros((h, w, 3))
        elif settings.channels_first:
            rendered_img_grad = rendered_img_grad.permute(1, 2, 0)
        v_image = rendered_img_grad.to(dtype=torch.float32).contiguous()
        v_depth = depth_grad.to(dtype=torch.float32).contiguous() if depth_grad is not None else None
        need = ctx.needs_input_grad
        coeffs = (settings.max_sh_degree + 1) ** 2
        a = arena.data_ptr()
        cov3d_ptr = cov_3d_precomp.data_ptr() if had_cov else a + lay.cov3d

        with torch.cuda.device(dev):
            cam, keep = _camera_for(settings, dev)
            f32 = dict(dtype=torch.float32, device=dev)
            v_means3d = torch.empty((n, 3), **f32) if need[0] else None
            v_means2d = torch.empty((n, 3), **f32) if need[1] else None
            v_shs = torch.empty((n, coeffs, 3), **f32) if (need[2] and had_shs) else None
            v_colors = torch.empty((n, 3), **f32) if (need[3] and had_colors) else None
            v_opac = torch.empty((n, 1), **f32) if need[4] else None
            v_scales = torch.empty((n, 3), **f32) if (need[5] and had_scales and had_rots) else None
            v_rots = torch.empty((n, 4), **f32) if (need[6] and had_scales and had_rots) else None
            v_cov3d = torch.empty((n, 6), **f32) if (need[7] and had_cov) else None
            _capi.check(lib.dsb_backward(
                C.byref(cam), n, means_3d.data_ptr(), _capi.ptr(scales), _capi.ptr(rotations), a + lay.records,
                cov3d_ptr, radii.data_ptr(), pair_arena.data_ptr() if ctx.num_pairs else None, a + lay.ranges,
                a + lay.final_t, a + lay.final_idx, v_image.data_ptr(), _capi.ptr(v_depth), a + lay.tile_marks,
                a + lay.grad_acc, _capi.ptr(v_means3d), _capi.ptr(v_means2d), _capi.ptr(v_shs), _capi.ptr(v_colors),
                _capi.ptr(v_opac), _capi.ptr(v_scales), _capi.ptr(v_rots), _capi.ptr(v_cov3d), 0, _capi.stream_ptr()))
        grads = [v_means3d, v_means2d, v_shs, v_colors, v_opac, v_scales, v_rots, v_cov3d]
        # gradients take the shape the caller's tensors had (opacities of shape [N], flattened shs, ...)
        grads = [g.view(shape) if g is not None and shape is not None and tuple(g.shape) != tuple(shape) else g
                 for g, shape in zip(grads, ctx.shapes)]
        return (*grads, None)


class GaussianRasterizer(torch.nn.Module):
    """Module wrapper with the reference's constructor and call signature (ds_splat/rasterizer.py:132-194)."""

    def __init__(self, raster_settings: GaussianRasterizationSettings):
        super().__init__()
        self._settings = raster_settings

    @property
    def raster_settings(self):
        return self._settings

    def forward(self, means_3d: Optional[torch.Tensor] = None, means_2d: Optional[torch.Tensor] = None,
                shs: Optional[torch.Tensor] = None, colors_precomp: Optional[torch.Tensor] = None,
                opacities: Optional[torch.Tensor] = None, scales: Optional[torch.Tensor] = None,
                rotations: Optional[torch.Tensor] = None, cov_3d_precomp: Optional[torch.Tensor] = None, *,
                means3D: Optional[torch.Tensor] = None, means2D: Optional[torch.Tensor] = None,
                cov3D_precomp: Optional[torch.Tensor] = None):
        means_3d = means_3d if means_3d is not None else means3D
        means_2d = means_2d if means_2d is not None else means2D
        cov_3d_precomp = cov_3d_precomp if cov_3d_precomp is not None else cov3D_precomp
        if means_3d is None or opacities is None:
            raise TypeError("means_3d and opacities are required")
        if (shs is None) == (colors_precomp is None) and shs is not None:
            raise ValueError("provide exactly one of shs and colors_precomp")
        if means_2d is None:
            means_2d = means_3d.new_zeros(means_3d.shape)
        empty = means_3d.new_empty(0)
        return DsRasterizerFunction.apply(
            means_3d, means_2d,
            shs if shs is not None else empty,
            colors_precomp if colors_precomp is not None else empty,
            opacities,
            scales if scales is not None else empty,
            rotations if rotations is not None else empty,
            cov_3d_precomp if cov_3d_precomp is not None else empty,
            self._settings)
