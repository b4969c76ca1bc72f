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
    if settings.max_sh_degree != 3 and settings.max_sh_degree not in (0, 1, 2):
        raise ValueError("max_sh_degree must be in 0..3")
    return _capi.make_camera(settings.image_height, settings.image_width, settings.tanfovx, settings.tanfovy, view,
                             proj, campos, bg, settings.sh_degree, settings.max_sh_degree, settings.scale_modifier,
                             transposed=True, drop_last=settings.strict_reference, tight_tiles=settings.tight_tiles)


class DsRasterizerFunction(torch.autograd.Function):
    """Counterpart of the reference's autograd Function (ds_splat/rasterizer.py:7-112): eight tensor inputs
    plus the settings; returns (image, radii) -- (image, radii, depth) with ``return_depth`` -- and backward returns
    one gradient per tensor input."""

    @staticmethod
    def forward(ctx, means_3d, means_2d, shs, colors_precomp, opacities, scales, rotations, cov_3d_precomp,
                raster_settings):
        lib = _capi.lib()
        if not isinstance(means_3d, torch.Tensor) or not means_3d.is_cuda:
            raise RuntimeError("means_3d must be a CUDA tensor")
        dev = means_3d.device
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
            f32 = dict(dtype=torch.float32, device=dev)
            records = torch.empty((n, _capi.RECORD_FLOATS), **f32)
            radii = torch.empty(n, dtype=torch.int32, device=dev)
            tiles = torch.empty(n, dtype=torch.int32, device=dev)
            cov3d = cov_3d_precomp if cov_3d_precomp is not None else torch.empty((n, 6), **f32)
            depth_keys = torch.empty((2, n), dtype=torch.int64, device=dev)
            offsets = torch.empty(n, dtype=torch.int32, device=dev)
            tile_marks = torch.empty(int(lib.dsb_tile_marks_bytes(h, w)), dtype=torch.uint8, device=dev)
            plan_bytes = int(lib.dsb_plan_workspace_bytes(n))
            plan_ws = torch.empty(plan_bytes, dtype=torch.uint8, device=dev)
            k = C.c_int64(0)
            _capi.check(lib.dsb_forward_plan(
                C.byref(cam), n, _capi.ptr(means_3d), _capi.ptr(shs), _capi.ptr(colors_precomp), _capi.ptr(opacities),
                _capi.ptr(scales), _capi.ptr(rotations), _capi.ptr(cov_3d_precomp), records.data_ptr(), radii.data_ptr(),
                tiles.data_ptr(), cov3d.data_ptr(), depth_keys[0].data_ptr(), depth_keys[1].data_ptr(),
                offsets.data_ptr(), tile_marks.data_ptr(), plan_ws.data_ptr(), plan_bytes, C.byref(k), stream))
            k = int(k.value)

            pairs = torch.empty((2, max(k, 1)), dtype=torch.int64, device=dev)
            sort_bytes = int(lib.dsb_sort_workspace_bytes(k))
            sort_ws = torch.empty(sort_bytes, dtype=torch.uint8, device=dev)
            ranges = torch.empty(_capi.num_tiles(h, w) + 1, dtype=torch.int32, device=dev)
            image = torch.empty((h, w, 3), **f32)
            final_t = torch.empty((h, w), **f32)
            final_idx = torch.empty((h, w), dtype=torch.int32, device=dev)
            depth = torch.empty((h, w), **f32) if raster_settings.return_depth else None
            _capi.check(lib.dsb_forward_render(
                C.byref(cam), n, k, records.data_ptr(), tiles.data_ptr(), depth_keys[0].data_ptr(), offsets.data_ptr(),
                pairs[0].data_ptr(), pairs[1].data_ptr(), tile_marks.data_ptr(), sort_ws.data_ptr(), sort_bytes,
                ranges.data_ptr(),
                image.data_ptr(), final_t.data_ptr(), final_idx.data_ptr(), _capi.ptr(depth), None, stream))
            sorted_pairs = pairs[0][:k]

        ctx.raster_settings = raster_settings
        ctx.num_pairs = k
        ctx.had = (shs is not None, colors_precomp is not None, scales is not None, rotations is not None,
                   cov_3d_precomp is not None)
        ctx.save_for_backward(means_3d, scales if scales is not None else means_3d.new_empty(0),
                              rotations if rotations is not None else means_3d.new_empty(0), records, cov3d, radii,
                              sorted_pairs, ranges, final_t, final_idx, tile_marks)
        ctx.mark_non_differentiable(radii)
        if raster_settings.channels_first:
            image = image.permute(2, 0, 1)
        if raster_settings.return_depth:
            return image, radii, depth
        return image, radii

    @staticmethod
    def backward(ctx, rendered_img_grad, _radii_grad, depth_grad=None):
        lib = _capi.lib()
        (means_3d, scales, rotations, records, cov3d, radii, sorted_pairs, ranges, final_t, final_idx,
         tile_order) = ctx.saved_tensors
        settings = ctx.raster_settings
        had_shs, had_colors, had_scales, had_rots, had_cov = ctx.had
        dev = means_3d.device
        n = means_3d.shape[0]
        if rendered_img_grad is None:  # only the depth map took part in the loss
            rendered_img_grad = final_t.new_zeros((settings.image_height, settings.image_width, 3))
        elif settings.channels_first:
            rendered_img_grad = rendered_img_grad.permute(1, 2, 0)
        v_image = rendered_img_grad.to(dtype=torch.float32).contiguous()
        v_depth = depth_grad.to(dtype=torch.float32).contiguous() if depth_grad is not None else None
        need = ctx.needs_input_grad
        coeffs = (settings.max_sh_degree + 1) ** 2

        with torch.cuda.device(dev):
            cam, keep = _camera_for(settings, dev)
            f32 = dict(dtype=torch.float32, device=dev)
            grad_acc = torch.empty((n, _capi.GRAD_FLOATS), **f32)
            v_means3d = torch.empty((n, 3), **f32) if need[0] else None
            v_means2d = torch.empty((n, 3), **f32) if need[1] else None
            v_shs = torch.empty((n, coeffs, 3), **f32) if (need[2] and had_shs) else None
            v_colors = torch.empty((n, 3), **f32) if (need[3] and had_colors) else None
            v_opac = torch.empty((n, 1), **f32) if need[4] else None
            v_scales = torch.empty((n, 3), **f32) if (need[5] and had_scales and had_rots) else None
            v_rots = torch.empty((n, 4), **f32) if (need[6] and had_scales and had_rots) else None
            v_cov3d = torch.empty((n, 6), **f32) if (need[7] and had_cov) else None
            _capi.check(lib.dsb_backward(
                C.byref(cam), n, means_3d.data_ptr(), _capi.ptr(scales), _capi.ptr(rotations), records.data_ptr(),
                cov3d.data_ptr(), radii.data_ptr(), _capi.ptr(sorted_pairs), ranges.data_ptr(), final_t.data_ptr(),
                final_idx.data_ptr(), v_image.data_ptr(), _capi.ptr(v_depth), tile_order.data_ptr(), grad_acc.data_ptr(),
                _capi.ptr(v_means3d),
                _capi.ptr(v_means2d),
                _capi.ptr(v_shs), _capi.ptr(v_colors), _capi.ptr(v_opac), _capi.ptr(v_scales), _capi.ptr(v_rots),
                _capi.ptr(v_cov3d), 0, _capi.stream_ptr()))
        return v_means3d, v_means2d, v_shs, v_colors, v_opac, v_scales, v_rots, v_cov3d, None


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
