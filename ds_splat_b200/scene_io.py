"""Scene input for the rasterizer: trained-model checkpoints, the reference test's input container, and the
camera path of the reference's fly-through benchmark.

Two on-disk forms are read:

  * the ``point_cloud.ply`` checkpoints that 3-D Gaussian Splatting training code writes and that users of the
    reference render (README.md:43-58 of the reference lists the training repositories it plugs into): a
    binary little-endian PLY whose vertex element carries, per splat, ``x y z``, optional normals, the DC colour
    coefficients ``f_dc_0..2``, the higher SH coefficients ``f_rest_*`` stored CHANNEL-major (all coefficients
    of red, then green, then blue), ``opacity`` as a logit, ``scale_0..2`` as logarithms and the quaternion
    ``rot_0..3`` (w, x, y, z), not normalised;
  * the container the reference's own timing tests load (tests/rasterizer_test.cpp:147-167): a TorchScript
    module -- or a plain dict saved with ``torch.save`` -- with the attributes ``means_3d, means_2d, shs,
    opacities, scales, rotations, image_height, image_width, tanfovx, tanfovy, scale_modifier, viewmatrix,
    projmatrix, sh_degree, campos``.

Both loaders return host tensors in the layout ``GaussianRasterizer`` takes: ``shs`` as ``[N, 16, 3]``
(coefficient-major, channel-minor), activated opacity ``[N, 1]``, linear scales, unit quaternions.  The
writers exist so that the loaders can be tested on files the tests write themselves; no trained scene ships
with this repository.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import numpy as np

from . import scenes

CONTAINER_TENSORS = ("means_3d", "means_2d", "shs", "opacities", "scales", "rotations", "viewmatrix", "projmatrix", "campos")
CONTAINER_SCALARS = {"image_height": int, "image_width": int, "tanfovx": float, "tanfovy": float, "scale_modifier": float,
                     "sh_degree": int}

_PLY_TYPES = {"float": "<f4", "float32": "<f4", "double": "<f8", "float64": "<f8", "uchar": "u1", "uint8": "u1",
              "char": "i1", "int8": "i1", "short": "<i2", "int16": "<i2", "ushort": "<u2", "uint16": "<u2",
              "int": "<i4", "int32": "<i4", "uint": "<u4", "uint32": "<u4"}


def _read_ply_vertices(path: str) -> np.ndarray:
    """The vertex element of a binary little-endian PLY as a numpy structured array."""
    with open(path, "rb") as f:
        if f.readline().strip() != b"ply":
            raise ValueError(f"{path}: not a PLY file")
        fmt, count, props, in_vertex = None, None, [], False
        while True:
            line = f.readline()
            if not line:
                raise ValueError(f"{path}: header ends without end_header")
            tok = line.decode("ascii", "replace").split()
            if not tok:
                continue
            if tok[0] == "end_header":
                break
            if tok[0] == "format":
                fmt = tok[1]
            elif tok[0] == "element":
                if in_vertex:
                    in_vertex = False   # later elements (faces) follow the vertex block and are not read
                elif tok[1] == "vertex":
                    if props:
                        raise ValueError(f"{path}: two vertex elements")
                    in_vertex, count = True, int(tok[2])
                elif count is None:
                    raise ValueError(f"{path}: element '{tok[1]}' precedes the vertex element")
            elif tok[0] == "property" and in_vertex:
                if tok[1] == "list":
                    raise ValueError(f"{path}: list property in the vertex element")
                if tok[1] not in _PLY_TYPES:
                    raise ValueError(f"{path}: unknown property type '{tok[1]}'")
                props.append((tok[2], _PLY_TYPES[tok[1]]))
        if fmt != "binary_little_endian":
            raise ValueError(f"{path}: only binary_little_endian PLY is supported (found {fmt})")
        if count is None:
            raise ValueError(f"{path}: no vertex element")
        dtype = np.dtype(props)
        data = np.fromfile(f, dtype=dtype, count=count)
        if data.shape[0] != count:
            raise ValueError(f"{path}: file holds {data.shape[0]} of {count} vertices")
        return data


def load_ply(path: str, activated: bool = True) -> Dict[str, np.ndarray]:
    """Reads a 3-D Gaussian Splatting checkpoint.  Returns float32 arrays ``means [N,3]``, ``shs [N,C,3]`` (C = 1, 4,
    9 or 16), ``opacities [N,1]``, ``scales [N,3]``, ``rotations [N,4]`` and ``sh_degree``.  ``activated`` applies
    what the training code applies before it calls the rasterizer: sigmoid, exp and quaternion normalisation."""
    v = _read_ply_vertices(path)
    names = v.dtype.names
    need = ("x", "y", "z", "f_dc_0", "f_dc_1", "f_dc_2", "opacity", "scale_0", "scale_1", "scale_2",
            "rot_0", "rot_1", "rot_2", "rot_3")
    missing = [n for n in need if n not in names]
    if missing:
        raise ValueError(f"{path}: missing properties {missing}")
    col = lambda n: np.asarray(v[n], np.float32)
    n = v.shape[0]
    means = np.stack([col("x"), col("y"), col("z")], 1)
    rest_names = sorted((m for m in names if m.startswith("f_rest_")), key=lambda m: int(m.split("_")[-1]))
    if len(rest_names) % 3 != 0:
        raise ValueError(f"{path}: {len(rest_names)} f_rest_* properties do not split over three channels")
    per_channel = len(rest_names) // 3
    coeffs = per_channel + 1
    if coeffs not in (1, 4, 9, 16):
        raise ValueError(f"{path}: {coeffs} SH coefficients per channel is not a full degree (1, 4, 9 or 16)")
    shs = np.empty((n, coeffs, 3), np.float32)
    shs[:, 0, :] = np.stack([col("f_dc_0"), col("f_dc_1"), col("f_dc_2")], 1)
    if per_channel:
        rest = np.stack([col(m) for m in rest_names], 1).reshape(n, 3, per_channel)   # channel-major on disk
        shs[:, 1:, :] = rest.transpose(0, 2, 1)
    opac = col("opacity").reshape(n, 1)
    scales_ = np.stack([col("scale_0"), col("scale_1"), col("scale_2")], 1)
    rots = np.stack([col("rot_0"), col("rot_1"), col("rot_2"), col("rot_3")], 1)
    if activated:
        opac = (1.0 / (1.0 + np.exp(-opac.astype(np.float64)))).astype(np.float32)
        scales_ = np.exp(scales_)
        rots = rots / np.maximum(np.linalg.norm(rots, axis=1, keepdims=True), 1e-12)
    return dict(means=np.ascontiguousarray(means), shs=shs, opacities=opac, scales=np.ascontiguousarray(scales_, np.float32),
                rotations=np.ascontiguousarray(rots, np.float32), sh_degree=int(round(math.sqrt(coeffs))) - 1)


def save_ply(path: str, means, shs, opacities, scales, rotations, activated: bool = True) -> None:
    """Writes the same checkpoint form (with zero normals, as the training code does).  ``activated`` says that the
    arrays are what the rasterizer takes (probabilities, linear scales); they are stored as logits and logarithms."""
    means, shs = np.asarray(means, np.float32), np.asarray(shs, np.float32)
    n, coeffs = means.shape[0], shs.shape[1]
    opac = np.asarray(opacities, np.float64).reshape(n)
    scales_ = np.asarray(scales, np.float64)
    if activated:
        opac = np.log(opac / (1.0 - opac))
        scales_ = np.log(scales_)
    names = (["x", "y", "z", "nx", "ny", "nz", "f_dc_0", "f_dc_1", "f_dc_2"] + [f"f_rest_{i}" for i in range(3 * (coeffs - 1))]
             + ["opacity", "scale_0", "scale_1", "scale_2", "rot_0", "rot_1", "rot_2", "rot_3"])
    rest = shs[:, 1:, :].transpose(0, 2, 1).reshape(n, 3 * (coeffs - 1))   # channel-major
    table = np.concatenate([means, np.zeros((n, 3), np.float32), shs[:, 0, :], rest, opac.reshape(n, 1).astype(np.float32),
                            scales_.astype(np.float32), np.asarray(rotations, np.float32)], 1).astype("<f4")
    header = "ply\nformat binary_little_endian 1.0\nelement vertex %d\n" % n
    header += "".join(f"property float {m}\n" for m in names) + "end_header\n"
    with open(path, "wb") as f:
        f.write(header.encode("ascii"))
        f.write(np.ascontiguousarray(table).tobytes())


def load_container(path: str, map_location="cpu") -> Dict[str, object]:
    """Reads the input container of the reference's timing tests (tests/rasterizer_test.cpp:147-167): a TorchScript
    module whose attributes are the rasterizer's inputs and settings, or a dict with the same keys saved with
    ``torch.save``.  Returns a dict of tensors and Python scalars under those names; ``viewmatrix`` and
    ``projmatrix`` are left in the transposed form the container holds (the form ``GaussianRasterizationSettings``
    takes; the reference's test transposes them itself, :158-159)."""
    import torch
    try:
        module = torch.jit.load(path, map_location=map_location)
        get = lambda name: getattr(module, name)
    except RuntimeError:
        blob = torch.load(path, map_location=map_location, weights_only=True)
        if not isinstance(blob, dict):
            raise ValueError(f"{path}: neither a TorchScript module nor a dict")
        get = blob.__getitem__
    out = {}
    for name in CONTAINER_TENSORS:
        try:
            value = get(name)
        except (AttributeError, KeyError):
            raise ValueError(f"{path}: attribute '{name}' is missing") from None
        if not isinstance(value, torch.Tensor):
            raise ValueError(f"{path}: attribute '{name}' is not a tensor")
        out[name] = value
    for name, kind in CONTAINER_SCALARS.items():
        try:
            out[name] = kind(get(name))
        except (AttributeError, KeyError):
            raise ValueError(f"{path}: attribute '{name}' is missing") from None
    return out


def save_container(path: str, data: Dict[str, object]) -> None:
    """Writes such a container as a TorchScript module (tensors as buffers, settings as typed attributes)."""
    import torch

    class Container(torch.nn.Module):
        def __init__(self, d):
            super().__init__()
            for name in CONTAINER_TENSORS:
                self.register_buffer(name, torch.as_tensor(d[name]).detach().clone())
            self.image_height: int = int(d["image_height"])
            self.image_width: int = int(d["image_width"])
            self.tanfovx: float = float(d["tanfovx"])
            self.tanfovy: float = float(d["tanfovy"])
            self.scale_modifier: float = float(d["scale_modifier"])
            self.sh_degree: int = int(d["sh_degree"])

        def forward(self):
            return self.means_3d

    torch.jit.save(torch.jit.script(Container(data)), path)


def settings_from_container(data: Dict[str, object], device):
    """``GaussianRasterizationSettings`` and the five parameter tensors of a loaded container, on ``device``."""
    import torch
    from .rasterizer import GaussianRasterizationSettings
    dev = torch.device(device)
    t = lambda name: data[name].to(device=dev, dtype=torch.float32).contiguous()
    settings = GaussianRasterizationSettings(
        image_height=data["image_height"], image_width=data["image_width"], tanfovx=data["tanfovx"], tanfovy=data["tanfovy"],
        bg=torch.zeros(3, device=dev), scale_modifier=data["scale_modifier"], viewmatrix=t("viewmatrix"),
        projmatrix=t("projmatrix"), sh_degree=data["sh_degree"], max_sh_degree=3, campos=t("campos"))
    params = dict(means_3d=t("means_3d"), shs=t("shs"), opacities=t("opacities"), scales=t("scales"), rotations=t("rotations"))
    return settings, params


def zoom_out_path(frames: int = 120, start_distance: float = 3.0, end_distance: float = 12.0, W: int = 1920, H: int = 1080,
                  focal: float = 1100.0, target=(0.0, 0.0, 0.0), sweep_degrees: float = 30.0) -> list:
    """Cameras of the reference's benchmark protocol (README.md:199-204: "120 frames as fly through a scene with zooming
    out to capture all Gaussians"): the camera backs away from ``target`` along a gentle arc, from ``start_distance`` to
    ``end_distance``, so that the number of splats in view -- and with it the frame time -- grows along the path."""
    views = []
    for i in range(frames):
        s = i / max(frames - 1, 1)
        dist = start_distance * (end_distance / start_distance) ** s     # constant zoom rate
        yaw = math.radians(sweep_degrees) * (s - 0.5)
        eye = (target[0] + dist * math.sin(yaw), target[1] - 0.15 * dist, target[2] - dist * math.cos(yaw))
        views.append(scenes.make_view(eye, target, W, H, focal))
    return views
