"""ctypes front end of the CPU oracle (``gs_oracle.cpp``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()`` as the checker and by
``bench.py`` for its CPU-baseline legs.  The product package never imports this module.

All functions take and return numpy arrays on the host.  ``Camera`` mirrors the fields of the
reference's ``TorchRasterizationSettings`` (cpp/ds_cuda_rasterizer/rasterizer_torch.hpp:7-22) with the
matrices already in the row-major form the kernels read (ds_splat/rasterizer.py:147-148).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libgs_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile gs_oracle.cpp with g++ -O3 -fopenmp into oracle/_build/ (no-op when up to date)."""
    src = os.path.join(_HERE, "gs_oracle.cpp")
    if (not force and os.path.exists(_LIB_PATH)
            and os.path.getmtime(_LIB_PATH) >= os.path.getmtime(src)):
        return _LIB_PATH
    os.makedirs(os.path.dirname(_LIB_PATH), exist_ok=True)
    cmd = ["g++", "-O3", "-march=native", "-fopenmp", "-shared", "-fPIC", src, "-o", _LIB_PATH]
    subprocess.run(cmd, check=True)
    return _LIB_PATH


class _Cam(C.Structure):
    _fields_ = [("view", C.c_float * 16), ("proj", C.c_float * 16), ("campos", C.c_float * 3),
                ("tanfovx", C.c_float), ("tanfovy", C.c_float), ("scale_modifier", C.c_float),
                ("bg", C.c_float * 3), ("H", C.c_int), ("W", C.c_int), ("sh_degree", C.c_int),
                ("max_sh_degree", C.c_int)]


@dataclass
class Camera:
    """Host-side camera/settings record; ``view`` and ``proj`` are row-major 4x4 (world->camera, P*V)."""
    view: np.ndarray
    proj: np.ndarray
    campos: np.ndarray
    tanfovx: float
    tanfovy: float
    H: int
    W: int
    sh_degree: int = 3
    max_sh_degree: int = 3
    scale_modifier: float = 1.0
    bg: tuple = (0.0, 0.0, 0.0)

    def c(self) -> _Cam:
        s = _Cam()
        s.view[:] = np.asarray(self.view, np.float32).reshape(16).tolist()
        s.proj[:] = np.asarray(self.proj, np.float32).reshape(16).tolist()
        s.campos[:] = np.asarray(self.campos, np.float32).reshape(3).tolist()
        s.tanfovx, s.tanfovy, s.scale_modifier = self.tanfovx, self.tanfovy, self.scale_modifier
        s.bg[:] = list(self.bg)
        s.H, s.W, s.sh_degree, s.max_sh_degree = self.H, self.W, self.sh_degree, self.max_sh_degree
        return s

    @property
    def num_tiles(self) -> int:
        return ((self.W + 15) // 16) * ((self.H + 15) // 16)


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.orc_count_pairs.restype = C.c_int64
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def num_threads() -> int:
    return int(lib().orc_num_threads())


def use_all_host_threads() -> int:
    """Run every following stage on all hardware threads of the host, whatever OMP_NUM_THREADS says (launchers such
    as torchrun export OMP_NUM_THREADS=1 to their workers); returns the thread count now in use."""
    lib().orc_set_threads(C.c_int(0))
    return num_threads()


def set_threads(n: int) -> int:
    lib().orc_set_threads(C.c_int(int(n)))
    return num_threads()


def _p(a, dtype=None):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    if dtype is not None:
        assert a.dtype == dtype, (a.dtype, dtype)
    return a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def preprocess(cam: Camera, means, shs, opacities, scales, rots, colors_precomp=None, cov3d_precomp=None):
    """Stage (a): returns dict(xy, depth, conic, rgb, radii, tiles, rect, cov3d)."""
    means = _f32(means)
    n = means.shape[0]
    shs, opacities, scales, rots = _f32(shs), _f32(opacities), _f32(scales), _f32(rots)
    colors_precomp, cov3d_precomp = _f32(colors_precomp), _f32(cov3d_precomp)
    out = dict(xy=np.empty((n, 2), np.float32), depth=np.empty(n, np.float32), conic=np.empty((n, 3), np.float32),
               rgb=np.empty((n, 3), np.float32), radii=np.empty(n, np.int32), tiles=np.empty(n, np.int32),
               rect=np.empty((n, 4), np.int32), cov3d=np.empty((n, 6), np.float32))
    cs = cam.c()
    lib().orc_preprocess(C.byref(cs), C.c_int(n), _p(means), _p(shs), _p(colors_precomp), _p(opacities), _p(scales),
                         _p(rots), _p(cov3d_precomp), _p(out["xy"]), _p(out["depth"]), _p(out["conic"]),
                         _p(out["rgb"]), _p(out["radii"]), _p(out["tiles"]), _p(out["rect"]), _p(out["cov3d"]))
    return out


def count_pairs(tiles, drop_last=True) -> int:
    tiles = np.ascontiguousarray(tiles, np.int32)
    return int(lib().orc_count_pairs(C.c_int(tiles.shape[0]), _p(tiles), C.c_int(int(drop_last))))


def duplicate_keys(cam: Camera, pre, drop_last=True):
    """Stage (b): unsorted (keys int64, ids int32) in the reference's emission order."""
    n = pre["radii"].shape[0]
    k = count_pairs(pre["tiles"], drop_last)
    keys, ids = np.empty(k, np.int64), np.empty(k, np.int32)
    cs = cam.c()
    lib().orc_duplicate_keys(C.byref(cs), C.c_int(n), _p(pre["xy"]), _p(pre["depth"]), _p(pre["radii"]),
                             _p(pre["tiles"]), C.c_int(int(drop_last)), _p(keys), _p(ids))
    return keys, ids


def sort_pairs(keys, ids):
    """Stage (c): stable ascending sort by signed 64-bit key; returns new arrays."""
    keys, ids = np.array(keys, np.int64, copy=True), np.array(ids, np.int32, copy=True)
    lib().orc_sort_pairs(C.c_int64(keys.shape[0]), _p(keys), _p(ids))
    return keys, ids


def tile_ranges(keys, H, W):
    """Stage (d): int32[T+1]; tile t owns sorted positions [r[t], r[t+1])."""
    keys = np.ascontiguousarray(keys, np.int64)
    t = ((W + 15) // 16) * ((H + 15) // 16)
    out = np.empty(t + 1, np.int32)
    lib().orc_tile_ranges(C.c_int64(keys.shape[0]), _p(keys), C.c_int(H), C.c_int(W), _p(out))
    return out


def blend_forward(cam: Camera, ids, ranges, xy, conic, rgb, opac, z=None):
    """Stage (e): returns image[H,W,3], final_T[H,W], final_idx[H,W], pairs evaluated -- and, when the per-splat
    view-space depths ``z`` are given, the blended depth map[H,W] as a fifth value."""
    ids, ranges = np.ascontiguousarray(ids, np.int32), np.ascontiguousarray(ranges, np.int32)
    xy, conic, rgb, opac = _f32(xy), _f32(conic), _f32(rgb), _f32(opac).reshape(-1)
    image = np.zeros((cam.H, cam.W, 3), np.float32)
    ft = np.ones((cam.H, cam.W), np.float32)
    fi = np.zeros((cam.H, cam.W), np.int32)
    pairs = np.zeros(2, np.int64)
    cs = cam.c()
    depth = None
    if z is not None:
        z = _f32(z).reshape(-1)
        depth = np.zeros((cam.H, cam.W), np.float32)
    lib().orc_blend_forward(C.byref(cs), _p(ids), _p(ranges), _p(xy), _p(conic), _p(rgb), _p(opac), _p(image),
                            _p(ft), _p(fi), _p(pairs), _p(z) if z is not None else None,
                            _p(depth) if depth is not None else None)
    if z is not None:
        return image, ft, fi, int(pairs[0]), depth
    return image, ft, fi, int(pairs[0])


def blend_backward(cam: Camera, n, ids, ranges, xy, conic, rgb, opac, final_T, final_idx, v_image, z=None, v_depth=None):
    """Stage (f1): returns v_xy[N,2], v_conic[N,3], v_rgb[N,3], v_opacity[N], pairs visited -- and, when ``z`` and the
    depth map's gradient ``v_depth`` are given, v_z[N] as a sixth value."""
    ids, ranges = np.ascontiguousarray(ids, np.int32), np.ascontiguousarray(ranges, np.int32)
    xy, conic, rgb, opac = _f32(xy), _f32(conic), _f32(rgb), _f32(opac).reshape(-1)
    final_T, v_image = _f32(final_T), _f32(v_image)
    final_idx = np.ascontiguousarray(final_idx, np.int32)
    v_xy, v_conic = np.empty((n, 2), np.float32), np.empty((n, 3), np.float32)
    v_rgb, v_op = np.empty((n, 3), np.float32), np.empty(n, np.float32)
    pairs = np.zeros(2, np.int64)
    with_depth = z is not None and v_depth is not None
    if with_depth:
        z, v_depth, v_z = _f32(z).reshape(-1), _f32(v_depth), np.zeros(n, np.float32)
        depth_args = (_p(z), _p(v_depth), _p(v_z))
    else:
        depth_args = (None, None, None)
    cs = cam.c()
    lib().orc_blend_backward(C.byref(cs), C.c_int(n), _p(ids), _p(ranges), _p(xy), _p(conic), _p(rgb), _p(opac),
                             _p(final_T), _p(final_idx), _p(v_image), _p(v_xy), _p(v_conic), _p(v_rgb), _p(v_op),
                             _p(pairs), *depth_args)
    if with_depth:
        return v_xy, v_conic, v_rgb, v_op, int(pairs[0]), v_z
    return v_xy, v_conic, v_rgb, v_op, int(pairs[0])


def sh_backward(cam: Camera, means, v_rgb, num_bases=16):
    means, v_rgb = _f32(means), _f32(v_rgb)
    n = means.shape[0]
    out = np.empty((n, num_bases, 3), np.float32)
    cs = cam.c()
    lib().orc_sh_backward(C.byref(cs), C.c_int(n), C.c_int(num_bases), _p(means), _p(v_rgb), _p(out))
    return out


def project_backward(cam: Camera, means, scales, rots, conic, cov3d, radii, v_xy, v_conic, v_z=None):
    means, scales, rots = _f32(means), _f32(scales), _f32(rots)
    conic, cov3d, v_xy, v_conic = _f32(conic), _f32(cov3d), _f32(v_xy), _f32(v_conic)
    radii = np.ascontiguousarray(radii, np.int32)
    n = means.shape[0]
    v_mean, v_scale = np.empty((n, 3), np.float32), np.empty((n, 3), np.float32)
    v_rot, v_cov3d = np.empty((n, 4), np.float32), np.empty((n, 6), np.float32)
    v_z = None if v_z is None else _f32(v_z).reshape(-1)
    cs = cam.c()
    lib().orc_project_backward(C.byref(cs), C.c_int(n), _p(means), _p(scales), _p(rots), _p(conic), _p(cov3d),
                               _p(radii), _p(v_xy), _p(v_conic), _p(v_mean), _p(v_scale), _p(v_rot), _p(v_cov3d),
                               _p(v_z))
    return v_mean, v_scale, v_rot, v_cov3d


def forward(cam: Camera, means, shs, opacities, scales, rots, drop_last=True, with_depth=False):
    """Whole forward the way cpp/rasterizer_torch.cu:170-208 chains the stages; returns a dict of every
    intermediate (pre, keys, ids, ranges, image, final_T, final_idx, K, pairs_fwd)."""
    pre = preprocess(cam, means, shs, opacities, scales, rots)
    keys, ids = duplicate_keys(cam, pre, drop_last)
    keys, ids = sort_pairs(keys, ids)
    ranges = tile_ranges(keys, cam.H, cam.W)
    opac = _f32(opacities).reshape(-1)
    depth = None
    if with_depth:
        image, ft, fi, pairs, depth = blend_forward(cam, ids, ranges, pre["xy"], pre["conic"], pre["rgb"], opac, pre["depth"])
    else:
        image, ft, fi, pairs = blend_forward(cam, ids, ranges, pre["xy"], pre["conic"], pre["rgb"], opac)
    return dict(pre=pre, keys=keys, ids=ids, ranges=ranges, image=image, final_T=ft, final_idx=fi,
                K=int(keys.shape[0]), pairs_fwd=pairs, depth=depth)


def backward(cam: Camera, fwd, means, shs, opacities, scales, rots, v_image, v_depth=None):
    """Whole backward (cpp/rasterizer_torch.cu:263-316); returns the reference's 8 gradients by name.  ``v_depth``
    (gradient of the optional depth map) is routed through the v_depth slot of the projection backward."""
    pre = fwd["pre"]
    n = _f32(means).shape[0]
    opac = _f32(opacities).reshape(-1)
    v_z = None
    if v_depth is not None:
        v_xy, v_conic, v_rgb, v_op, pairs, v_z = blend_backward(cam, n, fwd["ids"], fwd["ranges"], pre["xy"], pre["conic"],
                                                                pre["rgb"], opac, fwd["final_T"], fwd["final_idx"], v_image,
                                                                pre["depth"], v_depth)
    else:
        v_xy, v_conic, v_rgb, v_op, pairs = blend_backward(cam, n, fwd["ids"], fwd["ranges"], pre["xy"], pre["conic"],
                                                           pre["rgb"], opac, fwd["final_T"], fwd["final_idx"], v_image)
    num_bases = _f32(shs).shape[-2]
    v_sh = sh_backward(cam, means, v_rgb, num_bases)
    v_mean, v_scale, v_rot, v_cov3d = project_backward(cam, means, scales, rots, pre["conic"], pre["cov3d"],
                                                       pre["radii"], v_xy, v_conic, v_z)
    v_means2d = np.concatenate([v_xy, np.zeros((n, 1), np.float32)], axis=1)
    return dict(v_means3d=v_mean, v_means2d=v_means2d, v_shs=v_sh, v_colors=v_rgb, v_opacities=v_op.reshape(n, 1),
                v_scales=v_scale, v_rotations=v_rot, v_cov3d=v_cov3d, v_conic=v_conic, pairs_bwd=pairs)


def adam_step(param, grad, exp_avg, exp_avg_sq, lr, beta1=0.9, beta2=0.999, eps=1e-8, step=1, grad_scale=1.0):
    """Checker for the optimizer step that follows the operator in a training loop.  No reference file to cite: the
    reference's users call torch.optim.Adam; this restates that update (Kingma & Ba, algorithm 1, in the form
    torch applies it without weight decay or amsgrad) in float32 numpy, returning new (param, exp_avg, exp_avg_sq).
    tests/test_oracle.py pins it against torch.optim.Adam itself."""
    f = np.float32
    g = (_f32(grad) * f(grad_scale)).astype(np.float32)
    m = (f(beta1) * _f32(exp_avg) + f(1.0 - beta1) * g).astype(np.float32)
    v = (f(beta2) * _f32(exp_avg_sq) + f(1.0 - beta2) * g * g).astype(np.float32)
    bias1, bias2 = 1.0 - beta1 ** step, 1.0 - beta2 ** step
    denom = (np.sqrt(v) / f(np.sqrt(bias2)) + f(eps)).astype(np.float32)
    p = (_f32(param) - f(lr / bias1) * (m / denom)).astype(np.float32)
    return p, m, v
