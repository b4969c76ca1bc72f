"""ctypes front end of ``oracle/_ref/libref_splat.so``: the reference's own CUDA kernels, driven by
``ref_harness.cu``.  TEST INFRASTRUCTURE ONLY (parity checker + "reference on the same GPU" timings).

``available()`` is False when the library was not built (it needs the reference checkout at build time,
see oracle/Makefile) -- callers skip the reference-CUDA comparisons then.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libref_splat.so")
_lib = None


class _Args(C.Structure):
    _fields_ = ([(n, C.c_int32) for n in ("N", "H", "W", "sh_degree", "max_sh_degree")]
                + [(n, C.c_float) for n in ("tanfovx", "tanfovy", "scale_modifier")]
                + [(n, C.c_void_p) for n in ("means", "shs", "opac", "scales", "rots", "view", "proj", "campos", "bg", "v_image")]
                + [("radii", C.c_void_p), ("gaussians", C.c_void_p), ("cov3d", C.c_void_p), ("keys_sorted", C.c_void_p),
                   ("ids_sorted", C.c_void_p), ("k_capacity", C.c_int64), ("tile_indices", C.c_void_p), ("image", C.c_void_p),
                   ("final_T", C.c_void_p), ("final_idx", C.c_void_p)]
                + [(n, C.c_void_p) for n in ("v_mean", "v_xy", "v_conic", "v_colors", "v_opacity", "v_sh", "v_scale", "v_rot", "v_cov3d")]
                + [("k_out", C.c_int64), ("iters", C.c_int32), ("warmup", C.c_int32), ("do_backward", C.c_int32),
                   ("ms", C.c_float * 8), ("ms_forward", C.c_float), ("ms_backward", C.c_float)])


STAGE_NAMES = ("preprocess", "keys", "sort", "ranges", "blend", "bwd_blend", "bwd_sh", "bwd_projection")


def reference_root():
    """Where the reference's sources lie: the directory DSB_REFERENCE_ROOT names, else a ``reference`` checkout beside
    this repository; None when neither exists (a machine that only carries the prebuilt library)."""
    candidates = [os.environ.get("DSB_REFERENCE_ROOT"),
                  os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")]
    for c in candidates:
        if c and os.path.isdir(os.path.join(c, "cpp")):
            return c
    return None


def build(root=None) -> bool:
    """Run ``make ref`` when the reference checkout is present; returns availability."""
    root = root or reference_root()
    if root and os.path.isdir(root):
        subprocess.run(["make", "-C", _HERE, "ref", f"REF={root}"], check=True)
    return available()


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        _lib = C.CDLL(LIB_PATH)
        _lib.ref_last_error.restype = C.c_char_p
        _lib.ref_run.restype = C.c_int
    return _lib


def run(view, means, shs, opacities, scales, rots, v_image=None, sh_degree=3, k_capacity=None, iters=1, warmup=0,
        outputs=True, bg=(0.0, 0.0, 0.0), scale_modifier=1.0):
    """Run the reference's forward (and backward when ``v_image`` is given) on the current CUDA device.

    ``view`` is any object with H, W, tanfovx, tanfovy, view, proj, campos (row-major matrices).
    Returns a dict with every intermediate the reference produces plus per-stage milliseconds."""
    f32 = lambda a: np.ascontiguousarray(a, np.float32)
    means, shs, opacities, scales, rots = f32(means), f32(shs), f32(opacities).reshape(-1), f32(scales), f32(rots)
    n, H, W = means.shape[0], view.H, view.W
    t = ((W + 15) // 16) * ((H + 15) // 16)
    a = _Args()
    a.N, a.H, a.W, a.sh_degree, a.max_sh_degree = n, H, W, sh_degree, 3
    a.tanfovx, a.tanfovy, a.scale_modifier = view.tanfovx, view.tanfovy, float(scale_modifier)
    vm, pm, cp, bgc = f32(view.view).reshape(16), f32(view.proj).reshape(16), f32(view.campos), f32(bg)
    keep = [means, shs, opacities, scales, rots, vm, pm, cp, bgc]
    for name, arr in zip(("means", "shs", "opac", "scales", "rots", "view", "proj", "campos", "bg"), keep):
        setattr(a, name, arr.ctypes.data)
    if v_image is not None:
        v_image = f32(v_image)
        a.v_image = v_image.ctypes.data
        a.do_backward = 1
    out = {}
    if outputs:
        if k_capacity is None:
            k_capacity = 64 * n
        out = dict(radii=np.empty(n, np.int32), gaussians=np.empty((n, 12), np.float32), cov3d=np.empty((n, 6), np.float32),
                   keys_sorted=np.empty(k_capacity, np.int64), ids_sorted=np.empty(k_capacity, np.int32),
                   tile_indices=np.empty(t + 1, np.int32), image=np.empty((H, W, 3), np.float32),
                   final_T=np.empty((H, W), np.float32), final_idx=np.empty((H, W), np.int32))
        a.k_capacity = k_capacity
        if v_image is not None:
            out.update(v_mean=np.empty((n, 3), np.float32), v_xy=np.empty((n, 2), np.float32), v_conic=np.empty((n, 3), np.float32),
                       v_colors=np.empty((n, 3), np.float32), v_opacity=np.empty(n, np.float32), v_sh=np.empty((n, 16, 3), np.float32),
                       v_scale=np.empty((n, 3), np.float32), v_rot=np.empty((n, 4), np.float32), v_cov3d=np.empty((n, 6), np.float32))
        for name, arr in out.items():
            setattr(a, name, arr.ctypes.data)
    a.iters, a.warmup = iters, warmup
    rc = lib().ref_run(C.byref(a))
    if rc != 0:
        raise RuntimeError(f"reference harness failed ({rc}): {lib().ref_last_error().decode()}")
    k = int(a.k_out)
    if outputs:
        if k > k_capacity:
            raise RuntimeError(f"k_capacity {k_capacity} < K {k}")
        out["keys_sorted"], out["ids_sorted"] = out["keys_sorted"][:k], out["ids_sorted"][:k]
        g = out["gaussians"]
        out["xy"], out["depth"], out["conic"], out["rgb"], out["alpha"] = g[:, 0:2], g[:, 2], g[:, 3:6], g[:, 6:9], g[:, 9]
    out["K"] = k
    out["ms"] = dict(zip(STAGE_NAMES, [float(x) for x in a.ms]))
    out["ms_forward"], out["ms_backward"] = float(a.ms_forward), float(a.ms_backward)
    return out
