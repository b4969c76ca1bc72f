"""Shared fixtures: the `gpu` marker, scene -> tensors / oracle-camera helpers."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def oracle_camera(view, sh_degree=3, max_sh_degree=3, bg=(0.0, 0.0, 0.0)):
    from oracle import oracle as O
    return O.Camera(view=view.view, proj=view.proj, campos=view.campos, tanfovx=view.tanfovx, tanfovy=view.tanfovy,
                    H=view.H, W=view.W, sh_degree=sh_degree, max_sh_degree=max_sh_degree, bg=bg)


def scene_tensors(scene, device="cuda"):
    import torch
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
    return dict(means=t(scene.means), shs=t(scene.shs), opacities=t(scene.opacities), scales=t(scene.scales),
                rotations=t(scene.rotations))


def capi_camera(view, device="cuda", sh_degree=3, max_sh_degree=3, transposed=True, drop_last=True, bg=(0.0, 0.0, 0.0),
                row_binning=False):
    """DsbCamera for a scenes.View; returns (cam, keepalive)."""
    import torch
    from ds_splat_b200 import _capi
    vm = torch.from_numpy(view.viewmatrix_t if transposed else np.ascontiguousarray(view.view)).to(device)
    pm = torch.from_numpy(view.projmatrix_t if transposed else np.ascontiguousarray(view.proj)).to(device)
    cp = torch.from_numpy(np.ascontiguousarray(view.campos)).to(device)
    bgt = torch.tensor(bg, dtype=torch.float32, device=device)
    return _capi.make_camera(view.H, view.W, view.tanfovx, view.tanfovy, vm, pm, cp, bgt, sh_degree, max_sh_degree, 1.0,
                             transposed=transposed, drop_last=drop_last, row_binning=row_binning)


def settings_for(view, device="cuda", sh_degree=3, bg=(0.0, 0.0, 0.0), scale_modifier=1.0, **kw):
    import torch
    from ds_splat_b200 import GaussianRasterizationSettings
    return GaussianRasterizationSettings(
        image_height=view.H, image_width=view.W, tanfovx=view.tanfovx, tanfovy=view.tanfovy,
        bg=torch.tensor(bg, dtype=torch.float32, device=device), scale_modifier=scale_modifier,
        viewmatrix=torch.from_numpy(view.viewmatrix_t).to(device), projmatrix=torch.from_numpy(view.projmatrix_t).to(device),
        sh_degree=sh_degree, max_sh_degree=3, campos=torch.from_numpy(np.ascontiguousarray(view.campos)).to(device),
        prefiltered=False, debug=False, **kw)


def unpack_records(records_np):
    """Split the packed [N,12] records into the oracle's separate arrays."""
    r = records_np
    rect_x, rect_y = r[:, 10].view(np.uint32), r[:, 11].view(np.uint32)
    rect = np.stack([rect_x & 0xFFFF, rect_x >> 16, rect_y & 0xFFFF, rect_y >> 16], 1).astype(np.int32)
    return dict(xy=np.ascontiguousarray(r[:, 0:2]), conic=np.ascontiguousarray(np.stack([r[:, 2], r[:, 3], r[:, 4]], 1)),
                opac=np.ascontiguousarray(r[:, 5]), rgb=np.ascontiguousarray(np.stack([r[:, 6], r[:, 7], r[:, 8]], 1)),
                depth=np.ascontiguousarray(r[:, 9]), rect=rect)


def gradient_gate(got, want, name, rel=1e-3, max_bad_fraction=1e-4):
    """Per-element gradient comparison: an element fails when |got - want| > rel * |want| + rel * median|want| (the
    median over the non-zero entries keeps entries far below the tensor's typical size from being judged on rounding
    noise of the sums they came from; atomic accumulation order is not deterministic).  At most ``max_bad_fraction`` of
    the elements may fail.  Prints the distribution of the per-element error so that a run's log shows how close the
    gate was; returns the failing fraction."""
    got, want = np.asarray(got, np.float64).ravel(), np.asarray(want, np.float64).ravel()
    assert got.shape == want.shape, f"{name}: shapes differ"
    assert np.isfinite(got).all(), f"{name}: non-finite gradient"
    nz = np.abs(want) > 0
    typical = float(np.median(np.abs(want[nz]))) if nz.any() else 0.0
    err = np.abs(got - want)
    bound = rel * np.abs(want) + rel * typical
    bad = err > bound
    scaled = err / np.maximum(np.abs(want) + typical, 1e-300)
    q = np.quantile(scaled, [0.5, 0.99, 0.9999, 1.0]) if scaled.size else np.zeros(4)
    frac = float(bad.mean()) if bad.size else 0.0
    print(f"[gradient gate] {name}: {bad.sum()} of {bad.size} elements outside {rel:g} relative (fraction {frac:.2e}); "
          f"error / (|want| + median): median {q[0]:.2e}, p99 {q[1]:.2e}, p99.99 {q[2]:.2e}, max {q[3]:.2e}; "
          f"typical |want| {typical:.3e}")
    assert frac <= max_bad_fraction, f"{name}: {bad.sum()} of {bad.size} elements differ by more than {rel:g} relative"
    return frac
