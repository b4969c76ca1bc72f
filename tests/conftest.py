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


def capi_camera(view, device="cuda", sh_degree=3, max_sh_degree=3, transposed=True, drop_last=True, bg=(0.0, 0.0, 0.0)):
    """DsbCamera for a scenes.View; returns (cam, keepalive)."""
    import torch
    from ds_splat_b200 import _capi
    vm = torch.from_numpy(view.viewmatrix_t if transposed else np.ascontiguousarray(view.view)).to(device)
    pm = torch.from_numpy(view.projmatrix_t if transposed else np.ascontiguousarray(view.proj)).to(device)
    cp = torch.from_numpy(np.ascontiguousarray(view.campos)).to(device)
    bgt = torch.tensor(bg, dtype=torch.float32, device=device)
    return _capi.make_camera(view.H, view.W, view.tanfovx, view.tanfovy, vm, pm, cp, bgt, sh_degree, max_sh_degree, 1.0,
                             transposed=transposed, drop_last=drop_last)


def settings_for(view, device="cuda", sh_degree=3, **kw):
    import torch
    from ds_splat_b200 import GaussianRasterizationSettings
    return GaussianRasterizationSettings(
        image_height=view.H, image_width=view.W, tanfovx=view.tanfovx, tanfovy=view.tanfovy,
        bg=torch.zeros(3, device=device), scale_modifier=1.0,
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
