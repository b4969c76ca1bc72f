"""Parity against the REFERENCE's own CUDA kernels (oracle/_ref, built from the reference sources by
oracle/Makefile) on identical seeded inputs: radii, tile counts, sorted key/id lists and tile ranges
bit-exact; image within 1e-5 absolute; gradients within 1e-3 relative.  Skipped when the library was
not built (it needs the reference checkout at build time)."""
import numpy as np
import pytest

from conftest import scene_tensors, settings_for

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from ds_splat_b200 import GaussianRasterizer, _capi, scenes  # noqa: E402
from oracle import ref_cuda  # noqa: E402

needs_ref = pytest.mark.skipif(not ref_cuda.available(), reason="oracle/_ref/libref_splat.so not built")


def _rel_err(a, b):
    return float(np.abs(a - b).max()) / max(float(np.abs(b).max()), 1e-20)


@needs_ref
@pytest.mark.parametrize("name", ["tiny", "mid"])
def test_against_reference_cuda(name):
    sc = scenes.tiny() if name == "tiny" else scenes.headline(n=150_000, seed=11, W=800, H=608, focal=500.0)
    view = sc.views[0]
    v_image = sc.image_grad()
    ref = ref_cuda.run(view, sc.means, sc.shs, sc.opacities, sc.scales, sc.rotations, v_image=v_image)

    from conftest import capi_camera
    t = scene_tensors(sc)
    cam, keep = capi_camera(view)
    records, radii, tiles, cov3d, depth_keys = _capi.preprocess(cam, t["means"], t["shs"], t["opacities"], t["scales"], t["rotations"])
    offsets, k = _capi.plan_pairs(cam, tiles, depth_keys)
    pairs = _capi.emit_pairs(cam, k, records, tiles, depth_keys, offsets)
    tile_bits = max(1, int(np.ceil(np.log2(view.num_tiles))))
    sorted_pairs = _capi.sort_pairs(pairs, 32, 32 + tile_bits)
    ranges = _capi.identify_tile_ranges(sorted_pairs, view.H, view.W)
    keys_g, ids_g = _capi.export_reference_lists(sorted_pairs, records)

    # ---- bit-exact integer artefacts
    mism = int((radii.cpu().numpy() != ref["radii"]).sum())
    assert mism == 0, f"{mism} radii differ from the reference CUDA path"
    rec = records.cpu().numpy()
    np.testing.assert_array_equal(rec[:, 9].view(np.uint32), np.ascontiguousarray(ref["depth"]).view(np.uint32))
    assert k == ref["K"]
    np.testing.assert_array_equal(keys_g.cpu().numpy(), ref["keys_sorted"])
    np.testing.assert_array_equal(ids_g.cpu().numpy(), ref["ids_sorted"])
    np.testing.assert_array_equal(ranges.cpu().numpy(), ref["tile_indices"])

    # ---- operator level: image and gradients
    rast = GaussianRasterizer(settings_for(view))
    p = {k_: v.clone().requires_grad_(True) for k_, v in t.items()}
    means2d = torch.zeros_like(p["means"], requires_grad=True)
    image, radii_op = rast(p["means"], means2d, p["shs"], None, p["opacities"], p["scales"], p["rotations"], None)
    image.backward(torch.from_numpy(v_image).cuda())
    torch.cuda.synchronize()
    assert np.abs(image.detach().cpu().numpy() - ref["image"]).max() <= 1e-5
    np.testing.assert_array_equal(radii_op.cpu().numpy(), ref["radii"])
    grads = dict(v_mean=p["means"].grad, v_sh=p["shs"].grad, v_opacity=p["opacities"].grad.reshape(-1),
                 v_scale=p["scales"].grad, v_rot=p["rotations"].grad, v_xy=means2d.grad[:, :2])
    for name_, g in grads.items():
        e = _rel_err(g.cpu().numpy(), ref[name_])
        assert e < 1e-3, f"{name_}: relative error {e}"
