"""Parity against the REFERENCE's own CUDA kernels (oracle/_ref, built from the reference sources by
oracle/Makefile) on identical seeded inputs: radii, tile counts, sorted key/id lists and tile ranges
bit-exact; image within 1e-5 absolute; gradients within 1e-3 relative per element (conftest.gradient_gate).  Skipped when the library was
not built (it needs the reference checkout at build time)."""
import numpy as np
import pytest

from conftest import gradient_gate, scene_tensors, settings_for

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from ds_splat_b200 import GaussianRasterizer, _capi, scenes  # noqa: E402
from oracle import ref_cuda  # noqa: E402

needs_ref = pytest.mark.skipif(not ref_cuda.available(), reason="oracle/_ref/libref_splat.so not built")


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
    # everything a blend decision depends on is bit-identical too: pixel mean, conic, and the 3-D covariance behind them
    # (the fusion of their sums into multiply-adds is spelled out in the preprocess kernel to match the reference's build)
    bits = lambda a: np.ascontiguousarray(a, np.float32).view(np.uint32)
    np.testing.assert_array_equal(bits(rec[:, 0:2]), bits(ref["xy"]))
    np.testing.assert_array_equal(bits(rec[:, 2:5]), bits(ref["conic"]))
    np.testing.assert_array_equal(bits(cov3d.cpu().numpy()), bits(ref["cov3d"]))
    colour_off = (bits(rec[:, 6:9]) != bits(ref["rgb"])).any(axis=1).mean()
    assert colour_off < 0.03 and np.abs(rec[:, 6:9] - ref["rgb"]).max() < 1e-6   # SH sums: last-bit differences only
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
        gradient_gate(g.cpu().numpy(), ref[name_], f"{name}/{name_}")


def test_background_term_of_the_backward_against_reference_cuda():
    """The reference composites no background in the forward image but keeps the background term in the backward
    (cpp/gsplat/backward.cu:161-164): -T_final (bg . v_out) / (1 - alpha) in v_alpha.  The backward blend here folds that
    term into the start value of its per-pixel running sum, so it gets a test of its own with a background that is
    not black: same image as without, gradients those of the reference CUDA path, and noticeably different from the
    black-background ones."""
    sc = scenes.tiny()
    view = sc.views[0]
    v_image = sc.image_grad()
    bg = (0.3, 0.6, 0.1)
    ref = ref_cuda.run(view, sc.means, sc.shs, sc.opacities, sc.scales, sc.rotations, v_image=v_image, bg=bg)
    black = ref_cuda.run(view, sc.means, sc.shs, sc.opacities, sc.scales, sc.rotations, v_image=v_image)
    t = scene_tensors(sc)

    def operator_gradients(background):
        rast = GaussianRasterizer(settings_for(view, bg=background))
        p = {k_: v.clone().requires_grad_(True) for k_, v in t.items()}
        means2d = torch.zeros_like(p["means"], requires_grad=True)
        image, _ = rast(p["means"], means2d, p["shs"], None, p["opacities"], p["scales"], p["rotations"], None)
        image.backward(torch.from_numpy(v_image).cuda())
        torch.cuda.synchronize()
        return image.detach().cpu().numpy(), dict(v_mean=p["means"].grad, v_sh=p["shs"].grad,
                                                  v_opacity=p["opacities"].grad.reshape(-1), v_scale=p["scales"].grad,
                                                  v_rot=p["rotations"].grad, v_xy=means2d.grad[:, :2])

    image, grads = operator_gradients(bg)
    assert np.abs(image - ref["image"]).max() <= 1e-5
    np.testing.assert_array_equal(ref["image"], black["image"])        # the forward ignores the background
    for name_, g in grads.items():
        gradient_gate(g.cpu().numpy(), ref[name_], f"background/{name_}")
    moved = np.abs(ref["v_opacity"] - black["v_opacity"]).max() / np.abs(black["v_opacity"]).max()
    assert moved > 1e-2, "the background must change the opacity gradients for this test to mean anything"


def test_scale_modifier_against_reference_cuda():
    """settings.scale_modifier multiplies every splat's scale before the covariance is formed
    (cpp/rasterizer_kernels.cu:615-659) and its derivative multiplies the scale gradient
    (cpp/gsplat/backward.cu:387-389).  With 0.7: radii bit-exact, image and gradients as the reference CUDA path."""
    sc = scenes.tiny()
    view = sc.views[0]
    v_image = sc.image_grad()
    ref = ref_cuda.run(view, sc.means, sc.shs, sc.opacities, sc.scales, sc.rotations, v_image=v_image, scale_modifier=0.7)
    plain = ref_cuda.run(view, sc.means, sc.shs, sc.opacities, sc.scales, sc.rotations, v_image=v_image)
    assert (ref["radii"] != plain["radii"]).mean() > 0.2          # the modifier does change the splats
    t = scene_tensors(sc)
    rast = GaussianRasterizer(settings_for(view, scale_modifier=0.7))
    p = {k_: v.clone().requires_grad_(True) for k_, v in t.items()}
    means2d = torch.zeros_like(p["means"], requires_grad=True)
    image, radii = rast(p["means"], means2d, p["shs"], None, p["opacities"], p["scales"], p["rotations"], None)
    image.backward(torch.from_numpy(v_image).cuda())
    torch.cuda.synchronize()
    np.testing.assert_array_equal(radii.cpu().numpy(), ref["radii"])
    assert np.abs(image.detach().cpu().numpy() - ref["image"]).max() <= 1e-5
    grads = dict(v_mean=p["means"].grad, v_sh=p["shs"].grad, v_opacity=p["opacities"].grad.reshape(-1),
                 v_scale=p["scales"].grad, v_rot=p["rotations"].grad, v_xy=means2d.grad[:, :2])
    for name_, g in grads.items():
        gradient_gate(g.cpu().numpy(), ref[name_], f"scale_modifier/{name_}")


import json  # noqa: E402
import os  # noqa: E402

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "tile_ranges.json")


@pytest.mark.parametrize("case", json.load(open(GOLDEN)), ids=lambda c: c["name"])
def test_reference_known_answer_ranges_on_the_cuda_kernels(case):
    """The reference's two known-answer tests of the tile-range stage (tests/rasterizer_test.cpp:66-110), fed to the
    CUDA kernels: to dsb_identify_tile_ranges directly, and -- as (tile, splat) pairs sorted by the library's own
    sort -- through the path the fused render takes (sort on the tile bits, then ranges)."""
    h, w = case["image_height"], case["image_width"]
    keys = torch.tensor(case["keys"], dtype=torch.int64, device="cuda")
    got = _capi.identify_tile_ranges(keys, h, w)
    assert got.cpu().tolist() == case["expected"]
    # the same tiles as packed pairs in shuffled order: sort on the 3 live tile bits, then ranges
    order = torch.randperm(len(case["tiles"]), generator=torch.Generator().manual_seed(1))
    pairs = torch.tensor([(case["tiles"][i] << 32) | i for i in order.tolist()], dtype=torch.int64, device="cuda")
    sorted_pairs = _capi.sort_pairs(pairs, 32, 35)
    assert _capi.identify_tile_ranges(sorted_pairs, h, w).cpu().tolist() == case["expected"]


@needs_ref
def test_cpu_checker_against_reference_cuda_directly():
    """The CPU restatement (oracle/gs_oracle.cpp) against the reference's own CUDA kernels on the tiny configuration,
    with no kernel of this library in between: integer stages from the reference's own stage outputs bit-exact,
    the rest within the tolerances of a libm build against an approximate-intrinsics build."""
    from conftest import oracle_camera
    from oracle import oracle as O
    sc = scenes.tiny()
    view = sc.views[0]
    v_image = sc.image_grad()
    ref = ref_cuda.run(view, sc.means, sc.shs, sc.opacities, sc.scales, sc.rotations, v_image=v_image)
    cam = oracle_camera(view)
    pre = O.preprocess(cam, sc.means, sc.shs, sc.opacities, sc.scales, sc.rotations)
    diff = np.abs(pre["radii"] - ref["radii"])
    assert diff.max() <= 1 and (diff != 0).mean() < 2e-3       # ceil() of an approximate sqrt flips a few radii by one
    vis = ref["radii"] > 0
    np.testing.assert_allclose(pre["xy"][vis], ref["xy"][vis], rtol=1e-5, atol=2e-3)
    np.testing.assert_allclose(pre["conic"][vis], ref["conic"][vis], rtol=2e-3, atol=1e-6)
    np.testing.assert_allclose(pre["rgb"][vis], ref["rgb"][vis], rtol=1e-4, atol=1e-5)
    # keys, sort and ranges from the REFERENCE's own per-splat outputs: bit-exact
    pre_ref = dict(pre, xy=np.ascontiguousarray(ref["xy"]), depth=np.ascontiguousarray(ref["depth"]), radii=ref["radii"])
    tiles = np.zeros_like(ref["radii"])
    rect = np.zeros((sc.n, 4), np.int32)
    tw, th = (view.W + 15) // 16, (view.H + 15) // 16
    c, d = pre_ref["xy"] / np.float32(16), (ref["radii"] / np.float32(16)).astype(np.float32)
    trunc = lambda a: np.trunc(a).astype(np.int64)
    x0, x1 = np.clip(trunc(c[:, 0] - d), 0, tw), np.clip(trunc(c[:, 0] + d + np.float32(1)), 0, tw)
    y0, y1 = np.clip(trunc(c[:, 1] - d), 0, th), np.clip(trunc(c[:, 1] + d + np.float32(1)), 0, th)
    tiles = np.where(ref["radii"] > 0, (x1 - x0) * (y1 - y0), 0).astype(np.int32)
    pre_ref["tiles"] = tiles
    keys, ids = O.duplicate_keys(cam, pre_ref)
    keys, ids = O.sort_pairs(keys, ids)
    assert keys.shape[0] == ref["K"]
    np.testing.assert_array_equal(keys, ref["keys_sorted"])
    np.testing.assert_array_equal(ids, ref["ids_sorted"])
    np.testing.assert_array_equal(O.tile_ranges(keys, view.H, view.W), ref["tile_indices"])
    # blend from the reference's records and lists
    opac = sc.opacities.reshape(-1)
    image, ft, fi, _ = O.blend_forward(cam, ids, ref["tile_indices"], pre_ref["xy"], np.ascontiguousarray(ref["conic"]),
                                       np.ascontiguousarray(ref["rgb"]), opac)
    err = np.abs(image - ref["image"]).max(axis=2)
    assert (err > 1e-5).mean() < 2e-4 and (fi != ref["final_idx"]).mean() < 2e-4
    v_xy, v_conic, v_rgb, v_op, _ = O.blend_backward(cam, sc.n, ids, ref["tile_indices"], pre_ref["xy"], np.ascontiguousarray(ref["conic"]),
                                                     np.ascontiguousarray(ref["rgb"]), opac, ref["final_T"], ref["final_idx"], v_image)
    gradient_gate(v_xy, ref["v_xy"], "checker/v_xy")
    gradient_gate(v_conic, ref["v_conic"], "checker/v_conic")
    gradient_gate(v_rgb, ref["v_colors"], "checker/v_colors")
    gradient_gate(v_op, ref["v_opacity"], "checker/v_opacity")
