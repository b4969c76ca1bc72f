"""Headline-size checks (1,000,000 SH-3 splats at 1920x1080, about 11 million pairs).

The CPU checker is too slow to compare every stage at this size inside a test run, so correctness is
established two ways: (1) against the reference's own CUDA kernels (oracle/_ref), which do run at this
size in a few milliseconds -- integer artefacts bit-exact, image and gradients within tolerance; and
(2) through properties that hold at any size: the pair list is ordered by tile, then depth bits, then
splat id; the ranges partition it; the per-tile counts equal what the splats' tile rectangles imply;
the forward is reproducible bit for bit; the backward is linear in the image gradient.
"""
import numpy as np
import pytest

from conftest import capi_camera, gradient_gate, scene_tensors

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from ds_splat_b200 import _capi, scenes  # noqa: E402
from ds_splat_b200.dp import CameraTensors, GradientBuffer, ViewRenderer  # noqa: E402
from oracle import ref_cuda  # noqa: E402


@pytest.fixture(scope="module")
def full():
    sc = scenes.headline()
    view = sc.views[0]
    t = scene_tensors(sc)
    cam, keep = capi_camera(view)
    records, radii, tiles, cov3d, depth_keys = _capi.preprocess(cam, t["means"], t["shs"], t["opacities"], t["scales"],
                                                               t["rotations"])
    offsets, k = _capi.plan_pairs(cam, tiles, depth_keys)
    pairs = _capi.emit_pairs(cam, k, records, tiles, depth_keys, offsets)
    tile_bits = max(1, int(np.ceil(np.log2(view.num_tiles))))
    sorted_pairs = _capi.sort_pairs(pairs, 32, 32 + tile_bits)
    ranges = _capi.identify_tile_ranges(sorted_pairs, view.H, view.W)
    torch.cuda.synchronize()
    return dict(sc=sc, view=view, t=t, cam=cam, keep=keep, records=records, radii=radii, tiles=tiles, k=k,
                sorted_pairs=sorted_pairs, ranges=ranges)


def test_pair_list_is_ordered_by_tile_depth_id(full):
    sp, rec, k = full["sorted_pairs"], full["records"], full["k"]
    # capi_camera() builds cameras with the reference's "last splat is never drawn" behaviour
    assert k == int(full["tiles"][:-1].sum().item()) and sp.shape[0] == k and k > 5_000_000
    tile = sp >> 32
    ids = sp & 0xFFFFFFFF
    depth_bits = rec[:, 9].contiguous().view(torch.int32).to(torch.int64)[ids]  # positive floats order like their bits
    same_tile = tile[1:] == tile[:-1]
    assert bool((tile[1:] >= tile[:-1]).all())
    assert bool((~same_tile | (depth_bits[1:] >= depth_bits[:-1])).all())
    same_depth = same_tile & (depth_bits[1:] == depth_bits[:-1])
    assert bool((~same_depth | (ids[1:] > ids[:-1])).all())


def test_ranges_partition_the_list_and_match_rectangles(full):
    view, rec, ranges, sp, k = full["view"], full["records"], full["ranges"].to(torch.int64), full["sorted_pairs"], full["k"]
    assert int(ranges[0]) == 0 and int(ranges[-1]) == k and bool((ranges[1:] >= ranges[:-1]).all())
    # every entry of tile t's range carries tile id t
    tile_of_slot = torch.repeat_interleave(torch.arange(view.num_tiles, device=sp.device), ranges[1:] - ranges[:-1])
    assert bool((tile_of_slot == (sp >> 32)).all())
    # counts implied by the tile rectangles of the visible splats (corner marks + 2-D prefix sum)
    tx, ty = (view.W + 15) // 16, (view.H + 15) // 16
    rx, ry = rec[:, 10].contiguous().view(torch.int32).to(torch.int64), rec[:, 11].contiguous().view(torch.int32).to(torch.int64)
    x0, x1, y0, y1 = rx & 0xFFFF, rx >> 16, ry & 0xFFFF, ry >> 16
    vis = full["tiles"] > 0
    vis[-1] = False  # the last splat is never drawn (reference behaviour kept by capi_camera())
    x0, x1, y0, y1 = x0[vis], x1[vis], y0[vis], y1[vis]
    grid = torch.zeros((ty + 1) * (tx + 1), dtype=torch.int64, device=sp.device)
    one = torch.ones_like(x0)
    for yy, xx, sgn in ((y0, x0, 1), (y0, x1, -1), (y1, x0, -1), (y1, x1, 1)):
        grid.index_add_(0, yy * (tx + 1) + xx, sgn * one)
    counts = grid.view(ty + 1, tx + 1).cumsum(0).cumsum(1)[:ty, :tx].reshape(-1)
    assert bool((counts == ranges[1:] - ranges[:-1]).all())


def test_forward_is_reproducible_and_backward_is_linear(full):
    sc, view, t = full["sc"], full["view"], full["t"]
    r = ViewRenderer(t["means"], t["shs"], t["opacities"], t["scales"], t["rotations"])
    cam = CameraTensors.from_view(view, "cuda")
    img1 = r.forward(cam).clone()
    img2 = r.forward(cam).clone()
    assert torch.equal(img1, img2)
    assert bool(torch.isfinite(img1).all()) and float(img1.min()) >= 0.0
    v = torch.from_numpy(sc.image_grad()).cuda()
    g1, g2 = GradientBuffer(sc.n, "cuda"), GradientBuffer(sc.n, "cuda")
    r.backward(v, g1, accumulate=False)
    r.backward(2.0 * v, g2, accumulate=False)
    torch.cuda.synchronize()
    # float atomics add in a different order on every launch: linear up to rounding
    scale = float(g1.flat.abs().max())
    assert float((g2.flat - 2.0 * g1.flat).abs().max()) <= 1e-4 * scale
    r.backward(v, g2, accumulate=True)  # g2 = 2 g + g
    torch.cuda.synchronize()
    assert float((g2.flat - 3.0 * g1.flat).abs().max()) <= 2e-4 * scale


@pytest.mark.skipif(not ref_cuda.available(), reason="oracle/_ref/libref_splat.so not built")
def test_headline_size_against_reference_cuda(full):
    sc, view, t = full["sc"], full["view"], full["t"]
    v_image = sc.image_grad()
    ref = ref_cuda.run(view, sc.means, sc.shs, sc.opacities, sc.scales, sc.rotations, v_image=v_image)
    assert int((full["radii"].cpu().numpy() != ref["radii"]).sum()) == 0
    assert full["k"] == ref["K"]
    keys_g, ids_g = _capi.export_reference_lists(full["sorted_pairs"], full["records"])
    np.testing.assert_array_equal(keys_g.cpu().numpy(), ref["keys_sorted"])
    np.testing.assert_array_equal(ids_g.cpu().numpy(), ref["ids_sorted"])
    np.testing.assert_array_equal(full["ranges"].cpu().numpy(), ref["tile_indices"])

    r = ViewRenderer(t["means"], t["shs"], t["opacities"], t["scales"], t["rotations"])
    image = r.forward(CameraTensors.from_view(view, "cuda"))
    assert np.abs(image.cpu().numpy() - ref["image"]).max() <= 1e-5
    g = GradientBuffer(sc.n, "cuda")
    r.backward(torch.from_numpy(v_image).cuda(), g, accumulate=False)
    torch.cuda.synchronize()
    pairs = dict(v_mean=g.views["means3d"], v_sh=g.views["shs"], v_opacity=g.views["opacities"].reshape(-1),
                 v_scale=g.views["scales"], v_rot=g.views["rotations"])
    for name, got in pairs.items():
        want = ref[name]
        gradient_gate(got.cpu().numpy().reshape(want.shape), want, f"c1/{name}")
