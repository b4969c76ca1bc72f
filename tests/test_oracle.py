"""CPU checks of the oracle itself: the reference's known-answer vectors for the tile-range stage, and
internal consistency properties of the other stages (no GPU needed)."""
import json
import os

import numpy as np
import pytest

from conftest import oracle_camera
from ds_splat_b200 import scenes
from oracle import oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "tile_ranges.json")


@pytest.mark.parametrize("case", json.load(open(GOLDEN)), ids=lambda c: c["name"])
def test_tile_ranges_known_answers(case):
    keys = np.array(case["keys"], np.int64)
    got = O.tile_ranges(keys, case["image_height"], case["image_width"])
    assert got.tolist() == case["expected"]


def test_tile_ranges_empty_list():
    assert O.tile_ranges(np.zeros(0, np.int64), 30, 40).tolist() == [0] * 7


@pytest.fixture(scope="module")
def small():
    sc = scenes.tiny(n=3000, seed=3, W=160, H=112, focal=150.0)
    cam = oracle_camera(sc.views[0])
    fwd = O.forward(cam, sc.means, sc.shs, sc.opacities, sc.scales, sc.rotations)
    return sc, cam, fwd


def test_pair_count_drops_last_splat(small):
    sc, cam, fwd = small
    tiles = fwd["pre"]["tiles"]
    assert fwd["K"] == int(tiles[:-1].sum())
    assert O.count_pairs(tiles, drop_last=False) == int(tiles.sum())
    assert (fwd["ids"] != sc.n - 1).all()


def test_keys_sorted_and_stable(small):
    sc, cam, fwd = small
    keys, ids = fwd["keys"], fwd["ids"]
    assert (np.diff(keys) >= 0).all()
    same = np.diff(keys) == 0
    assert (np.diff(ids)[same] > 0).all()  # equal keys keep ascending splat id
    depth_bits = fwd["pre"]["depth"].view(np.int32).astype(np.int64)
    np.testing.assert_array_equal(keys & 0xFFFFFFFF, depth_bits[ids])
    r = fwd["ranges"]
    tile = keys >> 32
    for t in (0, 5, len(r) - 2):
        assert (tile[r[t]:r[t + 1]] == t).all()
    assert r[0] == 0 and r[-1] == fwd["K"] and (np.diff(r) >= 0).all()


def test_forward_blend_properties(small):
    sc, cam, fwd = small
    assert fwd["image"].shape == (cam.H, cam.W, 3)
    assert (fwd["final_T"] <= 1.0).all() and (fwd["final_T"] >= 1e-4 * (1 - 0.999)).all()
    untouched = fwd["final_idx"] == 0
    # pixels nothing was blended into keep T == 1 and colour 0 (no background is composited)
    blank = untouched & (fwd["final_T"] == 1.0)
    assert (fwd["image"][blank] == 0).all()
    assert fwd["image"].min() >= 0.0


def test_backward_matches_finite_differences(small):
    """The blend/colour part of the gradient is exact calculus (the reference's known simplifications are in
    the geometry part), so opacities and DC colour coefficients must agree with central differences."""
    sc, cam, fwd = small
    v_image = sc.image_grad()
    g = O.backward(cam, fwd, sc.means, sc.shs, sc.opacities, sc.scales, sc.rotations, v_image)
    rng = np.random.default_rng(0)
    vis = np.nonzero(fwd["pre"]["radii"][:-1] > 0)[0]
    picks = rng.choice(vis, 6, replace=False)

    def loss(shs, opac):
        f = O.forward(cam, sc.means, shs, opac, sc.scales, sc.rotations)
        return float((f["image"].astype(np.float64) * v_image).sum())

    for i in picks:
        eps = 1e-2
        sp, sm = sc.shs.copy(), sc.shs.copy()
        sp[i, 0, 1] += eps; sm[i, 0, 1] -= eps
        fd = (loss(sp, sc.opacities) - loss(sm, sc.opacities)) / (2 * eps)
        an = g["v_shs"][i, 0, 1]
        assert abs(fd - an) <= 0.05 * abs(an) + 1e-7, (i, fd, an)
        op, om = sc.opacities.copy(), sc.opacities.copy()
        eps = 2e-3
        op[i] += eps; om[i] -= eps
        fd = (loss(sc.shs, op) - loss(sc.shs, om)) / (2 * eps)
        an = g["v_opacities"][i, 0]
        assert abs(fd - an) <= 0.1 * abs(an) + 2e-6, (i, fd, an)


def test_geometry_gradient_rows_zero_for_invisible(small):
    sc, cam, fwd = small
    g = O.backward(cam, fwd, sc.means, sc.shs, sc.opacities, sc.scales, sc.rotations, sc.image_grad())
    hidden = fwd["pre"]["radii"] <= 0
    assert hidden.any()
    for name in ("v_means3d", "v_scales", "v_rotations", "v_cov3d"):
        assert (g[name][hidden] == 0).all()
    assert g["v_means2d"].shape == (sc.n, 3) and (g["v_means2d"][:, 2] == 0).all()


def test_scene_generators_are_deterministic():
    a, b = scenes.tiny(n=500), scenes.tiny(n=500)
    for name in ("means", "scales", "rotations", "opacities", "shs"):
        np.testing.assert_array_equal(getattr(a, name), getattr(b, name))
    np.testing.assert_allclose(np.linalg.norm(a.rotations, axis=1), 1.0, atol=1e-6)
    v = a.views[0]
    np.testing.assert_allclose(v.view[:3, :3] @ v.view[:3, :3].T, np.eye(3), atol=1e-6)
    np.testing.assert_array_equal(v.viewmatrix_t, v.view.T)


def test_depth_map_is_a_fourth_colour_channel(small):
    """The optional depth output has no reference counterpart; the checker defines it as the splat's view-space
    z blended like a colour.  Pin that definition against the colour path itself: rendering with z in the red
    channel must give the depth map, and its gradient must come back as v_z (and reach the same v_xy, v_conic,
    v_opacity) when the depth map's gradient is fed as the red channel's."""
    sc, cam, fwd = small
    pre = fwd["pre"]
    opac = sc.opacities.reshape(-1)
    z = pre["depth"]
    rgb_z = np.zeros_like(pre["rgb"])
    rgb_z[:, 0] = z
    img_z, ft, fi, _ = O.blend_forward(cam, fwd["ids"], fwd["ranges"], pre["xy"], pre["conic"], rgb_z, opac)
    image, ft2, fi2, _, depth = O.blend_forward(cam, fwd["ids"], fwd["ranges"], pre["xy"], pre["conic"], pre["rgb"], opac, z)
    np.testing.assert_array_equal(image, fwd["image"])
    np.testing.assert_array_equal(depth, img_z[:, :, 0])
    assert depth.max() > 0 and np.isfinite(depth).all()

    rng = np.random.default_rng(5)
    v_depth = rng.normal(0, 1e-3, (cam.H, cam.W)).astype(np.float32)
    v_img_z = np.zeros((cam.H, cam.W, 3), np.float32)
    v_img_z[:, :, 0] = v_depth
    zero_img = np.zeros_like(v_img_z)
    a = O.blend_backward(cam, sc.n, fwd["ids"], fwd["ranges"], pre["xy"], pre["conic"], rgb_z, opac, ft, fi, v_img_z)
    b = O.blend_backward(cam, sc.n, fwd["ids"], fwd["ranges"], pre["xy"], pre["conic"], pre["rgb"], opac, ft, fi, zero_img,
                         z, v_depth)
    np.testing.assert_allclose(b[0], a[0], rtol=1e-5, atol=1e-12)        # v_xy
    np.testing.assert_allclose(b[1], a[1], rtol=1e-5, atol=1e-12)        # v_conic
    np.testing.assert_allclose(b[3], a[3], rtol=1e-5, atol=1e-12)        # v_opacity
    np.testing.assert_allclose(b[5], a[2][:, 0], rtol=1e-5, atol=1e-12)  # v_z == gradient of the "red = z" channel
    assert np.abs(b[2]).max() == 0                                       # no colour gradient from a depth-only loss
    # v_z reaches the mean along the view matrix's third row (cpp/gsplat/backward.cu:253-259)
    zeros2, zeros3 = np.zeros((sc.n, 2), np.float32), np.zeros((sc.n, 3), np.float32)
    vm, _, _, _ = O.project_backward(cam, sc.means, sc.scales, sc.rotations, pre["conic"], pre["cov3d"], pre["radii"],
                                     zeros2, zeros3, b[5])
    vis = pre["radii"] > 0
    V = np.asarray(sc.views[0].view, np.float32).reshape(4, 4)
    np.testing.assert_allclose(vm[vis], b[5][vis, None] * V[2, :3][None, :], rtol=1e-6, atol=1e-12)
    assert np.abs(vm[~vis]).max() == 0


def test_adam_checker_equals_torch_optim_adam():
    """The optimizer-step checker has no reference source to follow; pin it against torch.optim.Adam itself."""
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(12)
    p0 = rng.normal(0, 1, 5000).astype(np.float32)
    grads = [(rng.normal(0, 1e-2, 5000) * (10.0 ** rng.integers(-3, 2))).astype(np.float32) for _ in range(4)]
    tp = torch.nn.Parameter(torch.from_numpy(p0.copy()))
    opt = torch.optim.Adam([tp], lr=1.6e-4, betas=(0.9, 0.999), eps=1e-15)
    p, m, v = p0.copy(), np.zeros_like(p0), np.zeros_like(p0)
    for step, g in enumerate(grads, start=1):
        tp.grad = torch.from_numpy(g.copy())
        opt.step()
        p, m, v = O.adam_step(p, g, m, v, lr=1.6e-4, beta1=0.9, beta2=0.999, eps=1e-15, step=step)
        np.testing.assert_allclose(p, tp.detach().numpy(), rtol=2e-6, atol=1e-9)
    st = opt.state[tp]
    # moments: sums of terms of mixed sign, so the tolerance is relative to the largest entry
    np.testing.assert_allclose(m, st["exp_avg"].numpy(), rtol=1e-5, atol=1e-6 * float(np.abs(m).max()))
    np.testing.assert_allclose(v, st["exp_avg_sq"].numpy(), rtol=1e-5, atol=1e-6 * float(v.max()))


def test_image_loss_checker_properties():
    """The loss checker is autograd over plain torch operations; pin the formula through cases with known answers."""
    torch = pytest.importorskip("torch")
    from oracle import loss_oracle as L
    rng = np.random.default_rng(3)
    img = rng.uniform(0, 1, (23, 31, 3)).astype(np.float32)
    loss_same, grad_same = L.image_loss_and_grad(img, img.copy())
    assert abs(loss_same) < 1e-12                       # identical images: L1 = 0 and SSIM = 1 everywhere
    assert np.abs(grad_same).max() < 1e-9               # ... and that is a stationary point (sign(0) = 0)
    other = rng.uniform(0, 1, img.shape).astype(np.float32)
    l_l1, _ = L.image_loss_and_grad(img, other, lambda_dssim=0.0)
    assert abs(l_l1 - float(np.abs(img.astype(np.float64) - other).mean())) < 1e-9
    l_full, g_full = L.image_loss_and_grad(img, other, lambda_dssim=0.2)
    assert 0.0 < l_full < 1.2 and g_full.shape == img.shape and np.isfinite(g_full).all()
    # SSIM of a constant image against another constant: only the luminance term is left, (2ab + C1) / (a^2 + b^2 + C1),
    # in the interior, where the window does not reach the zero padding
    a, b = 0.3, 0.6
    xa, xb = torch.full((400, 400, 3), a), torch.full((400, 400, 3), b)
    l_const = float(L.image_loss(xa, xb, lambda_dssim=1.0))
    inner = (2 * a * b + 1e-4) / (a * a + b * b + 1e-4)
    assert abs((1.0 - l_const) - inner) < 0.02          # the 5-pixel border changes the mean a little
