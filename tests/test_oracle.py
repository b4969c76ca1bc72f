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
