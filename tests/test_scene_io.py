"""Scene input: the 3-D Gaussian Splatting checkpoint format (.ply) and the input container of the reference's
timing tests (tests/rasterizer_test.cpp:147-167), both round-tripped through files the test writes itself, and the
camera path of the reference's fly-through protocol (README.md:199-204)."""
import numpy as np
import pytest

from ds_splat_b200 import scene_io, scenes

torch = pytest.importorskip("torch")


def test_ply_checkpoint_round_trip(tmp_path):
    sc = scenes.tiny(n=257, seed=3)
    path = str(tmp_path / "point_cloud.ply")
    scene_io.save_ply(path, sc.means, sc.shs, sc.opacities, sc.scales, sc.rotations)
    got = scene_io.load_ply(path)
    assert got["sh_degree"] == 3 and got["shs"].shape == (257, 16, 3)
    np.testing.assert_array_equal(got["means"], sc.means)
    np.testing.assert_array_equal(got["shs"], sc.shs)                      # stored verbatim, only reordered
    np.testing.assert_allclose(got["opacities"], sc.opacities, rtol=2e-6)  # logit and back
    np.testing.assert_allclose(got["scales"], sc.scales, rtol=2e-6)        # log and back
    np.testing.assert_allclose(got["rotations"], sc.rotations, atol=1e-6)
    raw = scene_io.load_ply(path, activated=False)
    np.testing.assert_allclose(raw["scales"], np.log(sc.scales), rtol=1e-6, atol=1e-6)


def test_ply_stores_higher_sh_bands_channel_major(tmp_path):
    # what the training code writes: all 15 coefficients of red, then green, then blue
    n = 3
    shs = np.arange(n * 16 * 3, dtype=np.float32).reshape(n, 16, 3)
    path = str(tmp_path / "p.ply")
    scene_io.save_ply(path, np.zeros((n, 3)), shs, np.full((n, 1), 0.5), np.ones((n, 3)), np.tile([1.0, 0, 0, 0], (n, 1)))
    v = scene_io._read_ply_vertices(path)
    assert v["f_rest_0"][0] == shs[0, 1, 0] and v["f_rest_1"][0] == shs[0, 2, 0]      # red: coefficients 1, 2, ...
    assert v["f_rest_15"][0] == shs[0, 1, 1] and v["f_rest_30"][0] == shs[0, 1, 2]    # then green, then blue
    assert v["f_dc_2"][1] == shs[1, 0, 2]
    np.testing.assert_array_equal(scene_io.load_ply(path)["shs"], shs)


def test_ply_of_lower_degree_and_bad_files(tmp_path):
    n = 5
    shs = np.random.default_rng(0).standard_normal((n, 4, 3)).astype(np.float32)
    path = str(tmp_path / "deg1.ply")
    scene_io.save_ply(path, np.zeros((n, 3)), shs, np.full((n, 1), 0.3), np.ones((n, 3)), np.tile([0.0, 1, 0, 0], (n, 1)))
    got = scene_io.load_ply(path)
    assert got["sh_degree"] == 1
    np.testing.assert_array_equal(got["shs"], shs)
    bad = tmp_path / "bad.ply"
    bad.write_bytes(b"ply\nformat ascii 1.0\nelement vertex 1\nproperty float x\nend_header\n0\n")
    with pytest.raises(ValueError, match="binary_little_endian"):
        scene_io.load_ply(str(bad))
    short = tmp_path / "short.ply"
    data = open(path, "rb").read()
    short.write_bytes(data[:-40])
    with pytest.raises(ValueError, match="vertices"):
        scene_io.load_ply(str(short))


def _container_dict(sc):
    v = sc.views[0]
    return dict(means_3d=torch.from_numpy(sc.means), means_2d=torch.zeros(sc.n, 3), shs=torch.from_numpy(sc.shs),
                opacities=torch.from_numpy(sc.opacities), scales=torch.from_numpy(sc.scales), rotations=torch.from_numpy(sc.rotations),
                viewmatrix=torch.from_numpy(v.viewmatrix_t), projmatrix=torch.from_numpy(v.projmatrix_t),
                campos=torch.from_numpy(np.ascontiguousarray(v.campos)), image_height=v.H, image_width=v.W, tanfovx=v.tanfovx,
                tanfovy=v.tanfovy, scale_modifier=1.0, sh_degree=3)


@pytest.mark.parametrize("form", ["torchscript", "dict"])
def test_reference_test_container_round_trip(tmp_path, form):
    sc = scenes.tiny(n=100, seed=4, W=64, H=48, focal=50.0)
    d = _container_dict(sc)
    path = str(tmp_path / "input_data.pt")
    if form == "torchscript":
        scene_io.save_container(path, d)
        # the reference's C++ test reads exactly these attributes from the scripted module
        m = torch.jit.load(path)
        assert int(m.image_height) == 48 and abs(float(m.tanfovx) - d["tanfovx"]) < 1e-12
    else:
        torch.save(d, path)
    got = scene_io.load_container(path)
    for name in scene_io.CONTAINER_TENSORS:
        assert torch.equal(got[name], d[name]), name
    for name, kind in scene_io.CONTAINER_SCALARS.items():
        assert isinstance(got[name], kind) and got[name] == kind(d[name])
    del d["shs"]
    torch.save(d, path)
    with pytest.raises(ValueError, match="shs"):
        scene_io.load_container(path)


def test_zoom_out_path_backs_away_and_keeps_looking_at_the_target():
    views = scene_io.zoom_out_path(120, start_distance=3.0, end_distance=12.0, W=320, H=180, focal=200.0)
    assert len(views) == 120
    dist = [float(np.linalg.norm(v.campos)) for v in views]
    assert all(b > a for a, b in zip(dist, dist[1:]))
    assert abs(dist[0] / 3.0 - 1.0) < 0.05 and abs(dist[-1] / 12.0 - 1.0) < 0.05
    for v in (views[0], views[60], views[-1]):
        origin_in_camera = v.view @ np.array([0, 0, 0, 1], np.float32)
        assert abs(origin_in_camera[0]) < 1e-4 and abs(origin_in_camera[1]) < 1e-4 and origin_in_camera[2] > 0
