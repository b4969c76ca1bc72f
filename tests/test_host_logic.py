"""Host-side behaviour of the Python operator that needs no GPU: the settings surface of the reference,
argument validation, and the loud failure when inputs are not CUDA tensors."""
import dataclasses

import pytest

torch = pytest.importorskip("torch")

from ds_splat_b200 import GaussianRasterizationSettings, GaussianRasterizer  # noqa: E402

REFERENCE_FIELDS = ["image_height", "image_width", "tanfovx", "tanfovy", "bg", "scale_modifier", "viewmatrix",
                    "projmatrix", "sh_degree", "max_sh_degree", "campos", "prefiltered", "debug"]


def _settings(**kw):
    base = dict(image_height=32, image_width=48, tanfovx=0.5, tanfovy=0.4, bg=torch.zeros(3), scale_modifier=1.0,
                viewmatrix=torch.eye(4), projmatrix=torch.eye(4), sh_degree=3, campos=torch.zeros(3),
                prefiltered=False, debug=False)
    base.update(kw)
    return GaussianRasterizationSettings(**base)


def test_settings_fields_match_reference_order():
    names = [f.name for f in dataclasses.fields(GaussianRasterizationSettings)]
    assert names[:13] == REFERENCE_FIELDS


def test_settings_positional_like_reference_and_keyword_like_graphdeco():
    s = GaussianRasterizationSettings(32, 48, 0.5, 0.4, torch.zeros(3), 1.0, torch.eye(4), torch.eye(4), 2, 3,
                                      torch.zeros(3), False, True)
    assert (s.sh_degree, s.max_sh_degree, s.debug) == (2, 3, True)
    g = _settings()  # graphdeco callers have no max_sh_degree
    assert g.max_sh_degree == 3 and g.strict_reference and not g.channels_first
    with pytest.raises(TypeError):
        GaussianRasterizationSettings(32, 48, 0.5, 0.4, torch.zeros(3), 1.0, torch.eye(4), torch.eye(4), 3)


def test_rasterizer_rejects_cpu_tensors_loudly():
    r = GaussianRasterizer(_settings())
    n = 4
    with pytest.raises(RuntimeError, match="CUDA"):
        r(torch.zeros(n, 3), torch.zeros(n, 3), torch.zeros(n, 16, 3), None, torch.zeros(n, 1), torch.ones(n, 3),
          torch.ones(n, 4), None)


def test_rasterizer_argument_checks():
    r = GaussianRasterizer(_settings())
    with pytest.raises(TypeError):
        r(None, None, None, None, None, None, None, None)
    with pytest.raises(ValueError):
        r(torch.zeros(2, 3), None, torch.zeros(2, 16, 3), torch.zeros(2, 3), torch.zeros(2, 1), None, None, None)


def test_graphdeco_keyword_names_are_accepted():
    r = GaussianRasterizer(_settings())
    with pytest.raises(RuntimeError, match="CUDA"):  # gets past argument mapping, stops at the device check
        r(means3D=torch.zeros(2, 3), means2D=torch.zeros(2, 3), shs=torch.zeros(2, 16, 3), opacities=torch.zeros(2, 1),
          scales=torch.ones(2, 3), rotations=torch.ones(2, 4), cov3D_precomp=None)


def test_launching_classes_refuse_tensors_that_are_not_on_a_cuda_device():
    """ImageLoss, FlatAdam and ViewRenderer launch kernels on the current device and stream; tensors that live
    elsewhere must raise instead of reaching a launch with foreign pointers."""
    import torch
    from ds_splat_b200 import _capi, dp
    with pytest.raises(RuntimeError, match="CUDA"):
        _capi.stream_ptr(torch.device("cpu"))
    img = torch.zeros(8, 8, 3)
    loss = dp.ImageLoss.__new__(dp.ImageLoss)   # no library needed for the device check
    with pytest.raises(RuntimeError, match="CUDA kernels"):
        loss.gradient(img, img)
    adam = dp.FlatAdam.__new__(dp.FlatAdam)
    adam.dev = torch.device("cpu")
    with pytest.raises(RuntimeError, match="launches CUDA kernels"):
        adam.step(dp.GradientBuffer(4, "cpu"))


def test_gradient_and_parameter_blocks_share_one_layout_and_pad_to_shards():
    import torch
    from ds_splat_b200 import dp
    g = dp.GradientBuffer(5, "cpu", shards=4)
    assert g.length == 5 * 59 and g.storage.numel() % 16 == 0 and g.storage.numel() - g.length < 16
    assert g.flat.data_ptr() == g.storage.data_ptr() and g.flat.numel() == g.length
    params = dict(means3d=torch.randn(5, 3), shs=torch.randn(5, 16, 3), opacities=torch.rand(5, 1), scales=torch.rand(5, 3),
                  rotations=torch.randn(5, 4))
    p = dp.ParameterBuffer.from_tensors(params, shards=4)
    assert p.segments == g.segments
    for name, tensor in params.items():
        assert torch.equal(p.views[name], tensor)
        a, b = p.segments[name]
        assert torch.equal(p.storage[a:b], tensor.reshape(-1))


def test_sharded_adam_slices_cover_every_chunk_once():
    """One process, three chunks: the rank's slices are the chunks themselves, every element belongs to exactly one
    part, the parts' places in the moment buffers do not overlap, and a block that does not split is refused."""
    import torch
    from ds_splat_b200 import dp
    params = dict(means3d=torch.randn(7, 3), shs=torch.randn(7, 16, 3), opacities=torch.rand(7, 1), scales=torch.rand(7, 3),
                  rotations=torch.randn(7, 4))
    lrs = {name: 1e-3 for name, _ in dp.SEGMENTS}
    p = dp.ParameterBuffer.from_tensors(params, shards=3)
    calls = []
    opt = dp.ShardedAdam(p, lrs, chunks=3, update=lambda *a: calls.append((a[0].data_ptr(), a[0].numel(), a[2].data_ptr())))
    assert len(opt.slices) == 3 and not opt.pipelined()
    covered = torch.zeros(p.storage.numel(), dtype=torch.int32)
    moments = torch.zeros(opt.m.numel(), dtype=torch.int32)
    for lo, hi, parts in opt.slices:
        for name, a, b, mo in parts:
            assert lo <= a < b <= hi and p.segments[name][0] <= a and b <= p.segments[name][1]
            covered[a:b] += 1
            moments[mo:mo + (b - a)] += 1
    assert int(covered[:p.length].min()) == 1 and int(covered.max()) == 1 and int(moments.max()) == 1
    opt.step(dp.GradientBuffer(7, "cpu", shards=3))
    assert sum(n for _, n, _ in calls) == p.length
    with pytest.raises(ValueError):
        dp.ShardedAdam(dp.ParameterBuffer.from_tensors(params, shards=1), lrs, chunks=7)
