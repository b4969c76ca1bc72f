"""The Python operator end to end on the GPU: agreement with the CPU checker from raw inputs, the edge
cases the reference leaves unhandled (no visible splat, a single splat, ragged image sizes), the optional
input forms (colors_precomp, lower SH degrees, cov_3d_precomp), stream use and error reporting."""
import numpy as np
import pytest

from conftest import oracle_camera, scene_tensors, settings_for

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from ds_splat_b200 import GaussianRasterizer, _capi, scenes  # noqa: E402
from ds_splat_b200.dp import CameraTensors, DensifyStats, GradientBuffer, ViewRenderer, data_parallel_step  # noqa: E402
from oracle import oracle as O  # noqa: E402


def _run_operator(sc, view, sh_degree=3, colors=None, **settings_kw):
    t = scene_tensors(sc)
    p = {k: v.clone().requires_grad_(True) for k, v in t.items()}
    m2 = torch.zeros_like(p["means"], requires_grad=True)
    rast = GaussianRasterizer(settings_for(view, sh_degree=sh_degree, **settings_kw))
    if colors is None:
        image, radii = rast(p["means"], m2, p["shs"], None, p["opacities"], p["scales"], p["rotations"], None)
    else:
        p["colors"] = colors.clone().requires_grad_(True)
        image, radii = rast(p["means"], m2, None, p["colors"], p["opacities"], p["scales"], p["rotations"], None)
    return p, m2, image, radii


def _rel(a, b):
    return float(np.abs(a - b).max()) / max(float(np.abs(b).max()), 1e-20)


@pytest.mark.parametrize("sh_degree", [0, 1, 2, 3])
def test_operator_matches_checker_from_raw_inputs(sh_degree):
    sc = scenes.tiny(n=8000, seed=31 + sh_degree, W=256, H=160, focal=220.0)
    view = sc.views[0]
    p, m2, image, radii = _run_operator(sc, view, sh_degree=sh_degree)
    v_image = sc.image_grad()
    image.backward(torch.from_numpy(v_image).cuda())
    cam = oracle_camera(view, sh_degree=sh_degree)
    fwd = O.forward(cam, sc.means, sc.shs, sc.opacities, sc.scales, sc.rotations)
    bwd = O.backward(cam, fwd, sc.means, sc.shs, sc.opacities, sc.scales, sc.rotations, v_image)
    assert image.shape == (view.H, view.W, 3) and radii.dtype == torch.int32
    err = np.abs(image.detach().cpu().numpy() - fwd["image"]).max(axis=2)
    assert (err > 1e-5).mean() < 2e-3 and err.max() < 5e-2
    assert (radii.cpu().numpy() != fwd["pre"]["radii"]).mean() < 3e-3
    # from raw inputs a flipped radius changes a splat's pair list, so gradients are compared at 1e-2
    assert _rel(p["opacities"].grad.cpu().numpy(), bwd["v_opacities"]) < 1e-2
    assert _rel(p["shs"].grad.cpu().numpy(), bwd["v_shs"]) < 1e-2
    assert _rel(p["means"].grad.cpu().numpy(), bwd["v_means3d"]) < 1e-2
    assert _rel(p["scales"].grad.cpu().numpy(), bwd["v_scales"]) < 1e-2
    assert _rel(p["rotations"].grad.cpu().numpy(), bwd["v_rotations"]) < 1e-2
    assert _rel(m2.grad.cpu().numpy(), bwd["v_means2d"]) < 1e-2
    nb = (sh_degree + 1) ** 2
    assert (p["shs"].grad[:, nb:, :] == 0).all()  # inactive bands get exact zeros


def test_colors_precomp_path_and_channels_first():
    sc = scenes.tiny(n=3000, seed=41, W=128, H=96, focal=110.0)
    view = sc.views[0]
    cam = oracle_camera(view)
    pre = O.preprocess(cam, sc.means, sc.shs, sc.opacities, sc.scales, sc.rotations)
    colors = torch.from_numpy(pre["rgb"]).cuda()
    p, m2, image, _ = _run_operator(sc, view, colors=colors, channels_first=True)
    assert image.shape == (3, view.H, view.W)
    fwd = O.forward(cam, sc.means, sc.shs, sc.opacities, sc.scales, sc.rotations)
    err = np.abs(image.detach().permute(1, 2, 0).cpu().numpy() - fwd["image"]).max(axis=2)
    assert (err > 1e-5).mean() < 2e-3
    v = torch.from_numpy(sc.image_grad()).cuda().permute(2, 0, 1)
    image.backward(v)
    bwd = O.backward(cam, fwd, sc.means, sc.shs, sc.opacities, sc.scales, sc.rotations, sc.image_grad())
    assert _rel(p["colors"].grad.cpu().numpy(), bwd["v_colors"]) < 1e-2
    assert p["shs"].grad is None


def test_no_visible_splats_and_single_splat():
    sc = scenes.tiny(n=64, seed=51, W=64, H=48, focal=50.0)
    sc.means[:, 0] += 1000.0  # everything far outside the frustum: K == 0, which the reference cannot handle
    p, m2, image, radii = _run_operator(sc, sc.views[0])
    image.sum().backward()
    torch.cuda.synchronize()
    assert float(image.detach().abs().max()) == 0.0 and int(radii.max()) == 0
    for name in ("means", "shs", "opacities", "scales", "rotations"):
        assert float(p[name].grad.abs().max()) == 0.0
    # centres behind the camera pass the frustum test (w < 0): radii are reported as the reference does,
    # but nothing is drawn and all gradients are finite zeros
    behind = scenes.tiny(n=64, seed=53, W=64, H=48, focal=50.0)
    behind.means[:, 2] = -50.0
    p, m2, image, radii = _run_operator(behind, behind.views[0])
    image.sum().backward()
    torch.cuda.synchronize()
    assert float(image.detach().abs().max()) == 0.0 and int(radii.max()) > 0
    for name in ("means", "shs", "opacities", "scales", "rotations"):
        assert torch.isfinite(p[name].grad).all() and float(p[name].grad.abs().max()) == 0.0
    one = scenes.tiny(n=1, seed=52, W=64, H=48, focal=50.0)
    one.means[:] = 0.0
    p, m2, image, radii = _run_operator(one, one.views[0], strict_reference=False)
    assert int(radii[0]) > 0 and float(image.detach().max()) > 0.0
    p2, _, image2, radii2 = _run_operator(one, one.views[0], strict_reference=True)
    # with the reference's rule the splat with the highest index is never drawn, but its radius is reported
    assert int(radii2[0]) == int(radii[0]) and float(image2.detach().max()) == 0.0


def test_cov3d_precomp_forward_equals_scale_rotation_forward():
    sc = scenes.tiny(n=2000, seed=61, W=96, H=80, focal=90.0)
    view = sc.views[0]
    t = scene_tensors(sc)
    rast = GaussianRasterizer(settings_for(view))
    img_a, rad_a = rast(t["means"], None, t["shs"], None, t["opacities"], t["scales"], t["rotations"], None)
    cam = oracle_camera(view)
    cov = torch.from_numpy(O.preprocess(cam, sc.means, sc.shs, sc.opacities, sc.scales, sc.rotations)["cov3d"]).cuda()
    img_b, rad_b = rast(means3D=t["means"], means2D=None, shs=t["shs"], opacities=t["opacities"], cov3D_precomp=cov)
    assert (rad_a != rad_b).float().mean() < 5e-3
    assert float((img_a - img_b).abs().max()) < 1e-2


def test_runs_on_the_current_stream_and_other_device_buffers_untouched():
    sc = scenes.tiny(n=5000, seed=71, W=160, H=128, focal=140.0)
    view = sc.views[0]
    t = scene_tensors(sc)
    rast = GaussianRasterizer(settings_for(view))
    ref_img, _ = rast(t["means"], None, t["shs"], None, t["opacities"], t["scales"], t["rotations"], None)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        img, _ = rast(t["means"], None, t["shs"], None, t["opacities"], t["scales"], t["rotations"], None)
    s.synchronize()
    assert torch.equal(img, ref_img)  # forward is deterministic


def test_errors_are_python_exceptions():
    sc = scenes.tiny(n=100, seed=81, W=64, H=48, focal=50.0)
    view = sc.views[0]
    t = scene_tensors(sc)
    rast = GaussianRasterizer(settings_for(view))
    with pytest.raises(RuntimeError, match="float32"):
        rast(t["means"].double(), None, t["shs"], None, t["opacities"], t["scales"], t["rotations"], None)
    with pytest.raises(RuntimeError, match="shs must be"):
        rast(t["means"], None, t["shs"][:, :9].contiguous(), None, t["opacities"], t["scales"], t["rotations"], None)
    with pytest.raises(RuntimeError, match="cov3D"):
        rast(t["means"], None, t["shs"], None, t["opacities"], None, None, None)
    with pytest.raises(_capi.DsbError):
        cam, keep = _capi.make_camera(0, 0, 1.0, 1.0, t["means"], t["means"], t["means"])
        _capi.blend_forward(cam, t["means"], t["means"].long(), t["means"].int())


def test_view_renderer_accumulates_like_autograd():
    """The fused multi-view path (gradient accumulation into the flat buffer) equals summed autograd gradients."""
    sc = scenes.headline(n=20_000, seed=91, W=320, H=192, focal=200.0, views=3, ring=True)
    t = scene_tensors(sc)
    r = ViewRenderer(t["means"], t["shs"], t["opacities"], t["scales"], t["rotations"])
    grads = GradientBuffer(sc.n, "cuda")
    grads.flat.fill_(5.0)
    cams = [CameraTensors.from_view(v, "cuda") for v in sc.views]
    vimgs = [torch.from_numpy(sc.image_grad(i)).cuda() for i in range(len(sc.views))]
    data_parallel_step(r, cams, vimgs, grads)
    p = {k: v.clone().requires_grad_(True) for k, v in t.items()}
    for v, vi in zip(sc.views, vimgs):
        img, _ = GaussianRasterizer(settings_for(v))(p["means"], None, p["shs"], None, p["opacities"], p["scales"], p["rotations"], None)
        img.backward(vi)
    torch.cuda.synchronize()
    for name, key in (("means", "means3d"), ("shs", "shs"), ("opacities", "opacities"), ("scales", "scales"), ("rotations", "rotations")):
        assert _rel(grads.views[key].cpu().numpy(), p[name].grad.cpu().numpy()) < 1e-3, name


def test_fused_render_matches_stage_calls():
    """dsb_forward_render derives tile ranges and sort digit counts from a per-tile count grid; its sorted list,
    ranges and image must equal those of the individual stage calls bit for bit (ragged image size on purpose)."""
    sc = scenes.headline(n=60_000, seed=93, W=500, H=297, focal=300.0)
    view = sc.views[0]
    t = scene_tensors(sc)
    r = ViewRenderer(t["means"], t["shs"], t["opacities"], t["scales"], t["rotations"], tight_tiles=False)
    image = r.forward(CameraTensors.from_view(view, "cuda")).clone()
    k = r.last_k
    fused_pairs = r.pairs[:k].clone()
    fused_ranges = r._ranges(r.cur, view.H, view.W)
    from conftest import capi_camera
    cam, keep = capi_camera(view)
    records, radii, tiles, cov3d, dk = _capi.preprocess(cam, t["means"], t["shs"], t["opacities"], t["scales"], t["rotations"])
    offsets, k2 = _capi.plan_pairs(cam, tiles, dk)
    pairs = _capi.emit_pairs(cam, k2, records, tiles, dk, offsets)
    bits = max(1, int(np.ceil(np.log2(view.num_tiles))))
    sp = _capi.sort_pairs(pairs, 32, 32 + bits)
    ranges = _capi.identify_tile_ranges(sp, view.H, view.W)
    img2, _, _ = _capi.blend_forward(cam, records, sp, ranges)
    assert k == k2 and k > 0
    assert torch.equal(fused_pairs, sp)
    assert torch.equal(fused_ranges, ranges)
    assert torch.equal(image, img2)


def test_return_depth_is_differentiable_and_leaves_the_image_alone():
    sc = scenes.tiny(n=6000, seed=77, W=208, H=144, focal=200.0)
    view = sc.views[0]
    p0, _, image0, radii0 = _run_operator(sc, view)
    t = scene_tensors(sc)
    p = {k: v.clone().requires_grad_(True) for k, v in t.items()}
    rast = GaussianRasterizer(settings_for(view, return_depth=True))
    image, radii, depth = rast(p["means"], None, p["shs"], None, p["opacities"], p["scales"], p["rotations"], None)
    assert torch.equal(image, image0) and torch.equal(radii, radii0) and depth.shape == (view.H, view.W)
    cam = oracle_camera(view)
    fwd = O.forward(cam, sc.means, sc.shs, sc.opacities, sc.scales, sc.rotations, with_depth=True)
    err = np.abs(depth.detach().cpu().numpy() - fwd["depth"])
    assert (err > 1e-4).mean() < 2e-3  # raw-input comparison: a flipped radius or threshold moves a few pixels
    # a loss on the depth map alone reaches the geometry but not the colours
    rng = np.random.default_rng(3)
    v_depth = rng.normal(0, 1e-3, (view.H, view.W)).astype(np.float32)
    depth.backward(torch.from_numpy(v_depth).cuda())
    torch.cuda.synchronize()
    bwd = O.backward(cam, fwd, sc.means, sc.shs, sc.opacities, sc.scales, sc.rotations,
                     np.zeros((view.H, view.W, 3), np.float32), v_depth)
    assert float(p["shs"].grad.abs().max()) == 0.0
    assert _rel(p["means"].grad.cpu().numpy(), bwd["v_means3d"]) < 1e-2
    assert _rel(p["opacities"].grad.cpu().numpy(), bwd["v_opacities"]) < 1e-2
    assert _rel(p["scales"].grad.cpu().numpy(), bwd["v_scales"]) < 1e-2


def test_batched_views_equal_one_view_at_a_time():
    """render_views sums the per-splat backward of up to eight views in one kernel; eleven views (two batches,
    the loss given as a callable) must give what eleven single-view backward calls with accumulation give."""
    sc = scenes.headline(n=15_000, seed=92, W=256, H=160, focal=180.0, views=11, ring=True)
    t = scene_tensors(sc)
    cams = [CameraTensors.from_view(v, "cuda") for v in sc.views]
    vimgs = [torch.from_numpy(sc.image_grad(i)).cuda() for i in range(len(sc.views))]
    batched = ViewRenderer(t["means"], t["shs"], t["opacities"], t["scales"], t["rotations"])
    g_b = GradientBuffer(sc.n, "cuda")
    g_b.flat.fill_(3.0)
    seen = []
    batched.render_views(cams, lambda i, image: (seen.append((i, tuple(image.shape))), vimgs[i])[1], g_b, accumulate=False)
    assert [i for i, _ in seen] == list(range(11)) and all(s == (160, 256, 3) for _, s in seen)
    single = ViewRenderer(t["means"], t["shs"], t["opacities"], t["scales"], t["rotations"])
    g_s = GradientBuffer(sc.n, "cuda")
    for i, cam in enumerate(cams):
        single.forward(cam)
        single.backward(vimgs[i], g_s, accumulate=i > 0)
    torch.cuda.synchronize()
    for key in ("means3d", "shs", "opacities", "scales", "rotations"):
        a, b = g_b.views[key].cpu().numpy(), g_s.views[key].cpu().numpy()
        assert _rel(a, b) < 1e-4, key
    # accumulate=True adds on top of what the buffer holds
    batched.render_views(cams[:2], vimgs[:2], g_b, accumulate=True)
    single.forward(cams[0]); single.backward(vimgs[0], g_s, accumulate=True)
    single.forward(cams[1]); single.backward(vimgs[1], g_s, accumulate=True)
    torch.cuda.synchronize()
    assert _rel(g_b.views["shs"].cpu().numpy(), g_s.views["shs"].cpu().numpy()) < 1e-4


@pytest.mark.parametrize("ndc_units", [False, True])
def test_densification_statistics_equal_what_a_loop_around_the_operator_collects(ndc_units):
    """The per-splat backward of a step keeps gradient-norm sums, visibility counts and largest radii; a training
    loop around the single-view operator builds the same numbers from v_means2d and radii of every view."""
    sc = scenes.headline(n=12_000, seed=97, W=256, H=160, focal=180.0, views=10, ring=True)
    t = scene_tensors(sc)
    cams = [CameraTensors.from_view(v, "cuda") for v in sc.views]
    vimgs = [torch.from_numpy(sc.image_grad(i)).cuda() for i in range(len(sc.views))]
    stats = DensifyStats(sc.n, "cuda", ndc_units=ndc_units)
    r = ViewRenderer(t["means"], t["shs"], t["opacities"], t["scales"], t["rotations"])
    g = GradientBuffer(sc.n, "cuda")
    r.render_views(cams, vimgs, g, accumulate=False, stats=stats)      # two batches: 8 + 2 views
    r.render_views(cams[:3], vimgs[:3], g, accumulate=False, stats=stats)  # statistics keep adding across steps
    want = DensifyStats(sc.n, "cuda", ndc_units=ndc_units)
    for i in list(range(10)) + [0, 1, 2]:
        p, m2, image, radii = _run_operator(sc, sc.views[i])
        image.backward(vimgs[i])
        want.add_view(m2.grad, radii, sc.views[i].H, sc.views[i].W)
    torch.cuda.synchronize()
    assert torch.equal(stats.visible_count, want.visible_count) and float(stats.visible_count.max()) == 13.0
    assert torch.equal(stats.max_radius, want.max_radius) and float(stats.max_radius.max()) > 0
    scale = float(want.grad_norm_sum.max())
    assert scale > 0 and float((stats.grad_norm_sum - want.grad_norm_sum).abs().max()) <= 1e-4 * scale
    never = stats.visible_count == 0
    assert bool(never.any()) and float(stats.grad_norm_sum[never].abs().max()) == 0.0
    stats.zero_()
    assert float(stats.flat.abs().max()) == 0.0


def test_preprocess_of_several_views_is_bit_identical_to_one_at_a_time():
    from conftest import capi_camera
    sc = scenes.headline(n=30_000, seed=94, W=400, H=240, focal=260.0, views=5, ring=True)
    t = scene_tensors(sc)
    cams, keep = zip(*[capi_camera(v) for v in sc.views])
    outs, cov3d = _capi.preprocess_views(list(cams), t["means"], t["shs"], t["opacities"], t["scales"], t["rotations"])
    torch.cuda.synchronize()
    for cam, (records, radii, tiles, dkeys, _marks) in zip(cams, outs):
        r1, ra1, t1, c1, d1 = _capi.preprocess(cam, t["means"], t["shs"], t["opacities"], t["scales"], t["rotations"])
        assert torch.equal(records.view(torch.int32), r1.view(torch.int32))
        assert torch.equal(radii, ra1) and torch.equal(tiles, t1) and torch.equal(dkeys, d1)
        assert torch.equal(cov3d, c1)
    assert int(outs[0][1].max()) > 0 and not torch.equal(outs[0][0], outs[1][0])


def test_torch_free_forward_equals_the_operator_image():
    """dsb_forward_core takes the argument list of the reference's C++ entry (row-major matrices, device pointers,
    no caller-side scratch) and must render what the operator renders."""
    import ctypes as C
    sc = scenes.tiny(n=9000, seed=61, W=336, H=208, focal=260.0)
    view = sc.views[0]
    _, _, image, _ = _run_operator(sc, view)
    t = scene_tensors(sc)
    vm = torch.from_numpy(np.ascontiguousarray(view.view, dtype=np.float32)).cuda()    # row-major [R|t]
    pm = torch.from_numpy(np.ascontiguousarray(view.proj, dtype=np.float32)).cuda()    # row-major P*V
    cp = torch.from_numpy(np.ascontiguousarray(view.campos, dtype=np.float32)).cuda()
    out = torch.full((view.H, view.W, 3), -1.0, device="cuda")
    lib = _capi.lib()
    _capi.check(lib.dsb_forward_core(t["means"].data_ptr(), t["shs"].data_ptr(), t["opacities"].data_ptr(),
                                     t["scales"].data_ptr(), t["rotations"].data_ptr(), sc.n, vm.data_ptr(), pm.data_ptr(),
                                     cp.data_ptr(), view.W, view.H, C.c_float(view.tanfovx), C.c_float(view.tanfovy),
                                     C.c_float(1.0), 3, 3, out.data_ptr(), _capi.stream_ptr()))
    torch.cuda.synchronize()
    assert torch.equal(out, image.detach())
    # no splats: a black image, no error
    _capi.check(lib.dsb_forward_core(None, None, None, None, None, 0, vm.data_ptr(), pm.data_ptr(), cp.data_ptr(), view.W,
                                     view.H, C.c_float(view.tanfovx), C.c_float(view.tanfovy), C.c_float(1.0), 3, 3,
                                     out.data_ptr(), _capi.stream_ptr()))
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0


def test_tight_tiles_change_the_pair_list_but_not_the_results():
    """DSB_FLAG_TIGHT_TILES drops the (tile, splat) pairs of tiles a splat cannot contribute to.  The pair count must
    fall, image and final transmittance must stay bit-identical, gradients equal up to atomic summation order."""
    for sc in (scenes.headline(n=120_000, seed=95, W=960, H=544, focal=560.0), scenes.stress(n=4_000, seed=96, W=640, H=368, focal=400.0)):
        view = sc.views[0]
        t = scene_tensors(sc)
        cam = CameraTensors.from_view(view, "cuda")
        v = torch.from_numpy(sc.image_grad()).cuda()
        out = {}
        for tight in (False, True):
            r = ViewRenderer(t["means"], t["shs"], t["opacities"], t["scales"], t["rotations"], tight_tiles=tight)
            image = r.forward(cam).clone()
            final_t = r._image_buffers(view.H, view.W)[1].clone()
            g = GradientBuffer(sc.n, "cuda")
            r.backward(v, g, accumulate=False)
            torch.cuda.synchronize()
            out[tight] = (r.last_k, image, final_t, g.flat.clone(), r.radii.clone())
        k_ref, img_ref, ft_ref, g_ref, radii_ref = out[False]
        k_tight, img_t, ft_t, g_t, radii_t = out[True]
        assert 0 < k_tight < 0.85 * k_ref
        assert torch.equal(img_t, img_ref) and torch.equal(ft_t, ft_ref) and torch.equal(radii_t, radii_ref)
        assert float((g_t - g_ref).abs().max()) <= 1e-5 * float(g_ref.abs().max())


def test_large_tile_grid_takes_the_global_memory_layout_path():
    """Above about 50,000 tiles the corner-mark grid no longer fits shared memory: the layout kernel then works in
    global memory and leaves no tile order.  Lists, ranges and image must still equal the per-stage calls."""
    sc = scenes.headline(n=3_000, seed=97, W=6000, H=4000, focal=3300.0)
    view = sc.views[0]
    assert view.num_tiles > 60_000
    t = scene_tensors(sc)
    r = ViewRenderer(t["means"], t["shs"], t["opacities"], t["scales"], t["rotations"], tight_tiles=False)
    image = r.forward(CameraTensors.from_view(view, "cuda")).clone()
    k = r.last_k
    fused_pairs = r.pairs[:k].clone()
    fused_ranges = r._ranges(r.cur, view.H, view.W).clone()
    g = GradientBuffer(sc.n, "cuda")
    r.backward(torch.from_numpy(sc.image_grad()).cuda(), g, accumulate=False)   # backward without a tile order
    from conftest import capi_camera
    cam, keep = capi_camera(view)
    records, radii, tiles, cov3d, dk = _capi.preprocess(cam, t["means"], t["shs"], t["opacities"], t["scales"], t["rotations"])
    offsets, k2 = _capi.plan_pairs(cam, tiles, dk)
    pairs = _capi.emit_pairs(cam, k2, records, tiles, dk, offsets)
    bits = max(1, int(np.ceil(np.log2(view.num_tiles))))
    sp = _capi.sort_pairs(pairs, 32, 32 + bits)
    ranges = _capi.identify_tile_ranges(sp, view.H, view.W)
    img2, ft2, fi2 = _capi.blend_forward(cam, records, sp, ranges)
    acc = _capi.blend_backward(cam, records, sp, ranges, ft2, fi2, torch.from_numpy(sc.image_grad()).cuda())
    out = _capi.geometry_backward(cam, t["means"], t["scales"], t["rotations"], records, cov3d, radii, acc)
    torch.cuda.synchronize()
    assert k == k2 and k > 0
    assert torch.equal(fused_pairs, sp) and torch.equal(fused_ranges, ranges) and torch.equal(image, img2)
    assert _rel(g.views["means3d"].cpu().numpy(), out["v_means3d"].cpu().numpy()) < 1e-4


@pytest.mark.parametrize("rows", [False, True])
def test_plan_of_several_views_equals_one_at_a_time(rows):
    """dsb_plan_views sorts the depth keys and scans the offsets of a batch in the same launches; every view's sorted
    keys, offsets and totals must equal those of the same call on that view alone, and what plain tensor operations
    give: keys in ascending order, offsets = running sum, in that order, of the tile counts (or, with row binning, of
    the rectangle heights: the first row item of every splat) with the last splat skipped as the reference skips it,
    pairs = sum of the tile counts."""
    import ctypes as C
    from conftest import capi_camera
    sc = scenes.headline(n=70_001, seed=98, W=640, H=400, focal=380.0, views=3, ring=True)   # odd length: rows are not tile-aligned
    t = scene_tensors(sc)
    cams, keep = zip(*[capi_camera(v, row_binning=rows) for v in sc.views])
    n, nv, lib = sc.n, 3, _capi.lib()
    h, w = sc.views[0].H, sc.views[0].W
    i32 = lambda *shape: torch.empty(shape, dtype=torch.int32, device="cuda")
    records = [torch.empty((n, _capi.RECORD_FLOATS), dtype=torch.float32, device="cuda") for _ in range(nv)]
    radii, tiles, offsets = [i32(n) for _ in range(nv)], i32(nv, n), i32(nv, n)
    keys = torch.empty((2, nv, n), dtype=torch.int64, device="cuda")
    marks = [torch.empty(int(lib.dsb_tile_marks_bytes(h, w)), dtype=torch.uint8, device="cuda") for _ in range(nv)]
    ranges = [i32(_capi.num_tiles(h, w) + 1) for _ in range(nv)]
    layout = [i32(_capi.LAYOUT_WORDS) for _ in range(nv)]
    cov3d = torch.empty((n, 6), dtype=torch.float32, device="cuda")
    ptrs = lambda ts: (C.c_void_p * len(ts))(*[x.data_ptr() for x in ts])
    _capi.check(lib.dsb_preprocess_views((_capi.DsbCamera * nv)(*cams), nv, n, t["means"].data_ptr(), t["shs"].data_ptr(), None,
                                         t["opacities"].data_ptr(), t["scales"].data_ptr(), t["rotations"].data_ptr(), None,
                                         ptrs(records), ptrs(radii), ptrs([tiles[v] for v in range(nv)]), cov3d.data_ptr(),
                                         ptrs([keys[0, v] for v in range(nv)]), ptrs(marks), ptrs(ranges), ptrs(layout),
                                         _capi.stream_ptr()))
    unsorted = keys[0].clone()
    ws_bytes = int(lib.dsb_plan_workspace_bytes_views(n, nv))
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    ks, krs = (C.c_int64 * nv)(), (C.c_int64 * nv)()
    _capi.check(lib.dsb_plan_views(C.byref(cams[0]), nv, n, n, ptrs(records), tiles.data_ptr(), keys[0].data_ptr(),
                                   keys[1].data_ptr(), offsets.data_ptr(), ptrs(layout), ws.data_ptr(), ws_bytes, ks, krs,
                                   _capi.stream_ptr()))
    torch.cuda.synchronize()
    assert _capi.dsb_row_binned(h, w)
    for v in range(nv):
        want_keys = torch.sort(unsorted[v]).values           # (depth bits, id): all distinct, depths positive
        assert torch.equal(keys[0, v], want_keys)
        ids = (want_keys & 0xFFFFFFFF)
        ry = records[v][:, 11].contiguous().view(torch.int32).to(torch.int64)
        height = torch.where(tiles[v].to(torch.int64) > 0, (ry >> 16) - (ry & 0xFFFF), torch.zeros_like(ry))
        count = tiles[v].to(torch.int64).clone()
        height[n - 1] = 0; count[n - 1] = 0                  # capi_camera() keeps the reference's dropped last splat
        in_order = (height if rows else count)[ids]
        want_off = torch.cumsum(in_order, 0) - in_order
        assert torch.equal(offsets[v].to(torch.int64), want_off)
        assert int(krs[v]) == (int(height.sum()) if rows else 0) and int(ks[v]) == int(count.sum())
        assert int(ranges[v][-1]) == int(ks[v])
        # the same view alone
        k1, kr1 = (C.c_int64 * 1)(), (C.c_int64 * 1)()
        key1 = torch.stack([unsorted[v], torch.empty_like(unsorted[v])])
        off1 = i32(n)
        _capi.check(lib.dsb_plan_views(C.byref(cams[v]), 1, n, n, ptrs([records[v]]), tiles[v].data_ptr(), key1[0].data_ptr(),
                                       key1[1].data_ptr(), off1.data_ptr(), ptrs([layout[v]]), ws.data_ptr(), ws_bytes, k1, kr1,
                                       _capi.stream_ptr()))
        assert int(k1[0]) == int(ks[v]) and int(kr1[0]) == int(krs[v])
        assert torch.equal(key1[0], keys[0, v]) and torch.equal(off1, offsets[v])
    # argument checks of the multi-view calls
    with pytest.raises(_capi.DsbError):
        _capi.check(lib.dsb_plan_views(C.byref(cams[0]), 9, n, n, ptrs(records), tiles.data_ptr(), keys[0].data_ptr(), keys[1].data_ptr(),
                                       offsets.data_ptr(), ptrs(layout), ws.data_ptr(), ws_bytes, ks, krs, _capi.stream_ptr()))
    with pytest.raises(_capi.DsbError):
        _capi.check(lib.dsb_plan_views(C.byref(cams[0]), nv, n, n, ptrs(records), tiles.data_ptr(), keys[0].data_ptr(), keys[1].data_ptr(),
                                       offsets.data_ptr(), ptrs(layout), ws.data_ptr(), 1024, ks, krs, _capi.stream_ptr()))
    if rows:   # row binning needs the records (for the rectangle heights) and the layout blocks (for the pair totals)
        with pytest.raises(_capi.DsbError):
            _capi.check(lib.dsb_plan_views(C.byref(cams[0]), nv, n, n, None, tiles.data_ptr(), keys[0].data_ptr(), keys[1].data_ptr(),
                                           offsets.data_ptr(), None, ws.data_ptr(), ws_bytes, ks, krs, _capi.stream_ptr()))


def test_adam_step_matches_the_checker_and_a_training_step_lowers_the_loss():
    from ds_splat_b200.dp import FlatAdam
    rng = np.random.default_rng(21)
    # the kernel alone: odd length (scalar tail) and an unaligned view (scalar path), three steps
    for count, offset in ((100_003, 0), (4_099, 1)):
        p0 = rng.normal(0, 1, count + offset).astype(np.float32)
        p = torch.from_numpy(p0.copy()).cuda()[offset:]
        m, v = torch.zeros_like(p), torch.zeros_like(p)
        po, mo, vo = p0[offset:].copy(), np.zeros(count, np.float32), np.zeros(count, np.float32)
        for step in (1, 2, 3):
            g = (rng.normal(0, 1e-2, count) * 10.0 ** rng.integers(-2, 2)).astype(np.float32)
            gt = torch.from_numpy(g).cuda()
            _capi.check(_capi.lib().dsb_adam_step(p.data_ptr(), gt.data_ptr(), m.data_ptr(), v.data_ptr(), count,
                                                  1e-3, 0.9, 0.999, 1e-15, step, 0.5, _capi.stream_ptr()))
            po, mo, vo = O.adam_step(po, g, mo, vo, lr=1e-3, eps=1e-15, step=step, grad_scale=0.5)
        torch.cuda.synchronize()
        np.testing.assert_allclose(p.cpu().numpy(), po, rtol=2e-6, atol=1e-8)
        np.testing.assert_allclose(m.cpu().numpy(), mo, rtol=1e-5, atol=1e-6 * float(np.abs(mo).max()))
        np.testing.assert_allclose(v.cpu().numpy(), vo, rtol=1e-5, atol=1e-6 * float(vo.max()))
    # a few optimisation steps towards a target image lower an L2 loss
    sc = scenes.tiny(n=5000, seed=41, W=192, H=128, focal=180.0)
    t = scene_tensors(sc)
    cam = CameraTensors.from_view(sc.views[0], "cuda")
    target = ViewRenderer(t["means"], t["shs"], t["opacities"], t["scales"], t["rotations"]).forward(cam).clone()
    params = dict(means3d=t["means"].clone(), shs=(t["shs"] * 0.5).contiguous(), opacities=t["opacities"].clone(),
                  scales=t["scales"].clone(), rotations=t["rotations"].clone())
    opt = FlatAdam(params, dict(means3d=0.0, shs=1e-2, opacities=0.0, scales=0.0, rotations=0.0))
    grads = GradientBuffer(sc.n, "cuda")
    losses = []
    for _ in range(6):
        r = ViewRenderer(params["means3d"], params["shs"], params["opacities"], params["scales"], params["rotations"])
        r.render_views([cam], lambda i, image: (losses.append(float(((image - target) ** 2).sum())), 2.0 * (image - target))[1],
                       grads)
        opt.step(grads)
    assert losses[-1] < 0.9 * losses[0] and all(np.isfinite(losses))


def test_image_loss_gradient_matches_the_autograd_checker():
    """dsb_image_loss_backward against oracle/loss_oracle.py (torch autograd in float64 on the CPU): ragged sizes that
    exercise the zero padding and partial tiles, both terms of the loss, and its use as the loss of render_views."""
    from ds_splat_b200.dp import ImageLoss
    from oracle import loss_oracle as L
    rng = np.random.default_rng(8)
    for (h, w), lam in (((37, 53), 0.2), ((64, 48), 1.0), ((19, 16), 0.0), ((130, 97), 0.2), ((131, 97), 0.0), ((256, 512), 0.0)):
        img = rng.uniform(0, 1, (h, w, 3)).astype(np.float32)
        tgt = np.clip(img + rng.normal(0, 0.1, img.shape), 0, 1).astype(np.float32)
        loss_o, grad_o = L.image_loss_and_grad(img, tgt, lam)
        v, loss = ImageLoss(lambda_dssim=lam).gradient(torch.from_numpy(img).cuda(), torch.from_numpy(tgt).cuda())
        torch.cuda.synchronize()
        assert abs(float(loss) - loss_o) <= 1e-5 * max(abs(loss_o), 1e-3)
        scale = float(np.abs(grad_o).max())
        assert float(np.abs(v.cpu().numpy() - grad_o).max()) <= 2e-4 * scale, (h, w, lam)
    # 8-bit targets (value / 255): the one-pass L1 entry point, and the conversion in front of the D-SSIM form
    for (h, w), lam in (((131, 97), 0.0), ((64, 64), 0.0), ((37, 53), 0.2)):
        img = rng.uniform(0, 1, (h, w, 3)).astype(np.float32)
        tgt8 = rng.integers(0, 256, (h, w, 3), dtype=np.uint8)
        loss_o, grad_o = L.image_loss_and_grad(img, tgt8.astype(np.float32) / np.float32(255.0), lam)
        v, loss = ImageLoss(lambda_dssim=lam).gradient(torch.from_numpy(img).cuda(), torch.from_numpy(tgt8).cuda())
        torch.cuda.synchronize()
        assert abs(float(loss) - loss_o) <= 1e-5 * max(abs(loss_o), 1e-3)
        scale = float(np.abs(grad_o).max())
        assert float(np.abs(v.cpu().numpy() - grad_o).max()) <= 2e-4 * scale, (h, w, lam, "u8")
    # as the loss of a multi-view step: the gradients equal those of a step fed with the checker's dL/dimage
    sc = scenes.headline(n=10_000, seed=99, W=240, H=144, focal=170.0, views=3, ring=True)
    t = scene_tensors(sc)
    cams = [CameraTensors.from_view(v, "cuda") for v in sc.views]
    targets = [torch.from_numpy(rng.uniform(0, 1, (144, 240, 3)).astype(np.float32)).cuda() for _ in cams]
    r = ViewRenderer(t["means"], t["shs"], t["opacities"], t["scales"], t["rotations"])
    loss_fn = ImageLoss(targets)
    g_fused = GradientBuffer(sc.n, "cuda")
    r.render_views(cams, loss_fn, g_fused)
    def checker_grad(i, image):
        _, g = L.image_loss_and_grad(image.cpu().numpy(), targets[i].cpu().numpy(), 0.2)
        return torch.from_numpy(g).cuda()
    g_check = GradientBuffer(sc.n, "cuda")
    r.render_views(cams, checker_grad, g_check)
    torch.cuda.synchronize()
    assert len(loss_fn.losses) == 3 and all(0.0 < float(l) < 1.5 for l in loss_fn.losses)
    # render_views runs neighbouring views on different streams: the loss keeps one set of buffers per stream
    side = torch.cuda.Stream()
    v_main, _ = loss_fn.gradient(targets[0], targets[1])
    with torch.cuda.stream(side):
        v_side, _ = loss_fn.gradient(targets[0], targets[1])
    side.synchronize()
    assert v_main.data_ptr() != v_side.data_ptr() and torch.equal(v_main, v_side)
    assert _rel(g_fused.views["shs"].cpu().numpy(), g_check.views["shs"].cpu().numpy()) < 1e-3
    assert _rel(g_fused.views["means3d"].cpu().numpy(), g_check.views["means3d"].cpu().numpy()) < 1e-3


def test_gradients_take_the_shape_of_non_canonical_inputs():
    """opacities given as [N] and shs flattened to [N, 48] render like the canonical shapes, and autograd receives
    gradients of exactly those shapes (the reference refuses such inputs with a TORCH_CHECK; here they are accepted)."""
    sc = scenes.tiny(n=3000, seed=72, W=160, H=128, focal=140.0)
    view = sc.views[0]
    t = scene_tensors(sc)
    rast = GaussianRasterizer(settings_for(view))
    v = torch.from_numpy(sc.image_grad()).cuda()
    canon = {k: x.clone().requires_grad_(True) for k, x in t.items()}
    img, _ = rast(canon["means"], None, canon["shs"], None, canon["opacities"], canon["scales"], canon["rotations"], None)
    img.backward(v)
    flat = {k: x.clone() for k, x in t.items()}
    flat["opacities"] = flat["opacities"].reshape(-1)
    flat["shs"] = flat["shs"].reshape(sc.n, 48)
    flat = {k: x.requires_grad_(True) for k, x in flat.items()}
    img2, _ = rast(flat["means"], None, flat["shs"], None, flat["opacities"], flat["scales"], flat["rotations"], None)
    assert torch.equal(img2, img)
    img2.backward(v)
    torch.cuda.synchronize()
    assert flat["opacities"].grad.shape == (sc.n,) and flat["shs"].grad.shape == (sc.n, 48)
    assert _rel(flat["opacities"].grad.cpu().numpy(), canon["opacities"].grad.reshape(-1).cpu().numpy()) < 1e-4
    assert _rel(flat["shs"].grad.cpu().numpy(), canon["shs"].grad.reshape(sc.n, 48).cpu().numpy()) < 1e-4


def test_operator_reuses_its_pair_buffers_from_the_previous_count():
    """The second call of a shape brings pair buffers sized from the first call's count, so plan and render run inside
    one library call; a view with many more pairs than the hint still renders correctly (buffers are grown)."""
    sc = scenes.headline(n=30_000, seed=73, W=400, H=240, focal=260.0, views=3, ring=True)
    t = scene_tensors(sc)
    imgs = []
    for rep in range(2):
        for v in sc.views:
            img, _ = GaussianRasterizer(settings_for(v))(t["means"], None, t["shs"], None, t["opacities"], t["scales"],
                                                        t["rotations"], None)
            imgs.append(img.clone())
    torch.cuda.synchronize()
    for a, b in zip(imgs[:3], imgs[3:]):
        assert torch.equal(a, b)
    # a much heavier view of the same shape (scales x4): the hint is too small, the operator grows the buffers
    big = t["scales"] * 4.0
    img_big, _ = GaussianRasterizer(settings_for(sc.views[0]))(t["means"], None, t["shs"], None, t["opacities"], big,
                                                              t["rotations"], None)
    r = ViewRenderer(t["means"], t["shs"], t["opacities"], big, t["rotations"], batch_views=1)
    assert torch.equal(img_big, r.forward(CameraTensors.from_view(sc.views[0], "cuda")))


@pytest.mark.parametrize("tight", [False, True])
def test_row_binning_builds_the_same_list_ranges_image_and_gradients(tight):
    """DSB_FLAG_ROW_BINNING changes how the fused render gets from depth-ordered splats to the sorted pair list (row
    items + one pass over the pairs instead of writing the pairs and sorting them); list, ranges, image and gradients
    must not change.  Ragged image size, a multi-view step, and a scene whose last tiles are empty."""
    sc = scenes.headline(n=60_000, seed=74, W=500, H=297, focal=300.0, views=3, ring=True)
    t = scene_tensors(sc)
    cams = [CameraTensors.from_view(v, "cuda") for v in sc.views]
    vimgs = [torch.from_numpy(sc.image_grad(i)).cuda() for i in range(len(sc.views))]
    out = {}
    for rows in (False, True):
        r = ViewRenderer(t["means"], t["shs"], t["opacities"], t["scales"], t["rotations"], tight_tiles=tight, row_binning=rows)
        image = r.forward(cams[0]).clone()
        k = r.last_k
        assert (r.last_k_rows > 0) == rows
        single = (image, r.pairs[:k].clone(), r._ranges(r.cur, sc.views[0].H, sc.views[0].W).clone(), k)
        g = GradientBuffer(sc.n, "cuda")
        r.render_views(cams, vimgs, g)
        torch.cuda.synchronize()
        assert _capi.take_device_status() == 0
        out[rows] = single + (g.flat.clone(), list(r.last_ks))
    a, b = out[False], out[True]
    assert a[3] == b[3] and a[3] > 0 and a[5] == b[5]
    assert torch.equal(a[1], b[1]) and torch.equal(a[2], b[2]) and torch.equal(a[0], b[0])
    assert _rel(b[4].cpu().numpy(), a[4].cpu().numpy()) < 1e-4
