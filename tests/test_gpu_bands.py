"""Views with more (tile, splat) pairs than one list may hold (2^30 - 1; the reference's own 32-bit pair count wraps at
2^31, cpp/rasterizer_torch.cu:101-107) are rendered in bands of tile rows.  Checked two ways: on a scene small enough
to render in one piece, bands against no bands (image, transmittance and last contributors bit for bit, gradients up
to the order of the atomic sums); and on a scene just past the limit -- the high-overlap stress configuration with its
scales raised until it holds about 1.2e9 pairs -- through what must hold at any size: every band under the limit, the
bands' pair counts adding up to the exact total the whole-image plan reported, and two different band splits
rendering the same image bit for bit."""
import numpy as np
import pytest

from conftest import scene_tensors

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from ds_splat_b200 import _capi, scenes  # noqa: E402
from ds_splat_b200.dp import CameraTensors, GradientBuffer, ViewRenderer  # noqa: E402


@pytest.mark.parametrize("tight", [False, True])
def test_bands_render_what_one_list_renders(tight):
    sc = scenes.headline(n=120_000, seed=75, W=960, H=544, focal=560.0)
    view = sc.views[0]
    t = scene_tensors(sc)
    cam = CameraTensors.from_view(view, "cuda")
    v = torch.from_numpy(sc.image_grad()).cuda()
    r = ViewRenderer(t["means"], t["shs"], t["opacities"], t["scales"], t["rotations"], batch_views=1, tight_tiles=tight,
                     strict_reference=False)
    image = r.forward(cam).clone()
    k = r.last_k
    _, final_t, final_idx = (x.clone() for x in r._image_buffers(view.H, view.W))
    g = GradientBuffer(sc.n, "cuda")
    r.backward(v, g, accumulate=False)
    torch.cuda.synchronize()

    rb = ViewRenderer(t["means"], t["shs"], t["opacities"], t["scales"], t["rotations"], batch_views=1, tight_tiles=tight,
                      strict_reference=False)
    image_b = rb.forward_banded(cam, max_pairs=k // 3 + 1)
    assert len(rb.bands) >= 3 and all(kb <= k // 3 + 1 for _, _, kb in rb.bands)
    assert sum(kb for _, _, kb in rb.bands) == k                         # the bands partition the pairs
    assert [b[0] for b in rb.bands] == [0] + [b[1] for b in rb.bands[:-1]] and rb.bands[-1][1] == (view.H + 15) // 16
    assert torch.equal(image_b, image)
    _, final_t_b, final_idx_b = rb._image_buffers(view.H, view.W)
    assert torch.equal(final_t_b, final_t)
    # last contributors are positions in a band's own list: compare the splats they name
    gb = GradientBuffer(sc.n, "cuda")
    gb.flat.fill_(7.0)
    rb.backward_banded(v, gb, accumulate=False)
    torch.cuda.synchronize()
    assert _capi.take_device_status() == 0
    scale = float(g.flat.abs().max())
    assert float((gb.flat - g.flat).abs().max()) <= 1e-4 * scale
    # a limit nothing exceeds: one band, the ordinary path
    rb.forward_banded(cam)
    assert rb.bands == [(0, (view.H + 15) // 16, k)]


def test_a_view_just_past_the_pair_limit_renders_in_bands():
    sc = scenes.stress(log_scale_mu=-2.65)          # about 1.2e9 pairs at 1920x1080
    view = sc.views[0]
    t = scene_tensors(sc)
    cam = CameraTensors.from_view(view, "cuda")
    r = ViewRenderer(t["means"], t["shs"], t["opacities"], t["scales"], t["rotations"], batch_views=1, tight_tiles=False)
    total, _, rc = r._plan_band(r._slot(0), cam, None)      # the whole image: refused, but counted exactly
    assert rc == _capi.DSB_ERR_TOO_MANY_PAIRS and total > _capi.MAX_PAIRS
    with pytest.raises(_capi.DsbError):
        r.forward(cam)
    image = r.forward_banded(cam).clone()
    bands = list(r.bands)
    assert len(bands) >= 2 and all(kb < _capi.MAX_PAIRS for _, _, kb in bands)
    assert sum(kb for _, _, kb in bands) == total
    assert bool(torch.isfinite(image).all()) and float(image.max()) > 0.1
    g = GradientBuffer(sc.n, "cuda")
    r.backward_banded(torch.from_numpy(sc.image_grad()).cuda(), g, accumulate=False)
    torch.cuda.synchronize()
    assert _capi.take_device_status() == 0
    assert bool(torch.isfinite(g.flat).all()) and float(g.flat.abs().max()) > 0
    # another split of the same view: finer bands, same image
    image2 = r.forward_banded(cam, max_pairs=total // 5)
    assert len(r.bands) > len(bands)
    assert torch.equal(image2, image)
