"""Multi-rank host logic of the data-parallel step, on CPU with the gloo backend (world_size 2):
view sharding, the flat gradient buffer and the all-reduce.  The per-view gradients come from the CPU
checker on a tiny scene, so the assertion is the real property: the all-reduced buffer of the sharded
run equals the serial sum over all views."""
import os
import socket

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402

from ds_splat_b200 import dp, scenes  # noqa: E402


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class OracleRenderer:
    """Stands in for ViewRenderer on CPU: same forward / backward / render_views protocol, gradients from the
    CPU checker."""

    def __init__(self, scene):
        from oracle import oracle as O
        self.O, self.sc = O, scene

    def forward(self, view):
        O, sc = self.O, self.sc
        self.cam = O.Camera(view=view.view, proj=view.proj, campos=view.campos, tanfovx=view.tanfovx, tanfovy=view.tanfovy,
                            H=view.H, W=view.W, sh_degree=3)
        self.fwd = O.forward(self.cam, sc.means, sc.shs, sc.opacities, sc.scales, sc.rotations)
        return self.fwd["image"]

    def backward(self, v_image, grads, accumulate=True, stats=None):
        sc = self.sc
        b = self.O.backward(self.cam, self.fwd, sc.means, sc.shs, sc.opacities, sc.scales, sc.rotations, v_image.numpy())
        if stats is not None:
            stats.add_view(torch.from_numpy(b["v_means2d"]), torch.from_numpy(self.fwd["pre"]["radii"]), self.cam.H, self.cam.W)
        pairs = (("means3d", "v_means3d"), ("shs", "v_shs"), ("opacities", "v_opacities"), ("scales", "v_scales"),
                 ("rotations", "v_rotations"))
        for dst, src in pairs:
            g = torch.from_numpy(b[src])
            if accumulate:
                grads.views[dst] += g
            else:
                grads.views[dst].copy_(g)

    def render_views(self, cameras, image_grads, grads, accumulate=False, stats=None):
        for idx, view in enumerate(cameras):
            image = self.forward(view)
            v_image = image_grads(idx, image) if callable(image_grads) else image_grads[idx]
            self.backward(v_image, grads, accumulate=accumulate or idx > 0, stats=stats)


def _scene():
    return scenes.headline(n=1500, seed=9, W=96, H=64, focal=60.0, views=5, ring=True)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sc = _scene()
    mine = dp.shard_views(len(sc.views), rank, world)
    grads = dp.GradientBuffer(sc.n, "cpu")
    grads.flat.fill_(123.0)  # stale contents must not leak into the result
    stats = dp.DensifyStats(sc.n, "cpu", ndc_units=True)
    dp.data_parallel_step(OracleRenderer(sc), [sc.views[i] for i in mine],
                          [torch.from_numpy(sc.image_grad(i)) for i in mine], grads, stats=stats)
    stats.allreduce()   # what the ranks do once before they densify
    if rank == 0:
        np.save(out, grads.flat.numpy())
        np.save(out + ".stats.npy", stats.flat.numpy())
    dist.destroy_process_group()


def test_shard_views_partition():
    for world in (1, 2, 3, 8):
        seen = sorted(i for r in range(world) for i in dp.shard_views(11, r, world))
        assert seen == list(range(11))
    assert dp.shard_views(3, 5, 8) == []
    with pytest.raises(ValueError):
        dp.shard_views(4, 2, 2)


def test_gradient_buffer_layout():
    g = dp.GradientBuffer(7, "cpu")
    assert g.flat.numel() == 7 * dp.FLOATS_PER_SPLAT == 7 * 59 and g.nbytes() == 7 * 236
    assert g.views["shs"].shape == (7, 16, 3) and g.views["rotations"].shape == (7, 4)
    g.views["opacities"].fill_(2.0)
    assert float(g.flat.sum()) == 14.0
    assert g.views["means3d"].data_ptr() == g.flat.data_ptr()


def test_two_rank_step_equals_serial_sum(tmp_path):
    out = str(tmp_path / "rank0.npy")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    got = np.load(out)
    sc = _scene()
    serial = dp.GradientBuffer(sc.n, "cpu")
    serial_stats = dp.DensifyStats(sc.n, "cpu", ndc_units=True)
    r = OracleRenderer(sc)
    for i, v in enumerate(sc.views):
        r.forward(v)
        r.backward(torch.from_numpy(sc.image_grad(i)), serial, accumulate=i > 0, stats=serial_stats)
    np.testing.assert_allclose(got, serial.flat.numpy(), rtol=1e-5, atol=1e-9)
    assert np.abs(got).max() > 0
    # densification statistics: sums and visibility counts add over ranks, the largest radius is a maximum
    got_stats = np.load(out + ".stats.npy")
    np.testing.assert_allclose(got_stats, serial_stats.flat.numpy(), rtol=1e-5, atol=1e-9)
    assert got_stats[1].max() >= 2 and got_stats[2].max() > 0 and got_stats[0].max() > 0
    mean = serial_stats.mean_grad_norm().numpy()
    assert np.all(mean[got_stats[1] == 0] == 0) and np.isfinite(mean).all()


# ---- sharded optimizer step: reduce-scatter -> Adam on 1/G -> all-gather ----------------------------------------

def _checker_update(p, g, m, v, lr, beta1, beta2, eps, step, grad_scale):
    """The per-slice Adam update on CPU tensors, through the checker's restatement (oracle.adam_step)."""
    from oracle import oracle as O
    pn, mn, vn = O.adam_step(p.numpy(), g.numpy(), m.numpy(), v.numpy(), lr=lr, beta1=beta1, beta2=beta2, eps=eps, step=step,
                             grad_scale=grad_scale)
    p.copy_(torch.from_numpy(pn)); m.copy_(torch.from_numpy(mn)); v.copy_(torch.from_numpy(vn))


LRS = dict(means3d=1e-3, shs=2e-3, opacities=3e-3, scales=4e-3, rotations=5e-3)
N_SHARDED = 37   # odd on purpose: 37 * 59 elements do not split into equal slices without padding


def _rank_gradients(rank, step):
    g = torch.Generator().manual_seed(100 * step + rank)
    return torch.randn(N_SHARDED * 59, generator=g)


def _initial_parameters():
    g = torch.Generator().manual_seed(7)
    return dict(means3d=torch.randn(N_SHARDED, 3, generator=g), shs=torch.randn(N_SHARDED, 16, 3, generator=g),
                opacities=torch.rand(N_SHARDED, 1, generator=g), scales=torch.rand(N_SHARDED, 3, generator=g),
                rotations=torch.randn(N_SHARDED, 4, generator=g))


def _sharded_worker(rank, world, port, out, chunks=1):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    params = dp.ParameterBuffer.from_tensors(_initial_parameters(), shards=world * chunks)
    grads = dp.GradientBuffer(N_SHARDED, "cpu", shards=world * chunks)
    # a second group as the pipelined form takes it; on CPU ranks the chunks simply run one after the other
    second = dist.new_group(backend="gloo") if chunks > 1 else None
    opt = dp.ShardedAdam(params, LRS, eps=1e-8, update=_checker_update, chunks=chunks, gather_group=second)
    assert opt.m.numel() * world == params.storage.numel()       # moments: 1/G per rank
    assert len(opt.slices) == chunks and not opt.pipelined()
    for step in (1, 2, 3):
        grads.flat.copy_(_rank_gradients(rank, step))
        opt.step(grads, grad_scale=0.5)
    np.save(f"{out}.{rank}.npy", params.flat.numpy())
    dist.destroy_process_group()


@pytest.mark.parametrize("chunks", [1, 3])
def test_sharded_adam_on_two_ranks_equals_allreduce_plus_full_adam(tmp_path, chunks):
    out = str(tmp_path / "params")
    world = 2
    mp.spawn(_sharded_worker, args=(world, _free_port(), out, chunks), nprocs=world, join=True)
    got = [np.load(f"{out}.{r}.npy") for r in range(world)]
    np.testing.assert_array_equal(got[0], got[1])        # every rank ends with the same parameters
    # replicated form in one process: sum of the ranks' gradients, Adam over everything
    params = dp.ParameterBuffer.from_tensors(_initial_parameters())
    m, v = torch.zeros(params.length), torch.zeros(params.length)
    for step in (1, 2, 3):
        total = sum(_rank_gradients(r, step) for r in range(world))
        for name, _ in dp.SEGMENTS:
            a, b = params.segments[name]
            _checker_update(params.flat[a:b], total[a:b], m[a:b], v[a:b], LRS[name], 0.9, 0.999, 1e-8, step, 0.5)
    np.testing.assert_allclose(got[0], params.flat.numpy(), rtol=1e-6, atol=1e-7)
    assert np.abs(got[0] - dp.ParameterBuffer.from_tensors(_initial_parameters()).flat.numpy()).max() > 1e-3


def test_sharded_adam_in_one_process_is_plain_adam():
    params = dp.ParameterBuffer.from_tensors(_initial_parameters())
    grads = dp.GradientBuffer(N_SHARDED, "cpu")
    opt = dp.ShardedAdam(params, LRS, eps=1e-8, update=_checker_update)
    assert opt.world == 1 and [p[0] for p in opt.pieces] == [n for n, _ in dp.SEGMENTS]
    grads.flat.copy_(_rank_gradients(0, 1))
    before = params.flat.clone()
    opt.step(grads)
    assert float((params.flat - before).abs().max()) > 0
    with pytest.raises(ValueError, match="laid out differently"):
        opt.step(dp.GradientBuffer(N_SHARDED + 1, "cpu"))
