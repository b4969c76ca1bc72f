"""The bounded waits inside the kernels, made to run out on purpose in the one safe form: a predecessor that is never
processed, a poll limit of a few hundred, well-formed inputs.  The starved block gives up, records
DSB_ERR_DEVICE_WAIT_EXPIRED and finishes like the others; the test checks that the kernel returns, that the host is
told through the same calls that would tell it in production, and that the device keeps working afterwards.  Nothing
here faults, traps or spins without a limit."""
import ctypes as C

import numpy as np
import pytest

from conftest import capi_camera, scene_tensors

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from ds_splat_b200 import _capi, scenes  # noqa: E402

WAIT_EXPIRED = -5


def _sorts_correctly_afterwards():
    g = torch.Generator(device="cuda").manual_seed(5)
    items = torch.randint(0, 1 << 40, (100_000,), generator=g, device="cuda", dtype=torch.int64)
    got = _capi.sort_pairs(items.clone(), 32, 40)
    key = (items >> 32) & 0xFF
    want = items[torch.sort(key, stable=True).indices]
    assert torch.equal(got, want)


def test_scan_wait_runs_out_and_the_plan_read_back_reports_it():
    sc = scenes.tiny(n=5000, seed=31, W=320, H=208, focal=260.0)
    t = scene_tensors(sc)
    cam, keep = capi_camera(sc.views[0])
    records, radii, tiles, cov3d, depth_keys = _capi.preprocess(cam, t["means"], t["shs"], t["opacities"], t["scales"], t["rotations"])
    lib = _capi.lib()
    n = sc.n
    ws_bytes = int(lib.dsb_plan_workspace_bytes(n))
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    offsets = torch.empty(n, dtype=torch.int32, device="cuda")
    _capi.check(lib.dsb_debug_expire_scan_wait(C.byref(cam), n, tiles.data_ptr(), depth_keys.data_ptr(), offsets.data_ptr(),
                                               ws.data_ptr(), ws_bytes, 200, _capi.stream_ptr()))
    k = (C.c_int64 * 1)()
    rc = lib.dsb_plan_totals_views(1, n, ws.data_ptr(), ws_bytes, k, None, _capi.stream_ptr())
    assert rc == WAIT_EXPIRED
    assert "wait expired" in lib.dsb_last_error().decode()
    # the read-back took the device's status word with it: the next check is clean, and a real plan works
    assert _capi.take_device_status() == 0
    offsets2, k2 = _capi.plan_pairs(cam, tiles, depth_keys)
    assert k2 == int(tiles[:-1].sum().item())
    _sorts_correctly_afterwards()


def test_sort_wait_runs_out_and_the_status_word_reports_it():
    g = torch.Generator(device="cuda").manual_seed(6)
    k = 3 * 4096 + 17
    items = torch.randint(0, 1 << 40, (k,), generator=g, device="cuda", dtype=torch.int64)
    alt = torch.zeros_like(items)
    lib = _capi.lib()
    ws_bytes = int(lib.dsb_sort_workspace_bytes(k))
    ws = torch.empty(ws_bytes + 256, dtype=torch.uint8, device="cuda")
    _capi.check(lib.dsb_debug_expire_sort_wait(items.data_ptr(), alt.data_ptr(), k, 32, 40, ws.data_ptr(), ws_bytes, 300,
                                               _capi.stream_ptr()))
    with pytest.raises(_capi.DsbError) as info:
        _capi.take_device_status()
    assert info.value.code == WAIT_EXPIRED
    assert _capi.take_device_status() == 0          # taken: cleared
    torch.cuda.synchronize()
    _sorts_correctly_afterwards()
    # argument checks of the hook itself: more than one pass, a list of one tile, an unbounded limit
    assert lib.dsb_debug_expire_sort_wait(items.data_ptr(), alt.data_ptr(), k, 32, 45, ws.data_ptr(), ws_bytes, 300, None) == -1
    assert lib.dsb_debug_expire_sort_wait(items.data_ptr(), alt.data_ptr(), 4096, 32, 40, ws.data_ptr(), ws_bytes, 300, None) == -1
    assert lib.dsb_debug_expire_sort_wait(items.data_ptr(), alt.data_ptr(), k, 32, 40, ws.data_ptr(), ws_bytes, 1 << 30, None) == -1


def test_preprocess_blocks_that_give_up_on_their_bulk_copies_read_the_rows_themselves():
    sc = scenes.tiny(n=256 * 40 + 7, seed=32, W=320, H=208, focal=260.0)   # full blocks (bulk copies) and a partial one
    t = scene_tensors(sc)
    cam, keep = capi_camera(sc.views[0])
    want = _capi.preprocess(cam, t["means"], t["shs"], t["opacities"], t["scales"], t["rotations"])
    assert _capi.take_device_status() == 0
    lib = _capi.lib()
    try:
        _capi.check(lib.dsb_debug_set_copy_wait_polls(1))    # one poll: the copies cannot have landed yet
        got = _capi.preprocess(cam, t["means"], t["shs"], t["opacities"], t["scales"], t["rotations"])
        status = _capi.take_device_status()
    finally:
        _capi.check(lib.dsb_debug_set_copy_wait_polls(0))
    for a, b in zip(got, want):
        assert torch.equal(a, b)          # same rows, read with plain loads: bit-identical records, radii, keys
    assert status in (0, 1)               # 1 = DSB_STATUS_COPY_WAIT_FELL_BACK; 0 if every copy beat the single poll
    assert _capi.take_device_status() == 0
