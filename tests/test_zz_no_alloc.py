"""The allocation-free sort entry point, dsb_sort_pairs_static, through the C ABI.

It exists for callers that cannot get device memory at the moment they need a sort -- a renderer living as a
plug-in in another engine's frame loop that owns all GPU memory, or a loop where cudaMalloc's device-wide stall is
not acceptable -- so its scratch is a fixed array inside the library.  The test checks that it produces exactly the
list dsb_sort_pairs produces and the list an independent stable sort (torch.sort) produces on the same bits (integer
work: bit-exact), on two calls in a row with different sizes and bit ranges,
so that leftovers of the first call in the shared array would show up in the second, and that lists beyond the
built-in limit are refused with a clear error.  This file sorts last in collection order on purpose: with
``pytest -x`` every other test has already run when it starts.
"""
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from ds_splat_b200 import _capi  # noqa: E402


def _random_pairs(k, tiles, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    tile = torch.randint(0, tiles, (k,), generator=g, device="cuda", dtype=torch.int64)
    ident = torch.randint(0, 1 << 31, (k,), generator=g, device="cuda", dtype=torch.int64)
    return (tile << 32) | ident


def test_static_sort_matches_workspace_sort_on_two_calls_in_a_row():
    cases = [(1_234_567, 8160, 32, 45, 1), (50_001, 200, 32, 40, 2)]  # (items, tiles, begin_bit, end_bit, seed)
    got = None
    for k, tiles, b0, b1, seed in cases:
        got = None  # drop the previous result now, so that freeing it is not mistaken for a change below
        pairs = _random_pairs(k, tiles, seed)
        want = _capi.sort_pairs(pairs.clone(), b0, b1)
        work, alt = pairs.clone(), torch.empty_like(pairs)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        got = _capi.sort_pairs_static(work, alt, b0, b1)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before  # nothing was taken from torch's allocator either
        assert torch.equal(got, want)
        # ... and the list an independent stable sort on the same bits produces (equal digits keep their input order)
        digit = (pairs >> b0) & ((1 << (b1 - b0)) - 1)
        assert torch.equal(got, pairs[torch.sort(digit, stable=True).indices])


def test_static_sort_refuses_lists_beyond_its_limit():
    lib = _capi.lib()
    import ctypes as C
    flag = C.c_int32(5)
    rc = lib.dsb_sort_pairs_static(None, None, _capi.STATIC_SORT_MAX_ITEMS + 1, 32, 45, C.byref(flag), None)
    assert rc == -3 and flag.value == 0
    msg = lib.dsb_last_error().decode()
    assert "at most" in msg and str(_capi.STATIC_SORT_MAX_ITEMS) in msg
    # the largest allowed size works
    k = _capi.STATIC_SORT_MAX_ITEMS
    pairs = _random_pairs(k, 32400, 3)
    want = _capi.sort_pairs(pairs.clone(), 32, 47)
    got = _capi.sort_pairs_static(pairs.clone(), torch.empty_like(pairs), 32, 47)
    assert torch.equal(got, want)
