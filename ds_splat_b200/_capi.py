"""ctypes binding of ``libdsb200.so`` (C ABI declared in ``include/dsb200.h``) plus thin per-stage
wrappers that take torch CUDA tensors.  torch is used for device memory and the current stream only.

The library is mandatory: importing a stage on a machine where ``libdsb200.so`` has not been built
raises ``RuntimeError`` -- there is no CPU or PyTorch fallback for any stage.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
# DSB200_LIBRARY points at a libdsb200.so built elsewhere (default: the in-tree build next to this file).
LIB_PATH = os.environ.get("DSB200_LIBRARY") or os.path.join(_HERE, "libdsb200.so")

DSB_FLAG_DROP_LAST_SPLAT = 1
DSB_FLAG_TIGHT_TILES = 2
DSB_FLAG_ROW_BINNING = 4
RECORD_FLOATS = 12
GRAD_FLOATS = 12
MAX_BATCH_VIEWS = 8
MAX_PAIRS = 1 << 30
LAYOUT_WORDS = 1024   # per-view layout block of the fused render
DSB_ERR_TOO_MANY_PAIRS = -4

EXPORTS = (
    "dsb_last_error", "dsb_version", "dsb_launch_count", "dsb_plan_workspace_bytes", "dsb_sort_workspace_bytes",
    "dsb_preprocess", "dsb_plan_pairs", "dsb_emit_pairs", "dsb_sort_pairs", "dsb_sort_by_keys",
    "dsb_identify_tile_ranges", "dsb_blend_forward", "dsb_blend_backward", "dsb_geometry_backward",
    "dsb_forward_plan", "dsb_forward_render", "dsb_backward", "dsb_preprocess_views", "dsb_plan_workspace_bytes_views", "dsb_plan_views", "dsb_plan_totals_views",
    "dsb_render_workspace_bytes", "dsb_row_binning_supported",
    "dsb_backward_blend",
    "dsb_geometry_backward_views", "dsb_geometry_backward_views_stats",
    "dsb_forward_core", "dsb_image_loss_workspace_bytes", "dsb_image_loss_backward", "dsb_l1_loss_backward_u8", "dsb_adam_step",
    "dsb_export_reference_lists",
    "dsb_stage_timing_enable", "dsb_stage_count", "dsb_stage_name", "dsb_stage_timing_read",
    "dsb_sort_pairs_static", "dsb_tile_marks_bytes", "dsb_forward", "dsb_take_device_status",
    "dsb_debug_expire_scan_wait", "dsb_debug_expire_sort_wait", "dsb_debug_set_copy_wait_polls",
    "dsb_debug_blend_forward_variant",
)
STATIC_SORT_MAX_ITEMS = 1 << 21


class DsbCamera(C.Structure):
    _fields_ = [("image_height", C.c_int32), ("image_width", C.c_int32), ("tanfovx", C.c_float), ("tanfovy", C.c_float),
                ("scale_modifier", C.c_float), ("sh_degree", C.c_int32), ("max_sh_degree", C.c_int32),
                ("matrices_transposed", C.c_int32), ("flags", C.c_int32), ("tile_row_band", C.c_int32),
                ("viewmatrix", C.c_void_p), ("projmatrix", C.c_void_p), ("campos", C.c_void_p), ("bg", C.c_void_p)]


class DsbError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"dsb200 error {code}: {message}")
        self.code = code


_lib = None


def lib():
    """Load the shared library once; fail loudly when it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} not found: build it with `python -m ds_splat_b200.build` (needs nvcc); "
                "this package has no fallback path")
        l = C.CDLL(LIB_PATH)
        l.dsb_last_error.restype = C.c_char_p
        l.dsb_version.restype = C.c_int32
        l.dsb_launch_count.restype = C.c_int64
        l.dsb_plan_workspace_bytes.restype = C.c_int64
        l.dsb_plan_workspace_bytes.argtypes = [C.c_int32]
        l.dsb_image_loss_workspace_bytes.restype = C.c_int64
        l.dsb_image_loss_workspace_bytes.argtypes = [C.c_int32, C.c_int32]
        l.dsb_plan_workspace_bytes_views.restype = C.c_int64
        l.dsb_plan_workspace_bytes_views.argtypes = [C.c_int32, C.c_int32]
        l.dsb_sort_workspace_bytes.restype = C.c_int64
        l.dsb_sort_workspace_bytes.argtypes = [C.c_int64]
        l.dsb_tile_marks_bytes.restype = C.c_int64
        l.dsb_tile_marks_bytes.argtypes = [C.c_int32, C.c_int32]
        l.dsb_render_workspace_bytes.restype = C.c_int64
        l.dsb_render_workspace_bytes.argtypes = [C.c_int32, C.c_int32, C.c_int64, C.c_int64]
        l.dsb_row_binning_supported.restype = C.c_int32
        l.dsb_row_binning_supported.argtypes = [C.c_int32, C.c_int32]
        l.dsb_stage_name.restype = C.c_char_p
        l.dsb_stage_name.argtypes = [C.c_int32]
        l.dsb_stage_count.restype = C.c_int32
        l.dsb_stage_timing_enable.argtypes = [C.c_int32]
        P, I32, I64, CAM = C.c_void_p, C.c_int32, C.c_int64, C.POINTER(DsbCamera)
        sig = {
            "dsb_preprocess": [CAM, I32] + [P] * 7 + [P] * 5 + [P],
            "dsb_plan_pairs": [CAM, I32, P, P, P, P, P, I64, C.POINTER(C.c_int64), P],
            "dsb_emit_pairs": [CAM, I32, I64, P, P, P, P, P, P],
            "dsb_sort_pairs": [P, P, I64, I32, I32, P, I64, C.POINTER(C.c_int32), P],
            "dsb_sort_by_keys": [P, P, P, P, I64, I32, I32, P, I64, C.POINTER(C.c_int32), P],
            "dsb_sort_pairs_static": [P, P, I64, I32, I32, C.POINTER(C.c_int32), P],
            "dsb_identify_tile_ranges": [P, I64, I32, I32, P, P],
            "dsb_blend_forward": [CAM, P, P, P, P, P, P, P, P],
            "dsb_blend_backward": [CAM, P, P, P, P, P, P, P, P, P],
            "dsb_geometry_backward": [CAM, I32] + [P] * 7 + [P] * 8 + [I32, P],
            "dsb_forward_plan": [CAM, I32] + [P] * 7 + [P] * 10 + [P, I64, C.POINTER(C.c_int64), C.POINTER(C.c_int64), P],
            "dsb_forward_render": [CAM, I32, I64, I64] + [P] * 8 + [P, I64] + [P] * 4 + [P],
            "dsb_backward": [CAM, I32] + [P] * 14 + [P] * 8 + [I32, P],
            "dsb_preprocess_views": [P, I32, I32] + [P] * 16,
            "dsb_plan_views": [CAM, I32, I32, I64, P, P, P, P, P, P, P, I64, P, P, P],
            "dsb_plan_totals_views": [I32, I32, P, I64, P, P, P],
            "dsb_backward_blend": [CAM, I32] + [P] * 9 + [I32, P],
            "dsb_geometry_backward_views": [P, I32, I32] + [P] * 15 + [I32, P],
            "dsb_geometry_backward_views_stats": [P, I32, I32] + [P] * 15 + [I32, C.c_float, C.c_float, P, P, P, P],
            "dsb_forward_core": [P, P, P, P, P, I32, P, P, P, I32, I32, C.c_float, C.c_float, C.c_float, I32, I32, P, P],
            "dsb_image_loss_backward": [P, P, I32, I32, C.c_float, P, I64, P, P, P],
            "dsb_l1_loss_backward_u8": [P, P, I32, I32, P, P, P],
            "dsb_adam_step": [P, P, P, P, I64, C.c_double, C.c_double, C.c_double, C.c_double, I32, C.c_double, P],
            "dsb_export_reference_lists": [P, I64, P, P, P, P],
            "dsb_forward": [CAM, I32] + [P] * 7 + [P] * 10 + [P, I64] + [P, I64] + [P, I64] + [P] * 4
                           + [C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_int32), P],
            "dsb_take_device_status": [C.POINTER(C.c_int32), P],
            "dsb_debug_expire_scan_wait": [CAM, I32, P, P, P, P, I64, C.c_uint32, P],
            "dsb_debug_expire_sort_wait": [P, P, I64, I32, I32, P, I64, C.c_uint32, P],
            "dsb_debug_set_copy_wait_polls": [C.c_uint32],
            "dsb_debug_blend_forward_variant": [CAM, I32, I32, I64, P, P, P, P, P, P, P, P, I64, P],
        }
        for name, argtypes in sig.items():
            fn = getattr(l, name)
            fn.restype = C.c_int
            fn.argtypes = argtypes
        _lib = l
    return _lib


def check(rc: int):
    if rc != 0:
        raise DsbError(rc, lib().dsb_last_error().decode(errors="replace"))


def take_device_status() -> int:
    """Synchronises the current stream and hands over the device's status word: raises ``DsbError`` when a bounded
    wait inside a kernel expired since the last check (lists sorted since are not valid), returns a positive
    DSB_STATUS_* note or 0 otherwise."""
    status = C.c_int32(0)
    check(lib().dsb_take_device_status(C.byref(status), stream_ptr()))
    return int(status.value)


def launch_count() -> int:
    return int(lib().dsb_launch_count())


def stage_timing(enable: bool):
    check(lib().dsb_stage_timing_enable(1 if enable else 0))


def read_stage_timings():
    """Returns {stage name: (total ms, calls)} for the stages recorded since timing was enabled."""
    n = int(lib().dsb_stage_count())
    ms = (C.c_double * n)()
    calls = (C.c_int64 * n)()
    check(lib().dsb_stage_timing_read(n, ms, calls))
    return {lib().dsb_stage_name(i).decode(): (float(ms[i]), int(calls[i])) for i in range(n)}


def ptr(t):
    """Device address of a tensor (None and empty tensors map to NULL)."""
    if t is None or t.numel() == 0:
        return None
    return t.data_ptr()


def stream_ptr(device=None):
    """Handle of torch's current stream -- of ``device`` when given, which must then be the current device: the
    library launches on the current device, so a stream of another one would take the kernels to the wrong GPU."""
    if device is not None:
        device = torch.device(device)
        if device.type != "cuda":
            raise RuntimeError(f"the rasterizer runs on CUDA devices, not on {device}")
        index = device.index if device.index is not None else torch.cuda.current_device()
        if index != torch.cuda.current_device():
            raise RuntimeError(f"tensors live on cuda:{index} but the current device is cuda:{torch.cuda.current_device()}; "
                               "wrap the call in torch.cuda.device(...)")
    return torch.cuda.current_stream().cuda_stream


def as_f32(t, device, name):
    """float32, contiguous, on ``device`` -- the requirements the reference checks with TORCH_CHECK
    (cpp/rasterizer_torch.cu:13-17,176-190); non-contiguous inputs are made contiguous instead of refused."""
    if t is None:
        return None
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if t.numel() == 0:
        return None
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if t.device != device:
        raise RuntimeError(f"{name} is on {t.device}, expected {device}")
    if t.dtype != torch.float32:
        raise RuntimeError(f"{name} must be float32")
    return t.contiguous()


def make_camera(image_height, image_width, tanfovx, tanfovy, viewmatrix, projmatrix, campos, bg=None, sh_degree=3,
                max_sh_degree=3, scale_modifier=1.0, transposed=True, drop_last=True, tight_tiles=False, row_binning=False):
    """Build a DsbCamera; returns (struct, keepalive list)."""
    cam = DsbCamera()
    cam.image_height, cam.image_width = int(image_height), int(image_width)
    cam.tanfovx, cam.tanfovy, cam.scale_modifier = float(tanfovx), float(tanfovy), float(scale_modifier)
    cam.sh_degree, cam.max_sh_degree = int(sh_degree), int(max_sh_degree)
    cam.matrices_transposed = 1 if transposed else 0
    cam.flags = ((DSB_FLAG_DROP_LAST_SPLAT if drop_last else 0) | (DSB_FLAG_TIGHT_TILES if tight_tiles else 0)
                 | (DSB_FLAG_ROW_BINNING if row_binning else 0))
    cam.viewmatrix, cam.projmatrix, cam.campos = viewmatrix.data_ptr(), projmatrix.data_ptr(), campos.data_ptr()
    cam.bg = bg.data_ptr() if bg is not None else None
    return cam, [viewmatrix, projmatrix, campos, bg]


def dsb_row_binned(h, w) -> bool:
    """Whether an image of this size is within the limits of row binning (at most 256 x 509 tiles)."""
    return bool(lib().dsb_row_binning_supported(int(h), int(w)))


def num_tiles(h, w):
    return ((w + 15) // 16) * ((h + 15) // 16)


# ---- per-stage wrappers (used by the tests and the benchmark's per-stage timers) -------------------------

def preprocess(cam, means3d, shs, opacities, scales, rotations, colors_precomp=None, cov3d_precomp=None):
    n, dev = means3d.shape[0], means3d.device
    records = torch.empty((n, RECORD_FLOATS), dtype=torch.float32, device=dev)
    radii = torch.empty(n, dtype=torch.int32, device=dev)
    tiles = torch.empty(n, dtype=torch.int32, device=dev)
    cov3d = cov3d_precomp if cov3d_precomp is not None else torch.empty((n, 6), dtype=torch.float32, device=dev)
    depth_keys = torch.empty(n, dtype=torch.int64, device=dev)
    check(lib().dsb_preprocess(C.byref(cam), n, ptr(means3d), ptr(shs), ptr(colors_precomp), ptr(opacities), ptr(scales),
                               ptr(rotations), ptr(cov3d_precomp), ptr(records), ptr(radii), ptr(tiles), ptr(cov3d),
                               ptr(depth_keys), stream_ptr()))
    return records, radii, tiles, cov3d, depth_keys


def preprocess_views(cams, means3d, shs, opacities, scales, rotations):
    """One preprocess launch for several cameras of one image size; returns a list of per-view
    (records, radii, tiles, depth_keys, tile_marks) and the shared cov3d."""
    n, dev, nv = means3d.shape[0], means3d.device, len(cams)
    h, w = cams[0].image_height, cams[0].image_width
    out = []
    for _ in range(nv):
        out.append((torch.empty((n, RECORD_FLOATS), dtype=torch.float32, device=dev),
                    torch.empty(n, dtype=torch.int32, device=dev), torch.empty(n, dtype=torch.int32, device=dev),
                    torch.empty(n, dtype=torch.int64, device=dev),
                    torch.empty(int(lib().dsb_tile_marks_bytes(h, w)), dtype=torch.uint8, device=dev)))
    cov3d = torch.empty((n, 6), dtype=torch.float32, device=dev)
    arr = lambda i: (C.c_void_p * nv)(*[o[i].data_ptr() for o in out])
    check(lib().dsb_preprocess_views((DsbCamera * nv)(*cams), nv, n, ptr(means3d), ptr(shs), None, ptr(opacities),
                                     ptr(scales), ptr(rotations), None, arr(0), arr(1), arr(2), ptr(cov3d), arr(3), arr(4),
                                     None, None, stream_ptr()))
    return out, cov3d


def plan_pairs(cam, tiles, depth_keys):
    """Sorts depth_keys in place; returns (offsets, K)."""
    n, dev = tiles.shape[0], tiles.device
    alt = torch.empty_like(depth_keys)
    offsets = torch.empty(n, dtype=torch.int32, device=dev)
    ws_bytes = int(lib().dsb_plan_workspace_bytes(n))
    ws = torch.empty(ws_bytes + 256, dtype=torch.uint8, device=dev)
    k = C.c_int64(0)
    check(lib().dsb_plan_pairs(C.byref(cam), n, ptr(tiles), ptr(depth_keys), ptr(alt), ptr(offsets), ws.data_ptr(),
                               ws_bytes, C.byref(k), stream_ptr()))
    return offsets, int(k.value)


def emit_pairs(cam, k, records, tiles, depth_keys_sorted, offsets):
    n = tiles.shape[0]
    pairs = torch.empty(k, dtype=torch.int64, device=tiles.device)
    check(lib().dsb_emit_pairs(C.byref(cam), n, k, ptr(records), ptr(tiles), ptr(depth_keys_sorted), ptr(offsets),
                               ptr(pairs), stream_ptr()))
    return pairs


def sort_pairs(items, begin_bit, end_bit):
    """Stable radix sort of int64 words on bits [begin_bit, end_bit) (unsigned digit order); returns the sorted tensor."""
    k = items.shape[0]
    alt = torch.empty_like(items)
    ws_bytes = int(lib().dsb_sort_workspace_bytes(k))
    ws = torch.empty(ws_bytes + 256, dtype=torch.uint8, device=items.device)
    in_alt = C.c_int32(0)
    check(lib().dsb_sort_pairs(ptr(items), ptr(alt), k, begin_bit, end_bit, ws.data_ptr(), ws_bytes, C.byref(in_alt),
                               stream_ptr()))
    take_device_status()   # the sort never synchronises by itself; this wrapper does, and reports an expired wait
    return alt if in_alt.value else items


def sort_pairs_static(items, items_alt, begin_bit, end_bit):
    """Same sort as sort_pairs() for callers that cannot allocate device memory when they need it (a plug-in inside
    another engine's frame loop, a loop where cudaMalloc's device-wide stall is unacceptable): the scratch is a fixed
    array inside the library, so the entry point itself allocates nothing -- which is why ``items_alt``, an int64
    tensor as long as ``items``, must be supplied by the caller here.  At most STATIC_SORT_MAX_ITEMS items; calls on
    one device must not overlap on the GPU.  Returns whichever of the two tensors holds the sorted list."""
    in_alt = C.c_int32(0)
    check(lib().dsb_sort_pairs_static(ptr(items), ptr(items_alt), items.shape[0], begin_bit, end_bit, C.byref(in_alt),
                                      stream_ptr()))
    take_device_status()   # allocates nothing either: one 4-byte copy to the host and a stream synchronisation
    return items_alt if in_alt.value else items


def sort_by_keys(keys, values, begin_bit=0, end_bit=64):
    """(int64 key, int32 value) pair sort, the reference's sort_by_keys interface; returns (keys, values)."""
    k = keys.shape[0]
    kalt, valt = torch.empty_like(keys), torch.empty_like(values)
    ws_bytes = int(lib().dsb_sort_workspace_bytes(k))
    ws = torch.empty(ws_bytes + 256, dtype=torch.uint8, device=keys.device)
    in_alt = C.c_int32(0)
    check(lib().dsb_sort_by_keys(ptr(keys), ptr(kalt), ptr(values), ptr(valt), k, begin_bit, end_bit, ws.data_ptr(),
                                 ws_bytes, C.byref(in_alt), stream_ptr()))
    take_device_status()
    return (kalt, valt) if in_alt.value else (keys, values)


def identify_tile_ranges(sorted_items, h, w):
    ranges = torch.empty(num_tiles(h, w) + 1, dtype=torch.int32, device=sorted_items.device)
    check(lib().dsb_identify_tile_ranges(ptr(sorted_items), sorted_items.shape[0], h, w, ptr(ranges), stream_ptr()))
    return ranges


def blend_forward(cam, records, sorted_pairs, ranges, with_depth=False):
    """Returns (image, final_T, final_idx), plus the blended depth map when ``with_depth``."""
    h, w, dev = cam.image_height, cam.image_width, records.device
    depth = torch.empty((h, w), dtype=torch.float32, device=dev) if with_depth else None
    image = torch.empty((h, w, 3), dtype=torch.float32, device=dev)
    final_t = torch.empty((h, w), dtype=torch.float32, device=dev)
    final_idx = torch.empty((h, w), dtype=torch.int32, device=dev)
    check(lib().dsb_blend_forward(C.byref(cam), ptr(records), ptr(sorted_pairs), ptr(ranges), ptr(image), ptr(final_t),
                                  ptr(final_idx), ptr(depth), stream_ptr()))
    return (image, final_t, final_idx, depth) if with_depth else (image, final_t, final_idx)


def blend_backward(cam, records, sorted_pairs, ranges, final_t, final_idx, v_image, v_depth=None):
    n = records.shape[0]
    grad_acc = torch.zeros((n, GRAD_FLOATS), dtype=torch.float32, device=records.device)
    check(lib().dsb_blend_backward(C.byref(cam), ptr(records), ptr(sorted_pairs), ptr(ranges), ptr(final_t),
                                   ptr(final_idx), ptr(v_image), ptr(v_depth), ptr(grad_acc), stream_ptr()))
    return grad_acc


def geometry_backward(cam, means3d, scales, rotations, records, cov3d, radii, grad_acc, num_coeff=16, accumulate=False,
                      out=None):
    n, dev = means3d.shape[0], means3d.device
    if out is None:
        mk = lambda *s: torch.empty(s, dtype=torch.float32, device=dev)
        out = dict(v_means3d=mk(n, 3), v_means2d=mk(n, 3), v_shs=mk(n, num_coeff, 3), v_colors=mk(n, 3),
                   v_opacities=mk(n, 1), v_scales=mk(n, 3), v_rotations=mk(n, 4), v_cov3d=mk(n, 6))
    check(lib().dsb_geometry_backward(C.byref(cam), n, ptr(means3d), ptr(scales), ptr(rotations), ptr(records), ptr(cov3d),
                                      ptr(radii), ptr(grad_acc), ptr(out["v_means3d"]), ptr(out["v_means2d"]),
                                      ptr(out["v_shs"]), ptr(out["v_colors"]), ptr(out["v_opacities"]),
                                      ptr(out["v_scales"]), ptr(out["v_rotations"]), ptr(out["v_cov3d"]),
                                      1 if accumulate else 0, stream_ptr()))
    return out


def export_reference_lists(sorted_pairs, records):
    k = sorted_pairs.shape[0]
    keys = torch.empty(k, dtype=torch.int64, device=records.device)
    ids = torch.empty(k, dtype=torch.int32, device=records.device)
    check(lib().dsb_export_reference_lists(ptr(sorted_pairs), k, ptr(records), ptr(keys), ptr(ids), stream_ptr()))
    return keys, ids
