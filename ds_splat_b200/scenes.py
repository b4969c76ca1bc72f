"""Seeded synthetic splat clouds and cameras for the benchmark and the parity tests.

The reference's published plots use trained Mip-NeRF-360 scenes that are not redistributable here; these
generators produce clouds with the same sizes (20k .. 6M splats, 640x480 .. 3840x2160) and the value
distributions of a trained model: log-normal scales, normalised random quaternions, sigmoid opacities,
degree-3 spherical harmonics with a strong DC band.  Everything is generated on the host with numpy's
PCG64 so the CPU checker and the GPU see identical bits.

Camera convention (the one graphdeco-style callers of ``GaussianRasterizer`` use): the camera looks
down +z, x right, y down; ``viewmatrix`` is the transposed world->camera matrix and ``projmatrix`` the
transposed full projection, exactly what ``GaussianRasterizationSettings`` expects
(ds_splat/rasterizer.py:115-129,147-148 transposes them back before the kernels read them).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np

ZNEAR, ZFAR = 0.01, 100.0


def look_at(eye, target, down=(0.0, 1.0, 0.0)) -> np.ndarray:
    """Row-major 4x4 world->camera matrix [R|t] for a camera at ``eye`` looking at ``target``."""
    eye, target, down = (np.asarray(v, np.float64) for v in (eye, target, down))
    f = target - eye
    f /= np.linalg.norm(f)
    x = np.cross(down, f)
    x /= np.linalg.norm(x)
    y = np.cross(f, x)
    m = np.eye(4)
    m[0, :3], m[1, :3], m[2, :3] = x, y, f
    m[:3, 3] = -m[:3, :3] @ eye
    return m.astype(np.float32)


def perspective(tanfovx: float, tanfovy: float, znear: float = ZNEAR, zfar: float = ZFAR) -> np.ndarray:
    """Row-major 4x4 perspective matrix with w = z_view and z_ndc in [0, 1]."""
    p = np.zeros((4, 4), np.float64)
    p[0, 0] = 1.0 / tanfovx
    p[1, 1] = 1.0 / tanfovy
    p[3, 2] = 1.0
    p[2, 2] = zfar / (zfar - znear)
    p[2, 3] = -(zfar * znear) / (zfar - znear)
    return p.astype(np.float32)


@dataclass
class View:
    """One camera.  ``view``/``proj`` are row-major (world->camera, P*V); the ``*_t`` properties give the
    transposed arrays that go into ``GaussianRasterizationSettings``."""
    H: int
    W: int
    tanfovx: float
    tanfovy: float
    view: np.ndarray
    proj: np.ndarray
    campos: np.ndarray

    @property
    def viewmatrix_t(self) -> np.ndarray:
        return np.ascontiguousarray(self.view.T)

    @property
    def projmatrix_t(self) -> np.ndarray:
        return np.ascontiguousarray(self.proj.T)

    @property
    def num_tiles(self) -> int:
        return ((self.W + 15) // 16) * ((self.H + 15) // 16)


def make_view(eye, target, W: int, H: int, focal: float) -> View:
    tanx, tany = W / (2.0 * focal), H / (2.0 * focal)
    v = look_at(eye, target)
    p = (perspective(tanx, tany).astype(np.float64) @ v.astype(np.float64)).astype(np.float32)
    return View(H=H, W=W, tanfovx=float(tanx), tanfovy=float(tany), view=v, proj=p,
                campos=np.asarray(eye, np.float32))


@dataclass
class Scene:
    name: str
    means: np.ndarray       # [N,3]
    scales: np.ndarray      # [N,3]  (already exponentiated)
    rotations: np.ndarray   # [N,4]  (w,x,y,z), unit norm
    opacities: np.ndarray   # [N,1]
    shs: np.ndarray         # [N,16,3]
    views: list = field(default_factory=list)
    sh_degree: int = 3
    note: str = ""

    @property
    def n(self) -> int:
        return int(self.means.shape[0])

    def image_grad(self, view_index: int = 0, seed: int = 7) -> np.ndarray:
        """Upstream dL/dimage ~ N(0, 1e-3), shape [H,W,3]."""
        v = self.views[view_index]
        rng = np.random.default_rng(seed * 7919 + view_index)
        return (rng.standard_normal((v.H, v.W, 3), dtype=np.float32) * np.float32(1e-3))


def _appearance(rng, n: int, log_scale_mu: float, log_scale_sigma: float, opacity_mu: float):
    scales = np.exp(rng.standard_normal((n, 3), dtype=np.float32) * np.float32(log_scale_sigma)
                    + np.float32(log_scale_mu)).astype(np.float32)
    q = rng.standard_normal((n, 4), dtype=np.float32)
    q /= np.linalg.norm(q, axis=1, keepdims=True)
    logits = rng.standard_normal((n, 1), dtype=np.float32) + np.float32(opacity_mu)
    opac = (1.0 / (1.0 + np.exp(-logits))).astype(np.float32)
    shs = rng.standard_normal((n, 16, 3), dtype=np.float32)
    shs[:, 0, :] *= np.float32(0.5)
    shs[:, 1:, :] *= np.float32(0.05)
    return scales, q.astype(np.float32), opac, shs


def _cluster_means(rng, n: int, clusters: int = 64, box: float = 4.0, sigma: float = 0.3) -> np.ndarray:
    centres = rng.uniform(-box, box, size=(clusters, 3)).astype(np.float32)
    which = rng.integers(0, clusters, size=n)
    return (centres[which] + rng.standard_normal((n, 3), dtype=np.float32) * np.float32(sigma)).astype(np.float32)


def ring_views(count: int, radius: float, W: int, H: int, focal: float, seed: int) -> list:
    """Cameras on a circle of ``radius`` in the xz-plane looking at the origin, pitch jittered by +-5 deg."""
    rng = np.random.default_rng(seed)
    out = []
    for k in range(count):
        a = 2.0 * math.pi * k / count
        pitch = math.radians(float(rng.uniform(-5.0, 5.0)))
        eye = (radius * math.sin(a) * math.cos(pitch), radius * math.sin(pitch), -radius * math.cos(a) * math.cos(pitch))
        out.append(make_view(eye, (0.0, 0.0, 0.0), W, H, focal))
    return out


def jittered_views(count: int, radius: float, W: int, H: int, focal: float, seed: int, degrees: float = 5.0) -> list:
    """``count`` cameras at ``radius`` from the origin looking at it: the first is the canonical one on the -z axis,
    the others are turned away from it by yaw and pitch angles drawn from U[-degrees, degrees] (seeded)."""
    rng = np.random.default_rng(seed)
    out = [make_view((0.0, 0.0, -radius), (0.0, 0.0, 0.0), W, H, focal)]
    for _ in range(1, count):
        yaw, pitch = (math.radians(float(a)) for a in rng.uniform(-degrees, degrees, size=2))
        eye = (radius * math.sin(yaw) * math.cos(pitch), radius * math.sin(pitch), -radius * math.cos(yaw) * math.cos(pitch))
        out.append(make_view(eye, (0.0, 0.0, 0.0), W, H, focal))
    return out


def tiny(n: int = 20_000, seed: int = 1000, W: int = 640, H: int = 480, focal: float = 600.0) -> Scene:
    """Config 0: uniform box [-2,2]^3, camera at z=-5 looking +z."""
    rng = np.random.default_rng(seed)
    means = rng.uniform(-2.0, 2.0, size=(n, 3)).astype(np.float32)
    sc, q, op, sh = _appearance(rng, n, -3.5, 0.5, 0.0)
    return Scene("c0_tiny", means, sc, q, op, sh, [make_view((0, 0, -5.0), (0, 0, 0), W, H, focal)])


def headline(n: int = 1_000_000, seed: int = 1001, W: int = 1920, H: int = 1080, focal: float = 1100.0,
             views: int = 1, ring: bool = False) -> Scene:
    """Config 1: 64 isotropic clusters (sigma 0.3) in [-4,4]^3, camera 6 units from the origin.  ``views`` > 1 adds
    cameras around the first one (pose jittered by +-5 degrees; view 0 stays the configuration's own camera), or a
    full ring of cameras with ``ring``."""
    rng = np.random.default_rng(seed)
    means = _cluster_means(rng, n)
    sc, q, op, sh = _appearance(rng, n, -3.5, 0.5, 0.0)
    if views > 1 and ring:
        vs = ring_views(views, 6.0, W, H, focal, seed + 17)
    else:
        vs = jittered_views(max(1, views), 6.0, W, H, focal, seed + 17)
    return Scene("c1_headline", means, sc, q, op, sh, vs)


def plane4k(n: int = 3_000_000, seed: int = 1002, W: int = 3840, H: int = 2160, focal: float = 2200.0) -> Scene:
    """Config 2: 70% of the splats on a thin ground plane, 30% in a central ball; camera raised 30 deg."""
    rng = np.random.default_rng(seed)
    n_plane = int(0.7 * n)
    plane = np.stack([rng.uniform(-5, 5, n_plane), rng.uniform(-0.05, 0.05, n_plane), rng.uniform(-5, 5, n_plane)], 1)
    d = rng.standard_normal((n - n_plane, 3))
    d /= np.linalg.norm(d, axis=1, keepdims=True)
    ball = d * (2.0 * rng.uniform(0, 1, (n - n_plane, 1)) ** (1.0 / 3.0))
    means = np.concatenate([plane, ball], 0).astype(np.float32)
    sc, q, op, sh = _appearance(rng, n, -4.0, 0.7, 0.0)
    eye = (0.0, -6.0 * math.sin(math.radians(30)), -6.0 * math.cos(math.radians(30)))
    return Scene("c2_plane4k", means, sc, q, op, sh, [make_view(eye, (0, 0, 0), W, H, focal)])


def multiview(n: int = 6_000_000, seed: int = 1003, views: int = 64, W: int = 1920, H: int = 1080,
              focal: float = 1100.0) -> Scene:
    """Config 3: config 1's mixture at 6M splats seen from a ring of cameras."""
    rng = np.random.default_rng(seed)
    means = _cluster_means(rng, n)
    sc, q, op, sh = _appearance(rng, n, -3.5, 0.5, 0.0)
    return Scene("c3_multiview", means, sc, q, op, sh, ring_views(views, 6.0, W, H, focal, seed + 17))


def stress(n: int = 2_000_000, seed: int = 1004, W: int = 1920, H: int = 1080, focal: float = 1100.0,
           log_scale_mu: float = -4.0) -> Scene:
    """Config 4: unit cube two units in front of the camera, low opacity (sigmoid(N(-2,1))).

    The default ``log_scale_mu=-4.0`` yields about 1e8 (tile, splat) pairs, the count the config's own
    description quotes; its literal scale law N(-2, 0.5) yields more than 2^31 pairs, which overflows the
    reference's 32-bit pair count and is rejected by this library with a clear error."""
    rng = np.random.default_rng(seed)
    means = np.stack([rng.uniform(-0.5, 0.5, n), rng.uniform(-0.5, 0.5, n), rng.uniform(1.5, 2.5, n)], 1).astype(np.float32)
    sc, q, op, sh = _appearance(rng, n, log_scale_mu, 0.5, -2.0)
    return Scene("c4_stress", means, sc, q, op, sh, [make_view((0, 0, 0), (0, 0, 1.0), W, H, focal)],
                 note=f"log-scale mean {log_scale_mu}")


CONFIGS = {"c0": tiny, "c1": headline, "c2": plane4k, "c3": multiview, "c4": stress}
