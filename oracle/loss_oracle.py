"""Checker for the photometric loss that sits between the forward and the backward of the operator in a training
loop (test infrastructure, like everything under oracle/).

Not a restatement of a reference file: the reference has no loss.  It is the loss 3-D Gaussian Splatting training
uses, L = (1 - lambda) * mean|x - y| + lambda * (1 - mean SSIM(x, y)), with SSIM as published (Wang et al., 2004):
per channel, 11x11 Gaussian window of sigma 1.5, zero padding, C1 = 0.01^2, C2 = 0.03^2.  Written with plain torch
operations on the CPU in float64, and differentiated by autograd, so that the hand-derived gradient of the CUDA
kernels is checked against an independent one.
"""
import numpy as np
import torch
import torch.nn.functional as F


def _window(size: int = 11, sigma: float = 1.5) -> torch.Tensor:
    g = torch.tensor([np.exp(-((i - size // 2) ** 2) / (2.0 * sigma ** 2)) for i in range(size)], dtype=torch.float64)
    g = g / g.sum()
    return (g[:, None] * g[None, :])[None, None]


def image_loss(image: torch.Tensor, target: torch.Tensor, lambda_dssim: float = 0.2) -> torch.Tensor:
    """image, target: [H, W, 3]; returns the scalar loss (float64)."""
    x = image.permute(2, 0, 1)[None].double()
    y = target.permute(2, 0, 1)[None].double()
    w = _window().expand(3, 1, 11, 11)
    conv = lambda t: F.conv2d(t, w, padding=5, groups=3)
    m1, m2 = conv(x), conv(y)
    s11, s22, s12 = conv(x * x) - m1 * m1, conv(y * y) - m2 * m2, conv(x * y) - m1 * m2
    c1, c2 = 0.01 ** 2, 0.03 ** 2
    ssim = ((2 * m1 * m2 + c1) * (2 * s12 + c2)) / ((m1 * m1 + m2 * m2 + c1) * (s11 + s22 + c2))
    return (1.0 - lambda_dssim) * (x - y).abs().mean() + lambda_dssim * (1.0 - ssim.mean())


def image_loss_and_grad(image: np.ndarray, target: np.ndarray, lambda_dssim: float = 0.2):
    """numpy [H, W, 3] in; returns (loss as float, dL/dimage as float32 numpy [H, W, 3])."""
    x = torch.from_numpy(np.ascontiguousarray(image, dtype=np.float32)).double().requires_grad_(True)
    y = torch.from_numpy(np.ascontiguousarray(target, dtype=np.float32)).double()
    loss = image_loss(x, y, lambda_dssim)
    loss.backward()
    return float(loss.detach()), x.grad.numpy().astype(np.float32)
