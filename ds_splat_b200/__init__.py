"""B200-native (sm_100a) Gaussian-splat rasterizer with the ds-splat operator surface.

    from ds_splat_b200 import GaussianRasterizationSettings, GaussianRasterizer

mirrors ``from ds_splat import ...`` of the reference (ds_splat/__init__.py:1-4).
"""
from .rasterizer import DsRasterizerFunction, GaussianRasterizationSettings, GaussianRasterizer

__all__ = ["GaussianRasterizationSettings", "GaussianRasterizer", "DsRasterizerFunction"]
