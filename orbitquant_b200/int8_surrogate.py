"""INT8 code tables for the integer (surrogate) W4A4 / W2A4 matmul.

The reference's fastest CUDA path does not multiply centroids: it maps both index streams
through small INT8 tables, contracts integers and rescales
(``src/orbitquant/layers.py:1097-1352``).  The tables are a symmetric INT8 rounding of the
codebook centroids whose scale is chosen by a 3001-point grid search around ``max|c| / 127``
(``src/orbitquant/kernels/triton_cuda.py:1826-1857``); restated here in the same float64
torch expressions, so codes and scale are identical to the reference's.
"""
from __future__ import annotations

from functools import lru_cache

import torch


def fit_int8_centroid_surrogate(centroids: torch.Tensor) -> tuple[torch.Tensor, float]:
    """``(int8 codes [levels], scale)`` with ``codes * scale ~ centroids``; 4, 8, 16 or 64
    centroids (2-, 3-, 4- and 6-bit codebooks)."""
    values = centroids.detach().to(device="cpu", dtype=torch.float64).flatten()
    if values.numel() not in (4, 8, 16, 64):
        raise ValueError("the INT8 centroid surrogate requires 4, 8, 16, or 64 centroids; "
                         f"got {values.numel()}")
    codes, scale = _fit(tuple(float(v) for v in values))
    return codes.clone(), scale


@lru_cache(maxsize=64)
def _fit(values: tuple[float, ...]) -> tuple[torch.Tensor, float]:
    v = torch.tensor(values, dtype=torch.float64)
    peak = float(v.abs().max())
    if peak == 0.0:
        return torch.zeros(len(values), dtype=torch.int8), 1.0
    scales = (peak / 127.0) * torch.linspace(0.5, 2.0, 3001, dtype=torch.float64)
    codes = torch.round(v[None, :] / scales[:, None]).clamp(-127, 127)
    errors = (codes * scales[:, None] - v[None, :]).square().mean(dim=1)
    best = int(errors.argmin())
    return codes[best].to(torch.int8), float(scales[best])
