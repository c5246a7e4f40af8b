"""Online activation quantisation (the definition in
``src/orbitquant/functional.py:9-22``), computed by the fused CUDA prologue.

``n = ||x||``; ``u = x/(n+eps)``; ``r = u @ R``; ``x_q = centroid[bucketize(r)] * n`` in
``x.dtype``.  No calibration data: the only inputs are the seeded rotation and the
closed-form codebook.
"""
from __future__ import annotations

import torch

from . import native
from .codebooks import LloydMaxCodebook
from .rotations import RPBHRotation


def quantize_activations(x: torch.Tensor, *, rotation: RPBHRotation, codebook: LloydMaxCodebook,
                         eps: float) -> torch.Tensor:
    if x.shape[-1] != rotation.dim:
        raise ValueError(f"expected last dimension {rotation.dim}, got {x.shape[-1]}")
    return native.quantize_activations(
        x, rotation.permutation, rotation.signs, codebook.centroids, codebook.boundaries,
        eps=eps, block_size=rotation.block_size)
