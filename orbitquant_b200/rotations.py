"""RPBH: randomized permuted block-Hadamard rotation (host-side constants).

``R = P . diag(s) . blockdiag(H_B) / sqrt(B)``: a global permutation of the ``dim``
input channels, Rademacher signs, then an independent Walsh-Hadamard transform on
every contiguous block of ``B`` channels.  Activations and weight rows are rotated by
the same ``R`` so ``x W^T = (xR)(WR)^T``.

The permutation and signs are part of the weight format: they are drawn from one CPU
``torch.Generator`` seeded with ``seed`` -- first ``randperm(dim)``, then
``randint(0, 2, (dim,))`` -- exactly as ``src/orbitquant/rotations/rpbh.py:55-63``
does, so packed weights produced by either implementation are interchangeable.
``block_size="paper"`` is the largest power of two dividing ``dim`` (``rpbh.py:13-17``).

The device-side application of R lives in the CUDA prologue kernel; the torch
implementation here is only used offline (weight quantisation) and by tests.
"""
from __future__ import annotations

import math
import warnings
from functools import lru_cache

import torch


def is_power_of_two(value: int) -> bool:
    return value > 0 and value & (value - 1) == 0


def paper_block_size(dim: int) -> int:
    block = 1
    while dim % (block * 2) == 0:
        block *= 2
    return block


def fwht(x: torch.Tensor) -> torch.Tensor:
    """Unnormalised Walsh-Hadamard transform over the last dimension.

    Stages h = 1, 2, 4, ... each map pairs ``(l, r)`` at distance h to
    ``(l + r, l - r)`` -- the same pairs and order as every implementation of the
    reference (``src/orbitquant/rotations/fwht.py:10-26``), which keeps fp32 results
    bit-identical across host and device."""
    n = x.shape[-1]
    if not is_power_of_two(n):
        raise ValueError("FWHT last dimension must be a power of two")
    shape = x.shape
    y = x.contiguous().reshape(-1, n)
    h = 1
    while h < n:
        v = y.reshape(-1, n // (2 * h), 2, h)
        lo, hi = v[:, :, 0, :], v[:, :, 1, :]
        y = torch.stack((lo + hi, lo - hi), dim=2).reshape(-1, n)
        h *= 2
    return y.reshape(shape)


class RPBHRotation:
    """Holds ``permutation`` (int64), ``inverse_permutation``, ``signs`` (int8, +-1),
    ``block_size``, ``num_blocks`` and ``normalization = 1/sqrt(block_size)``."""

    def __init__(self, dim: int, seed: int = 0, block_size: int | str = "paper") -> None:
        if dim <= 0:
            raise ValueError("dim must be positive")
        if block_size == "paper":
            block_size = paper_block_size(dim)
            if block_size == 1:
                warnings.warn(
                    "RPBH paper block-size policy selected block_size=1; rotation "
                    "degenerates to signs/permutation only.", RuntimeWarning, stacklevel=2)
        if not isinstance(block_size, int):
            raise TypeError("block_size must be an int or 'paper'")
        if block_size <= 0:
            raise ValueError("block_size must be positive")
        if not is_power_of_two(block_size):
            raise ValueError("block_size must be a power of two")
        if dim % block_size != 0:
            raise ValueError("block_size must divide dim")
        gen = torch.Generator(device="cpu")
        gen.manual_seed(int(seed))
        perm = torch.randperm(dim, generator=gen, dtype=torch.long, device="cpu")
        signs = torch.randint(0, 2, (dim,), generator=gen, dtype=torch.int8, device="cpu")
        inverse = torch.empty_like(perm)
        inverse[perm] = torch.arange(dim, dtype=torch.long)
        self.dim = dim
        self.seed = int(seed)
        self.block_size = block_size
        self.num_blocks = dim // block_size
        self.permutation = perm
        self.inverse_permutation = inverse
        self.signs = signs * 2 - 1
        self.normalization = 1.0 / math.sqrt(block_size)

    def _check(self, x: torch.Tensor) -> None:
        if x.shape[-1] != self.dim:
            raise ValueError(f"expected last dimension {self.dim}, got {x.shape[-1]}")

    def apply_to_activations(self, x: torch.Tensor) -> torch.Tensor:
        """``x @ R`` for row vectors (``rpbh.py:73-84``)."""
        self._check(x)
        y = x.index_select(-1, self.permutation.to(x.device)) * self.signs.to(x.device, x.dtype)
        y = fwht(y.reshape(*y.shape[:-1], self.num_blocks, self.block_size)) * self.normalization
        return y.reshape(x.shape)

    def apply_to_weight(self, weight: torch.Tensor) -> torch.Tensor:
        if weight.ndim != 2:
            raise ValueError("weight must be a rank-2 tensor")
        if weight.shape[-1] != self.dim:
            raise ValueError(f"expected in_features {self.dim}, got {weight.shape[-1]}")
        return self.apply_to_activations(weight)

    def apply_inverse_to_activations(self, x: torch.Tensor) -> torch.Tensor:
        """``x @ R^T`` (``rpbh.py:95-105``): H is symmetric, so undo in reverse order."""
        self._check(x)
        y = fwht(x.reshape(*x.shape[:-1], self.num_blocks, self.block_size)) * self.normalization
        y = y.reshape(x.shape) * self.signs.to(x.device, x.dtype)
        return y.index_select(-1, self.inverse_permutation.to(x.device))

    def apply_inverse_to_weight(self, weight: torch.Tensor) -> torch.Tensor:
        if weight.ndim != 2:
            raise ValueError("weight must be a rank-2 tensor")
        return self.apply_inverse_to_activations(weight)


@lru_cache(maxsize=256)
def get_rpbh_rotation(dim: int, seed: int = 0, block_size: int | str = "paper") -> RPBHRotation:
    return RPBHRotation(dim=dim, seed=seed, block_size=block_size)


def clear_rotation_cache() -> None:
    get_rpbh_rotation.cache_clear()
