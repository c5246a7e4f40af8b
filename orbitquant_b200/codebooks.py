"""Unit-sphere Lloyd-Max codebooks (host side, run once per ``(dim, bits)``).

A coordinate of a uniformly random point on ``S^{dim-1}`` has density proportional to
``(1 - t^2)^((dim-3)/2)`` on ``(-1, 1)``; ``t^2`` is ``Beta(1/2, (dim-1)/2)``.  The
codebook is the fixed point of Lloyd's iteration for that marginal: ``2^bits``
symmetric centroids, boundaries at the midpoints.  Quantising is
``index = #{boundaries < value}`` (ties go low), i.e. ``torch.bucketize``.

Bit-for-bit agreement with the reference generator is part of the weight-format
contract (packed indices are meaningless without the same centroids), so the float64
arithmetic follows ``src/orbitquant/codebooks/lloyd_max.py:267-448`` step by step:
Lentz continued fraction for the regularised incomplete beta, 96-step bisection for
the starting quantiles, Lloyd updates with 1.9x over-relaxation, stop at 1e-13.
The legacy grid codebook (version 1, ``lloyd_max.py:226-264``) is restated too because
artifacts written before codebook versioning load with ``codebook_version=1``
(``src/orbitquant/config.py:202-212``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from functools import lru_cache

import torch

SUPPORTED_VERSIONS = (1, 2)

_CF_EPS = 3e-14
_CF_TINY = 1e-300


@dataclass(frozen=True)
class LloydMaxCodebook:
    dim: int
    bits: int
    centroids: torch.Tensor  # float32 [2**bits], ascending, symmetric
    boundaries: torch.Tensor  # float32 [2**bits - 1], midpoints
    algorithm_version: int = 2

    def quantize_indices(self, values: torch.Tensor) -> torch.Tensor:
        edges = self.boundaries.to(device=values.device, dtype=values.dtype)
        return torch.bucketize(values, edges).to(torch.uint8)

    def quantize(self, values: torch.Tensor) -> torch.Tensor:
        table = self.centroids.to(device=values.device, dtype=values.dtype)
        return table[self.quantize_indices(values).to(torch.long)]


def _guard(value: float) -> float:
    return _CF_TINY if abs(value) < _CF_TINY else value


def _betacf(a: float, b: float, x: float) -> float:
    """Modified Lentz evaluation of the incomplete-beta continued fraction."""
    apb, ap1, am1 = a + b, a + 1.0, a - 1.0
    c = 1.0
    d = 1.0 / _guard(1.0 - apb * x / ap1)
    h = d
    for m in range(1, 10_001):
        m2 = 2 * m
        even = m * (b - m) * x / ((am1 + m2) * (a + m2))
        d = _guard(1.0 + even * d)
        c = _guard(1.0 + even / c)
        d = 1.0 / d
        h *= d * c
        odd = -((a + m) * (apb + m) * x / ((a + m2) * (ap1 + m2)))
        d = _guard(1.0 + odd * d)
        c = _guard(1.0 + odd / c)
        d = 1.0 / d
        step = d * c
        h *= step
        if abs(step - 1.0) < _CF_EPS:
            return h
    raise RuntimeError("incomplete beta continued fraction did not converge")


def _betainc(a: float, b: float, x: float) -> float:
    if x <= 0.0:
        return 0.0
    if x >= 1.0:
        return 1.0
    front = math.exp(
        math.lgamma(a + b) - math.lgamma(a) - math.lgamma(b)
        + a * math.log(x) + b * math.log1p(-x)
    )
    if x < (a + 1.0) / (a + b + 2.0):
        return front * _betacf(a, b, x) / a
    return 1.0 - front * _betacf(b, a, 1.0 - x) / b


def _half_quantile(dim: int, probability: float) -> float:
    """t >= 0 with P(|coordinate| <= t) = probability, by bisection on [0, 1]."""
    shape = (dim - 1) / 2
    lo, hi = 0.0, 1.0
    for _ in range(96):
        mid = (lo + hi) / 2
        if _betainc(0.5, shape, mid * mid) < probability:
            lo = mid
        else:
            hi = mid
    return (lo + hi) / 2


def _cell_mean(dim: int, left: float, right: float) -> float:
    """Conditional mean of the coordinate on [left, right] with 0 <= left < right <= 1."""
    shape = (dim - 1) / 2
    below = _betainc(0.5, shape, left * left)
    if right >= 1.0:
        span = _betainc(shape, 0.5, 1.0 - left * left)
    else:
        span = _betainc(0.5, shape, right * right) - below
    mass = 0.5 * span
    if mass <= 0.0:
        raise RuntimeError("Lloyd-Max interval has zero probability mass")
    log_l = shape * math.log1p(-(left * left)) if left < 1.0 else -math.inf
    log_r = shape * math.log1p(-(right * right)) if right < 1.0 else -math.inf
    raw = 0.0 if log_l == -math.inf else math.exp(log_l) * -math.expm1(log_r - log_l)
    scale = math.exp(math.lgamma(dim / 2) - 0.5 * math.log(math.pi) - math.lgamma(shape))
    return scale * raw / (2 * shape) / mass


def _exact_codebook(dim: int, bits: int) -> LloydMaxCodebook:
    levels = 2 ** bits
    half = levels // 2
    pos = [_half_quantile(dim, (i + 0.5) / half) for i in range(half)]
    budget = max(1_024, 6 * levels * levels)
    for _ in range(budget):
        edges = [0.0] + [(pos[i] + pos[i + 1]) / 2 for i in range(half - 1)] + [1.0]
        new = [_cell_mean(dim, edges[i], edges[i + 1]) for i in range(half)]
        if max(abs(n - o) for n, o in zip(new, pos)) < 1e-13:
            pos = new
            break
        pushed = [o + 1.9 * (n - o) for n, o in zip(new, pos)]
        ordered = all(
            0.0 < pushed[i] < (pushed[i + 1] if i + 1 < half else 1.0) for i in range(half)
        )
        pos = pushed if ordered else new
    else:
        raise RuntimeError(f"Lloyd-Max did not converge for dim={dim}, bits={bits}")
    centroids = torch.tensor([-v for v in reversed(pos)] + pos, dtype=torch.float64)
    boundaries = (centroids[:-1] + centroids[1:]) / 2
    return LloydMaxCodebook(dim, bits, centroids.to(torch.float32),
                            boundaries.to(torch.float32), 2)


def _grid_codebook(dim: int, bits: int) -> LloydMaxCodebook:
    """Version 1: Lloyd iteration on a 20001-point grid (kept for old artifacts)."""
    if dim < 2:
        raise ValueError("dim must be at least 2")
    levels = 2 ** bits
    grid = torch.linspace(-1 + 1e-6, 1 - 1e-6, 20001, dtype=torch.float64)
    alpha = (dim - 3) / 2
    inside = (1 - grid.square()).clamp_min(0)
    density = torch.ones_like(grid) if alpha == 0 else torch.exp(
        alpha * torch.log(inside.clamp_min(1e-45)))
    density[grid.abs() >= 1] = 0
    density = density / density.sum()
    cdf = torch.cumsum(density, dim=0)
    targets = (torch.arange(levels, dtype=torch.float64) + 0.5) / levels
    centroids = torch.empty(levels, dtype=torch.float64)
    for i, q in enumerate(targets):
        centroids[i] = grid[int(torch.searchsorted(cdf, q).clamp(max=grid.numel() - 1))]
    for _ in range(80):
        mids = (centroids[:-1] + centroids[1:]) / 2
        edges = torch.cat((torch.tensor([-1.0], dtype=torch.float64), mids,
                           torch.tensor([1.0], dtype=torch.float64)))
        new = torch.empty_like(centroids)
        for i in range(levels):
            lo, hi = float(edges[i]), float(edges[i + 1])
            mask = (grid >= lo) & (grid <= hi)
            w = density[mask]
            total = w.sum()
            new[i] = (lo + hi) / 2 if total <= 0 else float((grid[mask] * w).sum() / total)
        new = (new - torch.flip(new, dims=[0])) / 2
        done = torch.max(torch.abs(new - centroids)) < 1e-10
        centroids = new
        if done:
            break
    boundaries = (centroids[:-1] + centroids[1:]) / 2
    return LloydMaxCodebook(dim, bits, centroids.to(torch.float32),
                            boundaries.to(torch.float32), 1)


@lru_cache(maxsize=256)
def get_codebook(dim: int, bits: int, algorithm_version: int = 2) -> LloydMaxCodebook:
    if bits <= 0 or bits > 8:
        raise ValueError("bits must be in [1, 8]")
    if algorithm_version not in SUPPORTED_VERSIONS:
        raise ValueError(f"algorithm_version must be one of {list(SUPPORTED_VERSIONS)}")
    return _exact_codebook(dim, bits) if algorithm_version == 2 else _grid_codebook(dim, bits)


def clear_codebook_cache() -> None:
    get_codebook.cache_clear()
