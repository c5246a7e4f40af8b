"""Shared fixtures.  GPU tests carry ``@pytest.mark.gpu``; everything else runs on CPU."""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

REPO = Path(__file__).resolve().parent.parent
if str(REPO) not in sys.path:
    sys.path.insert(0, str(REPO))

GOLDEN = REPO / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200 / sm_100)")


def bf16_from_bits(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.astype(np.int16)).view(torch.bfloat16)


def bits_of(t: torch.Tensor) -> torch.Tensor:
    """Raw 16-bit patterns of a bf16/f16 tensor, for bit-exact comparisons."""
    return t.detach().cpu().contiguous().view(torch.int16)


@pytest.fixture(scope="session")
def golden_codebooks():
    return np.load(GOLDEN / "codebooks.npz")


@pytest.fixture(scope="session")
def golden_rotations():
    return np.load(GOLDEN / "rotations.npz")


@pytest.fixture(scope="session")
def golden_bitpack():
    return np.load(GOLDEN / "bitpack.npz")


@pytest.fixture(scope="session")
def golden_layers():
    return np.load(GOLDEN / "layer_cases.npz")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as module
    module.build()
    return module


def codebook_from_golden(golden, dim: int, bits: int, version: int = 2):
    """Build a LloydMaxCodebook from committed arrays (8-bit tables take minutes to derive)."""
    from orbitquant_b200.codebooks import LloydMaxCodebook
    key = f"v{version}_dim{dim}_bits{bits}"
    return LloydMaxCodebook(dim, bits, torch.from_numpy(golden[key + "_centroids"].copy()),
                            torch.from_numpy(golden[key + "_boundaries"].copy()), version)


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.double().flatten()
    b = b.double().flatten()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


@pytest.fixture
def tunables():
    """Pins tuning switches of the CUDA library for one test and releases them afterwards."""
    from orbitquant_b200 import native

    class _Tunables:
        def __init__(self):
            self.touched = set()

        def set(self, name, value):
            native.set_tunable(name, value)
            self.touched.add(name)

    handle = _Tunables()
    yield handle
    for name in handle.touched:
        native.set_tunable(name, None)
