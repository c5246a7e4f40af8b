"""Little-endian bit-stream packing of ``bits``-wide indices (host side).

Value ``i`` of the flattened index tensor occupies bits ``[i*bits, i*bits + bits)`` of
one flat ``uint8`` stream; a field may straddle two bytes (3- and 6-bit widths).  For
4 bits the even element is the low nibble.  This is the storage format of
``packed_weight_indices`` and is bit-exact with
``src/orbitquant/packing/bitpack.py:8-97``.  The CUDA kernels decode the same stream
in place; these numpy routines serve offline weight quantisation and tests.
"""
from __future__ import annotations

import numpy as np
import torch


def packed_length(value_count: int, bits: int) -> int:
    return (value_count * bits + 7) // 8


def _check_bits(bits: int) -> None:
    if bits <= 0 or bits > 8:
        raise ValueError("bits must be in [1, 8]")


def pack_lowbit(values: torch.Tensor, bits: int, *, validate: bool = True) -> torch.Tensor:
    _check_bits(bits)
    flat = values.detach().to("cpu").flatten()
    if validate and flat.numel() and (int(flat.min()) < 0 or int(flat.max()) > (1 << bits) - 1):
        raise ValueError(f"all values must fit in {bits} bits")
    v = flat.to(torch.uint8).numpy()
    # Expand every value to `bits` little-endian bits, then let numpy fold the bit
    # stream into bytes (bitorder="little" is exactly the stream definition above).
    stream = np.unpackbits(v[:, None], axis=1, bitorder="little")[:, :bits].reshape(-1)
    return torch.from_numpy(np.packbits(stream, bitorder="little"))


def unpack_lowbit(packed: torch.Tensor, bits: int, length: int) -> torch.Tensor:
    _check_bits(bits)
    if length < 0:
        raise ValueError("length must be non-negative")
    raw = packed.detach().to("cpu", torch.uint8).flatten().numpy()
    stream = np.unpackbits(raw, bitorder="little")[: length * bits].reshape(length, bits)
    weights = (1 << np.arange(bits, dtype=np.uint16)).astype(np.uint16)
    return torch.from_numpy((stream.astype(np.uint16) * weights).sum(axis=1).astype(np.uint8))
