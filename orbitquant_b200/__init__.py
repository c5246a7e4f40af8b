"""orbitquant_b200: the OrbitQuant quantized-linear forward for NVIDIA B200 (sm_100a).

Public surface (same names as the reference package for this path):
``OrbitQuantConfig``, ``OrbitQuantLinear``, ``get_codebook``, ``get_rpbh_rotation``,
``pack_lowbit`` / ``unpack_lowbit``, ``quantize_activations`` and the registered custom op
``torch.ops.orbitquant.packed_linear_forward``.
"""
from .adaln import RTNInt4Linear, quantize_adaln_weight
from .artifacts import load_orbitquant_artifact
from .codebooks import LloydMaxCodebook, get_codebook
from .config import OrbitQuantConfig
from .functional import quantize_activations
from .int8_surrogate import fit_int8_centroid_surrogate
from .layers import OrbitQuantLinear, quantize_weight
from .packing import pack_lowbit, packed_length, unpack_lowbit
from .rotations import RPBHRotation, fwht, get_rpbh_rotation

__all__ = [
    "load_orbitquant_artifact",
    "RTNInt4Linear",
    "quantize_adaln_weight",
    "LloydMaxCodebook", "OrbitQuantConfig", "OrbitQuantLinear", "RPBHRotation", "fwht",
    "fit_int8_centroid_surrogate", "get_codebook", "get_rpbh_rotation", "pack_lowbit", "packed_length", "quantize_activations",
    "quantize_weight", "unpack_lowbit",
]
__version__ = "0.1.0"
