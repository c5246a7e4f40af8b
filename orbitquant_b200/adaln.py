"""Symmetric INT4 round-to-nearest linear (group size 64) -- the weight-only format the
reference uses for AdaLN modulation layers (``src/orbitquant/adaln.py``).

``W[n, k] ~ (code[n, k] - 8) * scale[n, k // 64]`` with ``scale = max|w| / 7`` per group,
``code = clamp(round(w / scale), -8, 7) + 8`` packed two per byte (low nibble = even k), rows
padded to whole groups.  Activations stay bf16; the forward is
``bf16(sum_k x * bf16((code - 8) * scale) + bias)`` with fp32 accumulation, as the reference's
CPU kernel computes it (``orbitquant_packed_matmul_cpu/packed_adaln_cpu.cpp:54-100``).
State-dict keys as in the reference: ``packed_weight`` (uint8), ``scales`` (bf16
``[out_features, groups]``), ``bias``.
"""
from __future__ import annotations

import torch
from torch import nn

from . import native
from .config import OrbitQuantConfig
from .packing import pack_lowbit, packed_length, unpack_lowbit


def quantize_adaln_weight(weight: torch.Tensor, *, group_size: int = 64) -> tuple[torch.Tensor, torch.Tensor]:
    """``W [N, K]`` -> (packed codes, fp32 scales ``[N, groups]``); the reference's torch
    expression (``adaln.py:18-38``) op for op, on the CPU, so codes and scales are bit-identical."""
    if weight.ndim != 2:
        raise ValueError("weight must be a matrix")
    w = weight.detach().to(device="cpu", dtype=torch.float32)
    n, k = w.shape
    groups = (k + group_size - 1) // group_size
    padded = torch.zeros(n, groups * group_size, dtype=torch.float32)
    padded[:, :k] = w
    grouped = padded.reshape(n, groups, group_size)
    scales = grouped.abs().amax(dim=-1).clamp_min(1e-12) / 7.0
    signed = torch.round(grouped / scales[..., None]).clamp(-8, 7).to(torch.int16)
    packed = pack_lowbit((signed + 8).to(torch.uint8).flatten(), 4, validate=False)
    return packed, scales


class RTNInt4Linear(nn.Module):
    """INT4 group-64 RTN linear computed by the sm_100a few-token tensor-core kernel."""

    def __init__(self, *, in_features: int, out_features: int, group_size: int, module_name: str,
                 packed_weight: torch.Tensor, scales: torch.Tensor, bias: torch.Tensor | None) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.group_size = group_size
        self.module_name = module_name
        self.num_groups = (in_features + group_size - 1) // group_size
        self.packed_weight = nn.Parameter(packed_weight, requires_grad=False)
        self.scales = nn.Parameter(scales.to(torch.bfloat16), requires_grad=False)
        if bias is None:
            self.register_parameter("bias", None)
        else:
            self.bias = nn.Parameter(bias.detach().clone(), requires_grad=False)
        # same handle registry as OrbitQuantLinear: the module traces as one opaque node of
        # the shared custom op, with bf16_output=True (reference adaln.py:312-317)
        from .layers import _registry_register
        self._compile_handle = _registry_register(self)

    @classmethod
    def from_linear(cls, layer: nn.Module, *, config: OrbitQuantConfig, module_name: str) -> "RTNInt4Linear":
        if not isinstance(layer, nn.Linear):
            raise TypeError(f"no OrbitQuant linear adapter registered for {type(layer).__name__}")
        packed, scales = quantize_adaln_weight(layer.weight, group_size=config.adaln_group_size)
        device = layer.weight.device
        bias = None if layer.bias is None else layer.bias.detach()
        return cls(in_features=layer.in_features, out_features=layer.out_features,
                   group_size=config.adaln_group_size, module_name=module_name,
                   packed_weight=packed.to(device), scales=scales.to(device), bias=bias)

    @classmethod
    def empty_from_linear(cls, layer: nn.Module, *, config: OrbitQuantConfig,
                          module_name: str) -> "RTNInt4Linear":
        if not isinstance(layer, nn.Linear):
            raise TypeError(f"no OrbitQuant linear adapter registered for {type(layer).__name__}")
        group = config.adaln_group_size
        groups = (layer.in_features + group - 1) // group
        device = layer.weight.device
        packed = torch.empty(packed_length(layer.out_features * groups * group, 4), dtype=torch.uint8,
                             device=device)
        scales = torch.empty(layer.out_features, groups, dtype=torch.bfloat16, device=device)
        bias = None
        if layer.bias is not None:
            bias = torch.zeros(layer.out_features, dtype=layer.bias.dtype, device=layer.bias.device)
        return cls(in_features=layer.in_features, out_features=layer.out_features, group_size=group,
                   module_name=module_name, packed_weight=packed, scales=scales, bias=bias)

    def dequantize_weight(self, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        total = self.out_features * self.num_groups * self.group_size
        codes = unpack_lowbit(self.packed_weight.cpu(), 4, total).to(torch.int16).sub(8).to(torch.float32)
        grouped = codes.reshape(self.out_features, self.num_groups, self.group_size)
        weight = (grouped * self.scales.cpu().float()[..., None]).reshape(self.out_features, -1)
        return weight[:, : self.in_features].to(dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if torch.compiler.is_compiling():
            return torch.ops.orbitquant.packed_linear_forward(
                x, self._compile_handle, self.out_features, True)
        return self._forward_impl(x)

    def _forward_impl(self, x: torch.Tensor) -> torch.Tensor:
        if x.device.type != "cuda":
            raise RuntimeError("RTNInt4Linear (orbitquant_b200) requires CUDA input tensors on an "
                               f"sm_100 device; got {x.device.type}. There is no CPU path in this package.")
        if x.shape[-1] != self.in_features:
            raise ValueError(f"expected last dimension {self.in_features}, got {x.shape[-1]}")
        if self.packed_weight.device != x.device:
            raise RuntimeError("move the module to the input's device first")
        bias = self.bias
        if bias is not None and bias.dtype not in native.DTYPE_CODES:
            bias = bias.float()
        return native.rtn_int4_linear_forward(x, self.packed_weight, self.scales, bias,
                                              out_features=self.out_features, group_size=self.group_size)
