"""Loader for ``oracle/_ref/_orbitquant_ref_cpu.so`` (the reference's own CPU
kernels, compiled unmodified by ``oracle/build_ref.py``).

TEST INFRASTRUCTURE ONLY: used by ``tests/``, ``__graft_entry__.smoke()`` and
the CPU-baseline / reference arm of ``bench.py``.  The product path never
imports this module.

The two wrappers allocate outputs and coerce auxiliary dtypes the same way the
reference's Python shim does
(``native-kernels/orbitquant-packed-matmul/torch-ext/orbitquant_packed_matmul/
__init__.py:66-160``): row norms and bias become fp32 on CPU, a missing bias is a
1-element dummy with ``has_bias=False``.
"""
from __future__ import annotations

import os
from pathlib import Path

import torch

_SO = Path(__file__).resolve().parent / "_ref" / "_orbitquant_ref_cpu.so"
_NAMESPACE = "_orbitquant_ref_cpu"
_loaded = False


def available() -> bool:
    return _SO.exists()


def _ops():
    global _loaded
    if not _loaded:
        if not _SO.exists():
            raise RuntimeError(
                f"{_SO} is missing: run `python oracle/build_ref.py` where the reference "
                "sources are present"
            )
        torch.ops.load_library(str(_SO))
        _loaded = True
    return getattr(torch.ops, _NAMESPACE)


def set_isa(isa: str | None) -> None:
    """Pin the reference's ISA dispatch (read from the environment on every
    call, ``packed_matmul_cpu.cpp:72-113``): auto|scalar|avx2|avx512."""
    if isa is None:
        os.environ.pop("ORBITQUANT_CPU_ISA", None)
    else:
        os.environ["ORBITQUANT_CPU_ISA"] = isa


def host_isa_report() -> dict:
    flags = ""
    try:
        with open("/proc/cpuinfo") as fh:
            for line in fh:
                if line.startswith("flags"):
                    flags = line
                    break
    except OSError:
        pass
    return {
        "avx512f": " avx512f" in flags,
        "avx512_bf16": " avx512_bf16" in flags,
        "avx2": " avx2" in flags,
        "isa_env": os.environ.get("ORBITQUANT_CPU_ISA", "auto"),
        "cpu_capability": torch.backends.cpu.get_cpu_capability(),
    }


def quantize_activations_cpu(x, permutation, signs, centroids, boundaries, *, eps,
                             inv_sqrt_block, block_size):
    dim = x.shape[-1]
    values = x.contiguous().reshape(-1, dim)
    out = torch.empty_like(values)
    perm = permutation.to(device="cpu", dtype=torch.int32).contiguous()
    _ops().quantize_activations_cpu(
        out, values, perm,
        signs.to(device="cpu", dtype=torch.int8).contiguous(),
        centroids.to(device="cpu", dtype=torch.float32).contiguous(),
        boundaries.to(device="cpu", dtype=torch.float32).contiguous(),
        float(eps), float(inv_sqrt_block), int(block_size),
    )
    return out.reshape(x.shape)


def matmul_packed_weight(x, packed, row_norms, centroids, *, bits, out_features,
                         in_features, bias=None):
    x2 = x.contiguous().reshape(-1, in_features)
    out = torch.empty((x2.shape[0], out_features), dtype=x.dtype)
    if bias is None:
        bias_values = torch.empty((1,), dtype=torch.float32)
        has_bias = False
    else:
        bias_values = bias.to(device="cpu", dtype=torch.float32).contiguous()
        has_bias = True
    _ops().matmul_packed_weight(
        out, x2,
        packed.to(device="cpu", dtype=torch.uint8).contiguous(),
        row_norms.to(device="cpu", dtype=torch.float32).contiguous(),
        centroids.to(device="cpu", dtype=torch.float32).contiguous(),
        bias_values, has_bias, int(bits), int(out_features), int(in_features),
        64, 64, 128,
    )
    return out.reshape(*x.shape[:-1], out_features)


def linear_forward(x, packed, row_norms, bias, *, permutation, signs, act_centroids,
                   act_boundaries, w_centroids, w_bits, out_features, eps, block_size):
    """The reference CPU ``native_packed_matmul`` forward
    (``src/orbitquant/layers.py:1364-1380, 1427-1448``): activation pipeline then
    packed matmul, both by the reference's compiled kernels."""
    in_features = x.shape[-1]
    x_q = quantize_activations_cpu(
        x, permutation, signs, act_centroids, act_boundaries, eps=eps,
        inv_sqrt_block=1.0 / (block_size ** 0.5), block_size=block_size)
    return matmul_packed_weight(
        x_q, packed, row_norms, w_centroids, bits=w_bits, out_features=out_features,
        in_features=in_features, bias=bias)


def matmul_packed_adaln_int4(x, packed, scales, *, out_features, in_features, group_size=64, bias=None):
    """The reference's CPU RTN-INT4 kernel (``packed_adaln_cpu.cpp:807-878``): bf16 x, fp32
    scales ``[N, groups]``, fp32 bias -> bf16."""
    x2 = x.to(torch.bfloat16).contiguous().reshape(-1, in_features)
    out = torch.empty((x2.shape[0], out_features), dtype=torch.bfloat16)
    if bias is None:
        bias_values = torch.empty((1,), dtype=torch.float32)
        has_bias = False
    else:
        bias_values = bias.to(device="cpu", dtype=torch.float32).contiguous()
        has_bias = True
    _ops().matmul_packed_adaln_int4_cpu(
        out, x2, packed.to(device="cpu", dtype=torch.uint8).contiguous(),
        scales.to(device="cpu", dtype=torch.float32).contiguous(), bias_values, has_bias,
        int(out_features), int(in_features), int(group_size))
    return out.reshape(*x.shape[:-1], out_features)
