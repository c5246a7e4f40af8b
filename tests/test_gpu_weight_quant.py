"""Offline weight quantise-and-pack on the GPU (oq_quantize_weight) against the CPU path,
which runs the reference's torch ops in the reference's order (layers.py:quantize_weight)."""
from __future__ import annotations

import pytest
import torch

from orbitquant_b200 import OrbitQuantConfig, OrbitQuantLinear, RPBHRotation, get_codebook, unpack_lowbit
from orbitquant_b200.layers import quantize_weight, quantize_weight_gpu
from test_gpu_parity import _dev

pytestmark = pytest.mark.gpu

CASES = [
    # N, K, block, bits, dtype
    (9, 32, 8, 2, torch.float32), (9, 32, 8, 3, torch.float32), (9, 32, 8, 4, torch.float32),
    (9, 32, 8, 6, torch.float32),           # the reference's own GPU test shapes
    (40, 768, 256, 4, torch.float32), (33, 3072, 1024, 4, torch.float32),
    (17, 12288, 4096, 3, torch.float32), (24, 200, 8, 4, torch.float32),
    (64, 1024, 1024, 2, torch.bfloat16), (31, 768, 256, 6, torch.float16),
]


@pytest.mark.parametrize("n,k,block,bits,dtype", CASES)
def test_indices_bit_identical_given_the_same_row_norms(n, k, block, bits, dtype):
    dev = _dev()
    g = torch.Generator().manual_seed(n * 7 + k + bits)
    weight = (torch.randn(n, k, generator=g) * 0.02).to(dtype)
    weight[0, :3] *= 40.0
    if n > 4:
        weight[4] = 0.0          # zero row: norm 0 -> clamp to eps -> every direction 0
    rotation = RPBHRotation(k, seed=5, block_size=block)
    codebook = get_codebook(k, bits)
    packed_cpu, norms_cpu = quantize_weight(weight, rotation=rotation, codebook=codebook, bits=bits, eps=1e-10)
    fp32_norms = weight.to(torch.float32).norm(dim=-1)
    packed_gpu, norms_gpu = quantize_weight_gpu(weight.to(dev), rotation=rotation, codebook=codebook,
                                                bits=bits, eps=1e-10, row_norms=fp32_norms)
    assert torch.equal(packed_gpu.cpu(), packed_cpu), "packed index stream differs"
    assert torch.equal(norms_gpu.cpu(), norms_cpu)


def test_device_computed_norms_and_module_construction():
    dev = _dev()
    torch.manual_seed(3)
    lin = torch.nn.Linear(3072, 520)
    cfg = OrbitQuantConfig(weight_bits=4, activation_bits=4, rotation_seed=2)
    cpu = OrbitQuantLinear.from_linear(lin, config=cfg, module_name="wq.cpu")
    gpu = OrbitQuantLinear.from_linear(lin, config=cfg, module_name="wq.gpu", quantization_device=dev)
    # norms: double accumulation vs torch's fp32 reduction -> equal after bf16 rounding almost always
    same_norms = (gpu.row_norms.cpu() == cpu.row_norms).float().mean().item()
    assert same_norms >= 0.99
    a = unpack_lowbit(gpu.packed_weight_indices.cpu(), 4, 520 * 3072)
    b = unpack_lowbit(cpu.packed_weight_indices, 4, 520 * 3072)
    mismatch = (a != b).float().mean().item()
    assert mismatch <= 1e-4, mismatch          # only indices within an ulp of a boundary may move
    assert (a.int() - b.int()).abs().max().item() <= 1
    x = (torch.randn(300, 3072) * 0.5).to(torch.bfloat16).to(dev)
    y_gpu = gpu.to(dev)(x).float()
    y_cpu = cpu.to(dev)(x).float()
    assert float((y_gpu - y_cpu).norm() / y_cpu.norm()) < 2e-3
