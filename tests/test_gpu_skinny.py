"""The few-token tcgen05 kernel (1..128 rows: weight rows on the MMA's M side, tokens on its
N side, reduction slices summed by a second kernel), through the C ABI, against the CPU
oracle.  Tolerances as in test_gpu_parity."""
from __future__ import annotations

import pytest
import torch

from orbitquant_b200 import OrbitQuantConfig, OrbitQuantLinear, get_codebook, native
from test_gpu_parity import _check_close, _dev, _random_layer
from test_gpu_tcgen05 import _assert_status_clean

pytestmark = pytest.mark.gpu


def _case(oracle, rows, k, n, bits, cent, seed, with_bias=True):
    dev = _dev()
    native.gemm_clear_device_status()
    idx, packed, rn, bias = _random_layer(k, n, bits, seed=seed, bias=with_bias)
    x = (torch.randn(rows, k, generator=torch.Generator().manual_seed(seed)) * 1.2).to(torch.bfloat16)
    args = dict(bits=bits, out_features=n, in_features=k, bias=bias, kernel=native.KERNEL_TCGEN05)
    y = native.matmul_packed_weight(x.to(dev), packed.to(dev), rn, cent, **args)
    _assert_status_clean()
    ref = oracle.matmul_packed(x, packed, rn, cent, bits=bits, out_features=n, bias=bias,
                                  mode=oracle.MM_FP32_CENTROIDS)
    _check_close(y, ref, (rows, k, n, bits))
    again = native.matmul_packed_weight(x.to(dev), packed.to(dev), rn, cent, **args)
    assert torch.equal(y, again), "not deterministic"
    return y


@pytest.mark.parametrize("rows,k,n", [
    (1, 64, 8),          # one k step, one slice, a single partial weight tile
    (1, 3072, 3072), (16, 3072, 3072), (7, 768, 2304),
    (16, 12288, 1030),   # many slices, ragged last weight tile
    (5, 4736, 1536),     # 74 k steps: slices of unequal length
    (17, 192, 40), (33, 1024, 520), (64, 3072, 640), (100, 768, 264), (128, 2048, 384),
])
def test_skinny_vs_oracle(oracle, rows, k, n):
    _case(oracle, rows, k, n, 4, get_codebook(k, 4).centroids, seed=rows + k + n)


@pytest.mark.parametrize("bits", [2, 3, 6, 8])
@pytest.mark.parametrize("rows", [3, 16, 48])
def test_skinny_other_bit_widths(oracle, golden_codebooks, bits, rows):
    from conftest import codebook_from_golden
    k, n = 768, 456
    cent = (codebook_from_golden(golden_codebooks, k, 8) if bits == 8 else get_codebook(k, bits)).centroids
    _case(oracle, rows, k, n, bits, cent, seed=bits * 13 + rows, with_bias=bits != 3)


def test_skinny_agrees_with_large_row_kernel(tunables):
    """Same operands, same f16 products: the two tcgen05 kernels differ only in the order of
    the fp32 accumulation."""
    dev = _dev()
    k, n, rows = 3072, 1536, 96
    idx, packed, rn, bias = _random_layer(k, n, 4, seed=77)
    cent = get_codebook(k, 4).centroids
    x = torch.randn(rows, k).to(torch.bfloat16).to(dev)
    args = dict(bits=4, out_features=n, in_features=k, bias=bias, kernel=native.KERNEL_TCGEN05)
    a = native.matmul_packed_weight(x, packed.to(dev), rn, cent, **args)
    tunables.set("skinny", 0)
    b = native.matmul_packed_weight(x, packed.to(dev), rn, cent, **args)
    _assert_status_clean()
    _check_close(a, b, "few-token vs large-row kernel")


def test_module_forward_decode_batch_on_large_layer(oracle):
    """rows <= 16 on a layer of several megabytes: the module's forward takes the prologue in
    its f16-operand mode plus the few-token kernel; compare with the oracle's whole forward."""
    dev = _dev()
    torch.manual_seed(3)
    lin = torch.nn.Linear(3072, 3072, bias=True)
    cfg = OrbitQuantConfig(weight_bits=4, activation_bits=4, rotation_seed=1)
    q = OrbitQuantLinear.from_linear(lin, config=cfg, module_name="decode.big")
    x = (torch.randn(9, 3072) * 0.8).to(torch.bfloat16)
    y = q.to(dev)(x.to(dev))
    _assert_status_clean()
    rot, acb, wcb = q.rotation, get_codebook(3072, 4), get_codebook(3072, 4)
    ref = oracle.linear_forward(x, q.packed_weight_indices.cpu(), q.row_norms.cpu(), q.bias.cpu(),
                                   perm=rot.permutation, signs=rot.signs, block=rot.block_size,
                                   act_boundaries=acb.boundaries, act_centroids=acb.centroids,
                                   w_centroids=wcb.centroids, w_bits=4, out_features=3072,
                                   norm_order=oracle.NORM_AVX512, mode=oracle.MM_FP32_CENTROIDS)
    _check_close(y, ref, "module forward, 9 rows")
