"""The warp-per-block rotate-and-quantize kernel (large token counts): its quantised
activations must be bit-identical to the oracle's (AVX-512 operation order of the reference,
``quantize_activations_cpu.cpp:633-664``) and its f16-operand output must reproduce, through
the tensor-core GEMM, exactly what the multi-token-CTA kernel's output produces."""
from __future__ import annotations

import pytest
import torch

from conftest import bits_of, codebook_from_golden
from orbitquant_b200 import OrbitQuantConfig, OrbitQuantLinear, RPBHRotation, get_codebook, native
from test_gpu_parity import _dev

pytestmark = pytest.mark.gpu

CASES = [
    # rows, dim, block, bits, seed
    (1, 1024, 256, 4, 1), (5, 768, 256, 6, 4), (37, 3072, 256, 4, 0), (301, 3072, 1024, 4, 1),
    (23, 3072, 1024, 3, 2), (10, 5120, 1024, 4, 3), (7, 1024, 512, 2, 5), (9, 13824, 512, 4, 3),
    (6, 4096, 2048, 4, 7), (11, 12288, 4096, 4, 1), (5, 8192, 4096, 6, 2), (4, 1024, 1024, 8, 6),
    (700, 768, 256, 6, 9),
]


@pytest.mark.parametrize("rows,dim,block,bits,seed", CASES)
def test_warp_prologue_bit_exact_vs_oracle(oracle, golden_codebooks, tunables, rows, dim, block, bits, seed):
    dev = _dev()
    rot = RPBHRotation(dim, seed, block)
    cb = codebook_from_golden(golden_codebooks, 256, 8) if bits == 8 else get_codebook(dim, bits)
    g = torch.Generator().manual_seed(seed + 100)
    x = torch.randn(rows, dim, generator=g) * (torch.rand(rows, 1, generator=g) * 3 + 0.1)
    x[:, : max(1, dim // 200)] *= 20
    if rows > 2:
        x[rows // 2] = 0
    x = x.to(torch.bfloat16)
    xq_ref, _codes, _norms = oracle.quantize_activations(
        x, rot.permutation, rot.signs, block, cb.boundaries, cb.centroids, eps=1e-10,
        norm_order=oracle.NORM_AVX512)
    native.gemm_clear_device_status()
    tunables.set("prologue_kernel", 2)
    before = native.launch_count()
    xq = native.quantize_activations(x.to(dev), rot.permutation, rot.signs, cb.centroids,
                                     cb.boundaries, eps=1e-10, block_size=block)
    torch.cuda.synchronize()
    assert native.launch_count() - before == 1
    assert native.gemm_device_status() == 0
    assert torch.equal(bits_of(xq), bits_of(xq_ref)), "quantised activations differ"
    if rows > 2:
        assert torch.all(xq[rows // 2] == 0)
    tunables.set("prologue_kernel", 1)
    xq_other = native.quantize_activations(x.to(dev), rot.permutation, rot.signs, cb.centroids,
                                           cb.boundaries, eps=1e-10, block_size=block)
    assert torch.equal(bits_of(xq_other), bits_of(xq)), "the two specialised kernels differ"


@pytest.mark.parametrize("rows,k,n,w_bits,a_bits,block", [(600, 3072, 512, 4, 4, "paper"), (333, 1024, 384, 3, 3, 256),
                                                            (130, 4096, 256, 4, 4, "paper")])
def test_f16_operand_output_feeds_the_gemm_identically(tunables, rows, k, n, w_bits, a_bits, block):
    dev = _dev()
    torch.manual_seed(rows)
    cfg = OrbitQuantConfig(weight_bits=w_bits, activation_bits=a_bits, rotation_seed=2, block_size=block)
    module = OrbitQuantLinear.from_linear(torch.nn.Linear(k, n), config=cfg, module_name="p").to(dev)
    x = torch.randn(rows, k, device=dev)
    x[:, :5] *= 20
    x[3] = 0
    x = x.to(torch.bfloat16)
    native.gemm_clear_device_status()
    tunables.set("prologue_kernel", 1)
    y1 = module(x)
    tunables.set("prologue_kernel", 2)
    y2 = module(x)
    torch.cuda.synchronize()
    assert native.gemm_device_status() == 0
    assert torch.equal(y1, y2)


def test_large_batches_take_the_warp_kernel_by_default(oracle):
    """No tunable set: 4608 tokens of 3072 features (the benchmark's shape) against the oracle
    on a row sample, including the ragged last batch."""
    dev = _dev()
    dim, block, bits, rows = 3072, 1024, 4, 4607
    rot = RPBHRotation(dim, 1, block)
    cb = get_codebook(dim, bits)
    x = (torch.randn(rows, dim, generator=torch.Generator().manual_seed(3)) * 1.5).to(torch.bfloat16)
    xq = native.quantize_activations(x.to(dev), rot.permutation, rot.signs, cb.centroids,
                                     cb.boundaries, eps=1e-10, block_size=block).cpu()
    pick = torch.cat([torch.arange(0, 40), torch.arange(2300, 2340), torch.arange(rows - 40, rows)])
    ref, _c, _n = oracle.quantize_activations(x[pick], rot.permutation, rot.signs, block, cb.boundaries,
                                              cb.centroids, eps=1e-10, norm_order=oracle.NORM_AVX512)
    assert torch.equal(bits_of(xq[pick]), bits_of(ref))


def test_chained_layers_respect_stream_order():
    """Prologue and GEMM are launched programmatically (each may start while the kernel before
    it drains) and wait for their predecessor before touching its output.  Three dependent
    layers enqueued back to back must give the bits of the same layers run with a device
    synchronisation in between, every time."""
    dev = _dev()
    torch.manual_seed(11)
    cfg = OrbitQuantConfig(weight_bits=4, activation_bits=4, rotation_seed=2)
    dims = [(768, 1536), (1536, 768), (768, 1024)]
    layers = []
    for k, n in dims:
        lin = torch.nn.Linear(k, n)
        with torch.no_grad():
            lin.weight.mul_(0.05 / lin.weight.std())
        layers.append(OrbitQuantLinear.from_linear(lin, config=cfg, module_name=f"l{k}").to(dev))
    x = torch.randn(2304, 768).to(torch.bfloat16).to(dev)   # >= 2048 rows: the warp-per-block prologue
    assert "rotate_quantize" in native.forward_kernel_name(2304, 768, 1536, 4, 4, layers[0].rotation.block_size)

    def run(sync):
        h = x
        for layer in layers:
            h = layer(h)
            if sync:
                torch.cuda.synchronize()
        return h

    native.gemm_clear_device_status()
    reference = run(sync=True)
    for _ in range(6):
        assert torch.equal(run(sync=False), reference)
    torch.cuda.synchronize()
    assert native.gemm_device_status() == 0
