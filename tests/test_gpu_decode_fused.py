"""The single-launch decode forward (rows <= 16 on small layers): one kernel that rotates,
quantises and multiplies.  It must launch once, agree with the oracle within the matmul
tolerance, and reproduce the two-kernel path bit for bit (same prologue arithmetic, same
products, same summation order)."""
from __future__ import annotations

import pytest
import torch

from orbitquant_b200 import OrbitQuantConfig, OrbitQuantLinear, native
from test_gpu_parity import _check_close, _dev

pytestmark = pytest.mark.gpu

CASES = [
    # rows, K, N, a_bits, block, bias, weight_mode
    (1, 768, 2304, 6, "paper", True, "centroid"), (4, 768, 768, 6, "paper", True, "centroid"),
    (5, 768, 3072, 6, "paper", False, "centroid"), (1, 3072, 768, 6, "paper", True, "centroid"),
    (1, 3072, 768, 4, "paper", True, "bf16_scaled"), (3, 1024, 520, 4, 512, True, "centroid"),
    (16, 256, 77, 3, 256, True, "centroid"), (1, 4096, 264, 4, 2048, False, "centroid"),
    (2, 2048, 1000, 2, 256, True, "bf16_scaled"), (8, 512, 512, 4, 256, True, "centroid"),
]


@pytest.mark.parametrize("rows,k,n,a_bits,block,bias,mode", CASES)
def test_fused_decode_forward(oracle, tunables, golden_codebooks, rows, k, n, a_bits, block, bias, mode):
    dev = _dev()
    torch.manual_seed(rows * 7 + k)
    cfg = OrbitQuantConfig(weight_bits=4, activation_bits=a_bits, rotation_seed=4, block_size=block)
    lin = torch.nn.Linear(k, n, bias=bias)
    with torch.no_grad():
        lin.weight.mul_(0.02 / lin.weight.std())
    module = OrbitQuantLinear.from_linear(lin, config=cfg, module_name="d").to(dev)
    module.weight_mode = mode
    x = torch.randn(rows, k)
    x[:, :4] *= 20
    if rows > 2:
        x[1] = 0
    x = x.to(torch.bfloat16)
    assert native.forward_kernel_name(rows, k, n, 4, a_bits, module.rotation.block_size,
                                      weight_mode=native.WEIGHT_MODE_NAMES[mode]) == "decode_fused_kernel"
    before = native.launch_count()
    y = module(x.to(dev))
    torch.cuda.synchronize()
    assert native.launch_count() - before == 1
    ref = oracle.linear_forward(
        x, module.packed_weight_indices.cpu(), module.row_norms.cpu(),
        None if module.bias is None else module.bias.detach().cpu(), perm=module.rotation.permutation,
        signs=module.rotation.signs, block=module.rotation.block_size,
        act_boundaries=module.activation_codebook.boundaries, act_centroids=module.activation_codebook.centroids,
        w_centroids=module.weight_codebook.centroids, w_bits=4, out_features=n,
        mode=oracle.MM_BF16_LUT if mode == "bf16_scaled" else oracle.MM_FP32_CENTROIDS)
    _check_close(y, ref, (rows, k, n, a_bits, mode))
    if rows > 2 and module.bias is not None:
        assert torch.equal(y[1].float().cpu(), module.bias.detach().cpu().to(torch.bfloat16).float())
    tunables.set("fused_decode", 0)
    before = native.launch_count()
    two_kernels = module(x.to(dev))
    torch.cuda.synchronize()
    assert native.launch_count() - before == 2
    assert torch.equal(y, two_kernels)


def test_fused_decode_in_a_cuda_graph_chain():
    """Four dependent layers captured in one graph: every layer reads the previous one's output
    (the kernels overlap their start-up through programmatic dependent launch), replays agree
    with the eager result."""
    dev = _dev()
    torch.manual_seed(0)
    cfg = OrbitQuantConfig(weight_bits=4, activation_bits=6, rotation_seed=4)
    shapes = [(768, 2304), (2304, 768), (768, 3072), (3072, 768)]
    layers = []
    for k, n in shapes:
        lin = torch.nn.Linear(k, n)
        with torch.no_grad():
            lin.weight.mul_(0.02 / lin.weight.std())
        layers.append(OrbitQuantLinear.from_linear(lin, config=cfg, module_name=f"{k}x{n}").to(dev))
    x = torch.randn(4, 768, device=dev).to(torch.bfloat16)

    def chain(inp):
        h = inp
        for layer in layers:
            h = layer(h)
        return h

    eager = chain(x)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        chain(x)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    static_x = x.clone()
    with torch.cuda.graph(graph):
        out = chain(static_x)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
    static_x.copy_(torch.randn(4, 768, device=dev).to(torch.bfloat16))
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, chain(static_x))
