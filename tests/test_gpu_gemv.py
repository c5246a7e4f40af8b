"""The CUDA-core GEMV for one to four tokens on large W4 layers: it must be the kernel chosen
there, agree with the oracle within the matmul tolerance (fp32 centroids, fp32 accumulation),
stay close to the tensor-core few-token kernel it replaces, give the same bits on every run and
handle ragged shapes (out_features not a multiple of 8, in_features not a multiple of 1024)."""
from __future__ import annotations

import pytest
import torch

from orbitquant_b200 import OrbitQuantConfig, OrbitQuantLinear, native
from test_gpu_parity import _check_close, _dev, rel_l2

pytestmark = pytest.mark.gpu

CASES = [
    # rows, K, N, a_bits, bias, forced (the layer is below the size where the GEMV is the default)
    (1, 3072, 3072, 4, True, False), (2, 3072, 3072, 4, True, False), (3, 3072, 2304, 4, False, False),
    (4, 3072, 3072, 6, True, False), (1, 12288, 1024, 4, True, False), (4, 5120, 1536, 4, True, False),
    (1, 256, 8, 4, True, True), (2, 1280, 77, 3, True, True), (3, 768, 2304, 6, False, True),
    (4, 2304, 1003, 4, True, True), (1, 13824, 520, 4, True, False),
    # several passes of the persistent grid over the row blocks, the last block ragged
    (1, 3072, 12296, 4, True, False), (2, 1024, 9740, 4, False, True),
]


def _module(k, n, a_bits, bias, dev, seed):
    torch.manual_seed(seed)
    cfg = OrbitQuantConfig(weight_bits=4, activation_bits=a_bits, rotation_seed=5)
    lin = torch.nn.Linear(k, n, bias=bias)
    with torch.no_grad():
        lin.weight.mul_(0.02 / lin.weight.std())
    return OrbitQuantLinear.from_linear(lin, config=cfg, module_name="g").to(dev)


@pytest.mark.parametrize("rows,k,n,a_bits,bias,forced", CASES)
def test_gemv_forward(oracle, tunables, rows, k, n, a_bits, bias, forced):
    dev = _dev()
    module = _module(k, n, a_bits, bias, dev, rows * 11 + n)
    x = torch.randn(rows, k)
    x[:, :4] *= 20
    if rows > 2:
        x[1] = 0
    x = x.to(torch.bfloat16)
    if forced:
        tunables.set("gemv", 1)
    assert native.forward_kernel_name(rows, k, n, 4, a_bits, module.rotation.block_size) == \
        "rotate_quantize + gemv_w4_kernel"
    before = native.launch_count()
    y = module(x.to(dev))
    torch.cuda.synchronize()
    assert native.launch_count() - before == 2
    ref = oracle.linear_forward(
        x, module.packed_weight_indices.cpu(), module.row_norms.cpu(),
        None if module.bias is None else module.bias.detach().cpu(), perm=module.rotation.permutation,
        signs=module.rotation.signs, block=module.rotation.block_size,
        act_boundaries=module.activation_codebook.boundaries, act_centroids=module.activation_codebook.centroids,
        w_centroids=module.weight_codebook.centroids, w_bits=4, out_features=n, mode=oracle.MM_FP32_CENTROIDS)
    _check_close(y, ref, (rows, k, n, a_bits))
    if rows > 2 and module.bias is not None:
        assert torch.equal(y[1].float().cpu(), module.bias.detach().cpu().to(torch.bfloat16).float())
    again = module(x.to(dev))
    torch.cuda.synchronize()
    assert torch.equal(y, again)
    tunables.set("gemv", 0)
    assert "gemv" not in native.forward_kernel_name(rows, k, n, 4, a_bits, module.rotation.block_size)
    other = module(x.to(dev))
    torch.cuda.synchronize()
    assert rel_l2(y.float().cpu(), other.float().cpu()) <= 2e-3


def test_gemv_is_not_chosen_outside_its_range():
    name = native.forward_kernel_name
    assert "gemv" in name(4, 3072, 12288, 4, 4, 1024)
    assert "gemv" not in name(5, 3072, 12288, 4, 4, 1024)                      # more than four tokens
    assert "gemv" not in name(1, 768, 2304, 4, 6, 256)                         # small layer: one launch
    assert "gemv" not in name(1, 3072, 12288, 3, 4, 1024)                      # other bit widths
    assert "gemv" not in name(1, 3072, 12288, 4, 4, 1024, weight_mode=native.WEIGHT_MODE_NAMES["bf16_scaled"])


def test_gemv_in_a_cuda_graph_chain():
    """Dependent layers captured in one graph (every kernel is launched programmatically and
    starts before its predecessor has finished): replays agree with the eager result."""
    dev = _dev()
    shapes = [(3072, 3072), (3072, 12288), (12288, 3072)]
    layers = [_module(k, n, 4, True, dev, k + n) for k, n in shapes]
    x = torch.randn(2, 3072, device=dev).to(torch.bfloat16)

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
    static_x.copy_(torch.randn(2, 3072, device=dev).to(torch.bfloat16))
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, chain(static_x))
