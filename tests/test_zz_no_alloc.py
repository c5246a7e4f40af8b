"""The no-allocation entry point ``oq_linear_forward_static``.

Some users of the library cannot allocate device memory around a forward call: plugin code
that runs inside another runtime's enqueue callback, or programs that handed the whole GPU to
one memory pool at start-up.  For them the library carries a fixed 4 MiB scratch array and
this entry point uses it instead of a caller-provided workspace.  The test drives the entry
point through the C ABI directly and compares it with the regular entry point
(``oq_linear_forward``, caller-provided workspace) on two calls in a row -- the second call
finds the first call's leftovers in the shared array and must not be affected by them.

This file sorts last on purpose, so that a run that stops at the first failure has already
been through every other test.
"""
from __future__ import annotations

import ctypes

import pytest
import torch

from orbitquant_b200 import OrbitQuantConfig, OrbitQuantLinear, native

pytestmark = pytest.mark.gpu


def _forward_static(module: OrbitQuantLinear, x: torch.Tensor, kernel: int = 0,
                    out: torch.Tensor | None = None) -> tuple[int, torch.Tensor]:
    """One raw C-ABI call; every tensor already lives on the device in its final dtype."""
    lib = native.load()
    device = x.device
    module._ensure_derived_constants(device)
    x2 = x.contiguous().reshape(-1, module.in_features)
    if out is None:
        out = torch.empty((x2.shape[0], module.out_features), dtype=x.dtype, device=device)
    bias = module._bias_for(device)
    vp = ctypes.c_void_p
    with torch.cuda.device(device):
        status = lib.oq_linear_forward_static(
            vp(out.data_ptr()), vp(x2.data_ptr()), native.DTYPE_CODES[x.dtype], x2.shape[0],
            module.in_features, module.out_features, vp(module.packed_weight_indices.data_ptr()),
            module.packed_weight_indices.numel(), module.weight_bits,
            vp(module._row_norms_for(device).data_ptr()),
            vp(module._weight_codebook_centroids.data_ptr()),
            None if bias is None else vp(bias.data_ptr()),
            0 if bias is None else native.DTYPE_CODES[bias.dtype],
            vp(module._rotation_permutation.data_ptr()), vp(module._rotation_signs.data_ptr()),
            module.rotation.block_size, vp(module._activation_codebook_boundaries.data_ptr()),
            vp(module._activation_codebook_centroids.data_ptr()), module.activation_bits,
            float(module.activation_eps), 0, kernel,
            vp(torch.cuda.current_stream(device).cuda_stream))
    return status, out


@pytest.mark.parametrize("rows,k,n,w_bits,a_bits,bias,kernel", [
    (8, 768, 2304, 4, 6, True, "auto"),       # decode batch
    (200, 1024, 512, 4, 4, True, "auto"),     # tcgen05 kernel: scratch holds the f16 operand + token factors
    (24, 768, 96, 3, 3, True, "auto"),        # general tiled kernel
    (16, 3072, 3072, 4, 4, True, "tcgen05"),  # few-token kernel, several reduction slices: partial
                                              # sums and slice COUNTERS live in the shared array
    (96, 1024, 640, 4, 4, False, "tcgen05"),  # explicit kernel choice, no bias
    (2, 3072, 3072, 4, 4, True, "auto"),       # two tokens of a large layer: prologue + CUDA-core GEMV
])
def test_static_scratch_forward_matches_workspace_forward(rows, k, n, w_bits, a_bits, bias, kernel):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    device = torch.device("cuda", 0)
    torch.manual_seed(rows)
    config = OrbitQuantConfig(weight_bits=w_bits, activation_bits=a_bits, rotation_seed=5)
    module = OrbitQuantLinear.from_linear(torch.nn.Linear(k, n, bias=bias), config=config,
                                          module_name="no_alloc").to(device)
    module.kernel = kernel
    assert native.load().oq_static_scratch_bytes() == 4 << 20
    for call in range(2):  # the second call reuses the array the first one filled
        x = (torch.randn(rows, k, device=device) * (1.0 + call)).to(torch.bfloat16)
        expected = module(x)               # regular path, workspace allocated by torch
        status, got = _forward_static(module, x, native.KERNEL_NAMES[kernel])
        assert status == 0, native.load().oq_last_error().decode()
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        rel = float((got.float() - expected.float()).norm() / expected.float().norm())
        assert rel <= 1e-3, (call, rel)    # same kernels: in practice the outputs are identical
        assert torch.equal(got, expected), call


def test_static_scratch_call_allocates_nothing_and_takes_empty_batches():
    """After one warm-up call per device, a call through the entry point leaves the device's
    free memory exactly as it found it (no cudaMalloc, no allocator of any library), and a
    batch of zero rows is accepted and launches nothing."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    device = torch.device("cuda", 0)
    torch.manual_seed(3)
    config = OrbitQuantConfig(weight_bits=4, activation_bits=4, rotation_seed=5)
    module = OrbitQuantLinear.from_linear(torch.nn.Linear(1024, 512), config=config,
                                          module_name="no_alloc").to(device)
    x = torch.randn(64, 1024, device=device).to(torch.bfloat16)
    out = torch.empty((64, 512), dtype=torch.bfloat16, device=device)
    status, _ = _forward_static(module, x, out=out)     # warm-up: symbol lookup, module load
    assert status == 0
    torch.cuda.synchronize()
    free_before, _total = torch.cuda.mem_get_info(device)
    reserved_before = torch.cuda.memory_reserved(device)
    launches = native.launch_count()
    status, _ = _forward_static(module, x, out=out)
    torch.cuda.synchronize()
    assert status == 0 and native.launch_count() - launches == 2
    assert torch.cuda.mem_get_info(device)[0] == free_before
    assert torch.cuda.memory_reserved(device) == reserved_before
    launches = native.launch_count()
    empty = torch.empty((0, 1024), dtype=torch.bfloat16, device=device)
    status, got = _forward_static(module, empty)
    assert status == 0 and got.shape == (0, 512) and native.launch_count() == launches


def test_static_scratch_rejects_problems_beyond_its_size():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    device = torch.device("cuda", 0)
    config = OrbitQuantConfig(weight_bits=4, activation_bits=4)
    module = OrbitQuantLinear.from_linear(torch.nn.Linear(1024, 64), config=config,
                                          module_name="too_big").to(device)
    x = torch.zeros(4096, 1024, dtype=torch.bfloat16, device=device)   # 8 MiB of activations
    status, _ = _forward_static(module, x)
    assert status == -4
    message = native.load().oq_last_error().decode()
    assert "built-in scratch" in message and "oq_linear_forward" in message
