"""The integer-index formulations: INT8-surrogate matmul and exact pair-product table.

CPU part: the host-side surrogate fit and the oracle restatements against vectors generated
from the reference (``tests/golden/make_int_paths.py``).  GPU part: the CUDA kernels against the
oracle, through the C ABI.

Tolerances: the surrogate fit, the packed / INT8 activation streams and the pair-product kernel
are bit-exact against their oracles.  The surrogate matmul's integer contraction is exact; its
fp32 epilogue multiplies in another order than the oracle, hence rel-L2 <= 1e-5 before the bf16
rounding shows (asserted <= 1e-3 on bf16), and -- being an approximation of the exact centroid
forward by construction -- it is held to the reference's own bound for this path, relative
error <= 3e-2 against the exact forward (reference ``tests/test_kernels.py:1152-1205``).
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import GOLDEN, bf16_from_bits, bits_of, rel_l2
from orbitquant_b200 import (OrbitQuantConfig, OrbitQuantLinear, RPBHRotation, fit_int8_centroid_surrogate,
                             get_codebook, pack_lowbit)


@pytest.fixture(scope="module")
def golden_int_paths():
    return np.load(GOLDEN / "int_paths.npz")


@pytest.mark.parametrize("dim", [768, 3072, 12288])
@pytest.mark.parametrize("bits", [2, 3, 4, 6])
def test_surrogate_fit_equals_reference(golden_int_paths, dim, bits):
    codes, scale = fit_int8_centroid_surrogate(get_codebook(dim, bits).centroids)
    assert codes.dtype == torch.int8
    assert np.array_equal(codes.numpy(), golden_int_paths[f"surrogate_dim{dim}_bits{bits}_codes"])
    assert scale == float(golden_int_paths[f"surrogate_dim{dim}_bits{bits}_scale"])
    with pytest.raises(ValueError):
        fit_int8_centroid_surrogate(torch.linspace(-1, 1, 256))


def _lut_case(golden, name):
    dtype = {"torch.float32": torch.float32, "torch.float16": torch.float16}[
        bytes(golden[name + "_dtype"]).decode()]
    x = torch.from_numpy(golden[name + "_x"].copy()).to(dtype)
    k = x.shape[-1]
    bias = golden[name + "_bias"]
    acb = get_codebook(k, 4)
    return dict(
        x=x, packed=torch.from_numpy(golden[name + "_packed"].copy()),
        row_norms=bf16_from_bits(golden[name + "_row_norms_bits"]),
        bias=None if bias.size == 0 else torch.from_numpy(bias.copy()),
        perm=torch.from_numpy(golden[name + "_perm"].copy()), signs=torch.from_numpy(golden[name + "_signs"].copy()),
        block=int(golden[name + "_block"]), acb=acb,
        lut=(acb.centroids.float()[:, None] * acb.centroids.float()[None, :]).flatten().contiguous(),
        y=torch.from_numpy(golden[name + "_y"].copy()))


@pytest.mark.parametrize("name", ["lut_k256", "lut_k768"])
def test_pair_lut_oracle_matches_reference_function(oracle, golden_int_paths, name):
    """Same table, same indices (the tiny cases hold no value within an ulp of a boundary), sums
    in another order: fp32 summation noise only."""
    c = _lut_case(golden_int_paths, name)
    n = c["row_norms"].numel()
    y, y32 = oracle.pair_lut_linear(c["x"], c["packed"], c["row_norms"], c["bias"], perm=c["perm"],
                                    signs=c["signs"], block=c["block"], act_boundaries=c["acb"].boundaries,
                                    act_centroids=c["acb"].centroids, pair_lut=c["lut"], out_features=n)
    assert y.dtype == c["x"].dtype
    assert rel_l2(y32, c["y"]) < (2e-3 if c["x"].dtype == torch.float16 else 2e-6)
    assert torch.all(y32[2] == (0 if c["bias"] is None else c["bias"]))   # zero token -> bias


# ---- GPU -------------------------------------------------------------------------------------

def _dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,dim,block", [(5, 768, 256), (33, 1024, 1024), (130, 3072, 1024)])
def test_packed_and_int8_activation_streams(oracle, rows, dim, block):
    from orbitquant_b200 import native
    dev = _dev()
    rot = RPBHRotation(dim, 3, block)
    cb = get_codebook(dim, 4)
    x = (torch.randn(rows, dim, generator=torch.Generator().manual_seed(rows)) * 1.3).to(torch.bfloat16)
    x[rows // 2] = 0
    _xq, codes_ref, norms_ref = oracle.quantize_activations(x, rot.permutation, rot.signs, block,
                                                            cb.boundaries, cb.centroids)
    packed, norms = native.quantize_activations_packed_w4(
        x.to(dev), rot.permutation, rot.signs, cb.centroids, cb.boundaries, eps=1e-10, block_size=block)
    assert packed.shape == (rows, dim // 2) and packed.dtype == torch.uint8
    assert torch.equal(packed.cpu().flatten(), pack_lowbit(codes_ref, 4))
    assert torch.equal(norms.cpu(), norms_ref)
    table, _scale = fit_int8_centroid_surrogate(cb.centroids)
    int8_codes, norms2 = native.quantize_activations_int8(
        x.to(dev), rot.permutation, rot.signs, cb.centroids, cb.boundaries, table, eps=1e-10, block_size=block)
    assert int8_codes.dtype == torch.int8
    assert torch.equal(int8_codes.cpu(), table[codes_ref.long()])
    assert torch.equal(norms2.cpu(), norms_ref)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,k,n,w_bits", [(17, 512, 512, 4), (300, 1024, 384, 4), (77, 768, 264, 2),
                                              (40, 768, 200, 3)])
def test_int8_surrogate_matmul(oracle, rows, k, n, w_bits):
    from orbitquant_b200 import native
    dev = _dev()
    torch.manual_seed(rows + k)
    cfg = OrbitQuantConfig(weight_bits=w_bits, activation_bits=4, rotation_seed=6)
    lin = torch.nn.Linear(k, n)
    with torch.no_grad():
        lin.weight.mul_(0.02 / lin.weight.std())
    module = OrbitQuantLinear.from_linear(lin, config=cfg, module_name="s").to(dev)
    x = torch.randn(rows, k)
    x[:, :4] *= 15
    x = x.to(torch.bfloat16)
    exact = module(x.to(dev))
    module.weight_mode = "int8_surrogate"
    native.gemm_clear_device_status()
    got = module(x.to(dev))
    torch.cuda.synchronize()
    assert native.gemm_device_status() == 0
    a_codes, a_scale = fit_int8_centroid_surrogate(module.activation_codebook.centroids)
    w_codes, w_scale = fit_int8_centroid_surrogate(module.weight_codebook.centroids)
    ref, _ref32 = oracle.int8_surrogate_linear(
        x, module.packed_weight_indices.cpu(), module.row_norms.cpu(), module.bias.detach().cpu(),
        perm=module.rotation.permutation, signs=module.rotation.signs, block=module.rotation.block_size,
        act_boundaries=module.activation_codebook.boundaries, act_centroids=module.activation_codebook.centroids,
        act_codes=a_codes, act_scale=a_scale, w_codes=w_codes, w_scale=w_scale, w_bits=w_bits, out_features=n)
    assert rel_l2(got.float().cpu(), ref.float()) <= 1e-3
    assert rel_l2(got.float(), exact.float()) <= 3e-2     # the reference's bound for this path


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["lut_k256", "lut_k768"])
def test_pair_lut_kernel_bit_exact_vs_oracle_and_close_to_reference(oracle, golden_int_paths, name):
    from orbitquant_b200 import native
    dev = _dev()
    c = _lut_case(golden_int_paths, name)
    n = c["row_norms"].numel()
    y = native.linear_w4a4_pair_lut(
        c["x"].to(dev), c["packed"].to(dev), c["row_norms"].to(dev), None if c["bias"] is None else c["bias"].to(dev),
        permutation=c["perm"], signs=c["signs"], block_size=c["block"], act_boundaries=c["acb"].boundaries,
        act_centroids=c["acb"].centroids, pair_lut=c["lut"], out_features=n, eps=1e-10)
    ref, _ = oracle.pair_lut_linear(c["x"], c["packed"], c["row_norms"], c["bias"], perm=c["perm"],
                                    signs=c["signs"], block=c["block"], act_boundaries=c["acb"].boundaries,
                                    act_centroids=c["acb"].centroids, pair_lut=c["lut"], out_features=n)
    assert y.dtype == c["x"].dtype
    assert torch.equal(y.cpu(), ref)
    assert rel_l2(y.float().cpu(), c["y"]) < (2e-3 if c["x"].dtype == torch.float16 else 2e-6)


@pytest.mark.gpu
def test_pair_lut_module_mode_matches_exact_forward(oracle):
    """bf16 module, ragged shape: the table formulation equals the oracle bit for bit.  Against
    the centroid kernels it differs by what those round: they contract bf16(centroid * norm)
    activations (2^-9 relative per value), the table holds fp32 products."""
    dev = _dev()
    torch.manual_seed(4)
    cfg = OrbitQuantConfig(weight_bits=4, activation_bits=4, rotation_seed=1, block_size=128)
    module = OrbitQuantLinear.from_linear(torch.nn.Linear(640, 130), config=cfg, module_name="l").to(dev)
    x = torch.randn(37, 640).to(torch.bfloat16)
    exact = module(x.to(dev))
    module.weight_mode = "pair_lut"
    got = module(x.to(dev))
    lut = (module.activation_codebook.centroids.float()[:, None]
           * module.weight_codebook.centroids.float()[None, :]).flatten()
    ref, _ = oracle.pair_lut_linear(
        x, module.packed_weight_indices.cpu(), module.row_norms.cpu(), module.bias.detach().cpu().float(),
        perm=module.rotation.permutation, signs=module.rotation.signs, block=128,
        act_boundaries=module.activation_codebook.boundaries, act_centroids=module.activation_codebook.centroids,
        pair_lut=lut, out_features=130)
    assert torch.equal(bits_of(got), bits_of(ref))
    assert rel_l2(got.float(), exact.float()) <= 5e-3


@pytest.mark.gpu
@pytest.mark.parametrize("rows,k,n", [(300, 1024, 384), (1100, 768, 840), (2048, 3072, 1024)])
def test_int8_surrogate_matmul_on_int8_tensor_cores(oracle, rows, k, n):
    """Above 128 rows a W4 layer with in_features % 128 == 0 contracts INT8 operands
    (tcgen05.mma kind::i8, int32 accumulation): the integers of the reference's INT8 kernels.
    The same layer through the f16 route (INT8 codes are exact in f16, the fp32 accumulator exact
    below 2^24) must give the same bits."""
    from orbitquant_b200 import native
    dev = _dev()
    torch.manual_seed(rows + n)
    cfg = OrbitQuantConfig(weight_bits=4, activation_bits=4, rotation_seed=3)
    lin = torch.nn.Linear(k, n)
    with torch.no_grad():
        lin.weight.mul_(0.02 / lin.weight.std())
    module = OrbitQuantLinear.from_linear(lin, config=cfg, module_name="i8").to(dev)
    module.weight_mode = "int8_surrogate"
    x = torch.randn(rows, k)
    x[:, :4] *= 15
    x = x.to(torch.bfloat16).to(dev)
    native.gemm_clear_device_status()
    try:
        native.set_tunable("int8_mma", 0)
        via_f16 = module(x)
        native.set_tunable("int8_mma", None)
        via_i8 = module(x)
        torch.cuda.synchronize()
    finally:
        native.set_tunable("int8_mma", None)
    assert native.gemm_device_status() == 0
    assert torch.equal(via_f16, via_i8)
    a_codes, a_scale = fit_int8_centroid_surrogate(module.activation_codebook.centroids)
    w_codes, w_scale = fit_int8_centroid_surrogate(module.weight_codebook.centroids)
    ref, _ref32 = oracle.int8_surrogate_linear(
        x.cpu(), module.packed_weight_indices.cpu(), module.row_norms.cpu(), module.bias.detach().cpu(),
        perm=module.rotation.permutation, signs=module.rotation.signs, block=module.rotation.block_size,
        act_boundaries=module.activation_codebook.boundaries, act_centroids=module.activation_codebook.centroids,
        act_codes=a_codes, act_scale=a_scale, w_codes=w_codes, w_scale=w_scale, w_bits=4, out_features=n)
    assert rel_l2(via_i8.float().cpu(), ref.float()) <= 1e-3


@pytest.mark.gpu
@pytest.mark.parametrize("rows,k,n,block", [(129, 256, 136, 256), (777, 1536, 520, 512), (1500, 2048, 384, 2048),
                                            (515, 4096, 264, 4096), (2048, 3072, 1024, None)])
def test_int8_surrogate_fused_linear_equals_the_two_calls(rows, k, n, block):
    """The fused INT8-surrogate linear (rotate + quantise straight to the INT8 operand, then the
    INT8 tensor-core matmul) against the packed-activation route it shortens
    (quantize_activations_packed_w4 + matmul_packed_w4a4_int8): same indices, same integers, same
    per-token factor, hence the same bits -- for every rotation block the prologue covers,
    including the blocks two and four warps share."""
    from orbitquant_b200 import native
    dev = _dev()
    torch.manual_seed(rows * 3 + n)
    kwargs = {} if block is None else {"block_size": block}
    cfg = OrbitQuantConfig(weight_bits=4, activation_bits=4, rotation_seed=11, **kwargs)
    lin = torch.nn.Linear(k, n)
    with torch.no_grad():
        lin.weight.mul_(0.02 / lin.weight.std())
    module = OrbitQuantLinear.from_linear(lin, config=cfg, module_name="i8f").to(dev)
    module.weight_mode = "int8_surrogate"
    x = torch.randn(rows, k)
    x[:, :4] *= 15
    x[rows // 2] = 0          # a zero token: norm clamps to eps, codes are the middle level
    x = x.to(torch.bfloat16).to(dev)
    assert native.linear_w4a4_int8_supported(x, k, n, module.rotation.block_size)
    native.gemm_clear_device_status()
    fused = module(x)
    assert module.last_activation_kernel_backend == "orbit_b200_int8_surrogate_fused"
    a_codes, a_scale, w_codes, w_scale = module._int8_surrogate_constants(dev)
    packed_x, token_norms = native.quantize_activations_packed_w4(
        x, module._rotation_permutation, module._rotation_signs, module._activation_codebook_centroids,
        module._activation_codebook_boundaries, eps=module.activation_eps,
        block_size=module.rotation.block_size)
    two_calls = native.matmul_packed_w4a4_int8(
        packed_x, module.packed_weight_indices, token_norms, module._row_norms_for(dev), a_codes, w_codes,
        act_scale=a_scale, weight_scale=w_scale, out_features=n, in_features=k, weight_bits=4,
        bias=module._bias_for(dev))
    torch.cuda.synchronize()
    assert native.gemm_device_status() == 0
    assert torch.equal(fused, two_calls)


@pytest.mark.gpu
def test_int8_surrogate_fused_linear_declines_what_it_does_not_cover():
    from orbitquant_b200 import native
    dev = _dev()
    x = torch.zeros(64, 1024, dtype=torch.bfloat16, device=dev)
    assert not native.linear_w4a4_int8_supported(x, 1024, 256, 1024)          # few rows: other kernels
    x = torch.zeros(512, 1024, dtype=torch.float16, device=dev)
    assert not native.linear_w4a4_int8_supported(x, 1024, 256, 1024)          # f16 rows
    x = torch.zeros(512, 1024, dtype=torch.bfloat16, device=dev)
    assert not native.linear_w4a4_int8_supported(x, 1024, 256, 128)           # narrow rotation block
    assert not native.linear_w4a4_int8_supported(x, 1024, 256, 1024, weight_bits=2)
    assert native.linear_w4a4_int8_supported(x, 1024, 256, 1024)
