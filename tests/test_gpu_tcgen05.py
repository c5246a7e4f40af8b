"""The tcgen05/TMEM codebook-decode GEMM (large row counts), through the C ABI, against the
CPU oracle -- and, at the benchmark's full sizes, against the library's own general tiled
kernel and through size-independent properties (linearity in the bias, zero tokens,
determinism, column-shard independence)."""
from __future__ import annotations

import pytest
import torch

from conftest import rel_l2
from orbitquant_b200 import OrbitQuantConfig, OrbitQuantLinear, get_codebook, native, pack_lowbit
from test_gpu_parity import _check_close, _dev, _random_layer

pytestmark = pytest.mark.gpu


def _run(x, packed, rn, cent, n, k, bias, kernel):
    return native.matmul_packed_weight(x, packed, rn, cent, bits=4, out_features=n, in_features=k,
                                       bias=bias, kernel=kernel)


def _assert_status_clean():
    torch.cuda.synchronize()
    assert native.gemm_device_status() == 0, "a bounded wait inside the tcgen05 kernel gave up"


@pytest.mark.parametrize("rows,k,n", [
    (256, 64, 256), (256, 128, 128), (128, 256, 256), (17, 192, 40), (300, 768, 520),
    (513, 3072, 264), (1000, 1024, 1152),
])
def test_tcgen05_vs_oracle(oracle, rows, k, n):
    dev = _dev()
    native.gemm_clear_device_status()
    idx, packed, rn, bias = _random_layer(k, n, 4, seed=rows + k)
    cent = get_codebook(k, 4).centroids
    x = (torch.randn(rows, k) * 1.3).to(torch.bfloat16)
    y = _run(x.to(dev), packed.to(dev), rn, cent, n, k, bias, native.KERNEL_TCGEN05)
    _assert_status_clean()
    ref = oracle.matmul_packed(x, packed, rn, cent, bits=4, out_features=n, bias=bias,
                                  mode=oracle.MM_FP32_CENTROIDS)
    _check_close(y, ref, (rows, k, n))


@pytest.mark.parametrize("tile_n", ["128", "192", "256"])
def test_tcgen05_every_tile_width(oracle, tile_n, tunables):
    dev = _dev()
    tunables.set("tile_n", int(tile_n))
    native.gemm_clear_device_status()
    rows, k, n = 520, 512, 840          # ragged in M and in N for every width
    idx, packed, rn, bias = _random_layer(k, n, 4, seed=int(tile_n))
    cent = get_codebook(k, 4).centroids
    x = (torch.randn(rows, k) * 0.7).to(torch.bfloat16)
    y = _run(x.to(dev), packed.to(dev), rn, cent, n, k, bias, native.KERNEL_TCGEN05)
    _assert_status_clean()
    ref = oracle.matmul_packed(x, packed, rn, cent, bits=4, out_features=n, bias=bias,
                                  mode=oracle.MM_FP32_CENTROIDS)
    _check_close(y, ref, ("tile", tile_n))


@pytest.mark.parametrize("tile_n", ["128", "192", "256"])
@pytest.mark.parametrize("bits", [2, 3, 6, 8])
def test_tcgen05_other_bit_widths(oracle, golden_codebooks, bits, tile_n, tunables):
    """2/3-bit tables decode through register byte-permutes, 6/8-bit through a shared-memory
    table; 3-bit tiles are the one width the expanders fetch from global memory themselves."""
    from conftest import codebook_from_golden
    dev = _dev()
    tunables.set("tile_n", int(tile_n))
    native.gemm_clear_device_status()
    rows, k, n = 300, 768, 456
    idx, packed, rn, bias = _random_layer(k, n, bits, seed=bits * 11)
    cent = (codebook_from_golden(golden_codebooks, k, 8) if bits == 8 else get_codebook(k, bits)).centroids
    x = (torch.randn(rows, k) * 0.9).to(torch.bfloat16)
    y = native.matmul_packed_weight(x.to(dev), packed.to(dev), rn, cent, bits=bits, out_features=n,
                                    in_features=k, bias=bias, kernel=native.KERNEL_TCGEN05)
    _assert_status_clean()
    ref = oracle.matmul_packed(x, packed, rn, cent, bits=bits, out_features=n, bias=bias,
                                  mode=oracle.MM_FP32_CENTROIDS)
    _check_close(y, ref, ("bits", bits, "tile", tile_n))


def test_mixed_bit_modules_use_the_tensor_core_kernel(oracle):
    """The mixed-bit policy shapes (W2A4 for Q/K, W3A3 elsewhere) at a row count that takes
    the tcgen05 kernel by default."""
    dev = _dev()
    torch.manual_seed(21)
    for wb, ab in ((2, 4), (3, 3)):
        cfg = OrbitQuantConfig(weight_bits=wb, activation_bits=ab, rotation_seed=2)
        lin = torch.nn.Linear(3072, 384)
        with torch.no_grad():
            lin.weight.mul_(0.02 / lin.weight.std())
        module = OrbitQuantLinear.from_linear(lin, config=cfg, module_name="mixed").to(dev)
        x = torch.randn(260, 3072)
        x[:, :15] *= 20
        x = x.to(torch.bfloat16)
        assert native.load().oq_gemm_tcgen05_supported(260, 3072, 384, wb, 2, 0) == 1
        y = module(x.to(dev))
        _assert_status_clean()
        ref = oracle.linear_forward(
            x, module.packed_weight_indices.cpu(), module.row_norms.cpu(), module.bias.detach().cpu(),
            perm=module.rotation.permutation, signs=module.rotation.signs,
            block=module.rotation.block_size, act_boundaries=module.activation_codebook.boundaries,
            act_centroids=module.activation_codebook.centroids,
            w_centroids=module.weight_codebook.centroids, w_bits=wb, out_features=384)
        _check_close(y, ref, ("mixed", wb, ab))


def test_f16_operand_rescaling_is_exact():
    """Token scales spanning 2^-40 .. 2^40 must not change the result beyond the scale."""
    dev = _dev()
    k, n, rows = 256, 64, 40
    idx, packed, rn, _ = _random_layer(k, n, 4, seed=3, bias=False)
    cent = get_codebook(k, 4).centroids
    base = torch.randn(rows, k).to(torch.bfloat16)
    scales = torch.tensor([2.0 ** e for e in range(-40, 40, 2)])[:, None]
    y1 = _run(base.to(dev), packed.to(dev), rn, cent, n, k, None, native.KERNEL_TCGEN05).float().cpu()
    y2 = _run((base.float() * scales).to(torch.bfloat16).to(dev), packed.to(dev), rn, cent, n, k, None,
              native.KERNEL_TCGEN05).float().cpu()
    assert torch.allclose(y2 / scales, y1, rtol=1e-2, atol=0)   # bf16 output rounding only
    operand, factor, _ = native.rows_to_f16_operand(base.to(dev))
    assert torch.equal((operand.float() * factor[:, None]).cpu(), base.float())


def test_tcgen05_structured_inputs_catch_layout_errors():
    """One-hot activations pick out single weight columns, so any swizzle / descriptor /
    nibble-order mistake shows up as a wrong exact value rather than as noise."""
    dev = _dev()
    k, n, rows = 256, 256, 256
    idx, packed, rn, _ = _random_layer(k, n, 4, seed=77, bias=False)
    cent = get_codebook(k, 4).centroids
    x = torch.zeros(rows, k)
    x[torch.arange(rows), torch.arange(rows) % k] = 1.0
    y = _run(x.to(torch.bfloat16).to(dev), packed.to(dev), rn, cent, n, k, None, native.KERNEL_TCGEN05)
    _assert_status_clean()
    w = rn.float()[:, None] * cent[idx.long().reshape(n, k)]      # [n, k]
    expect = w.T[torch.arange(rows) % k]                             # row m = column (m % k) of W
    assert rel_l2(y.float().cpu(), expect) < 4e-3                    # bf16 output rounding only
    assert float((y.float().cpu() - expect).abs().max()) < 1e-2


@pytest.mark.parametrize("rows,k,n", [(4608, 3072, 3072), (4608, 3072, 9216), (4608, 12288, 3072),
                                      (32760, 5120, 5120)])
def test_tcgen05_full_size_properties(rows, k, n):
    dev = _dev()
    native.gemm_clear_device_status()
    g = torch.Generator().manual_seed(k + n)
    packed = torch.randint(0, 256, (n * k // 2,), generator=g, dtype=torch.uint8).to(dev)
    rn = (torch.rand(n, generator=g) + 0.5).to(torch.bfloat16).to(dev)
    cent = get_codebook(k, 4).centroids.to(dev)
    x = torch.randn(rows, k, generator=g).to(torch.bfloat16).to(dev)
    x[5] = 0
    bias = torch.randn(n, generator=g).to(dev)
    y0 = _run(x, packed, rn, cent, n, k, None, native.KERNEL_TCGEN05)
    y0_again = _run(x, packed, rn, cent, n, k, None, native.KERNEL_TCGEN05)
    yb = _run(x, packed, rn, cent, n, k, bias, native.KERNEL_TCGEN05)
    _assert_status_clean()
    assert torch.equal(y0, y0_again)                                  # deterministic
    assert torch.all(y0[5] == 0)                                      # zero token -> zero
    assert torch.equal(yb[5].float(), bias.to(torch.bfloat16).float())  # ... or exactly the bias
    # a row subset through the general kernel (independent code path, same arithmetic class)
    pick = torch.tensor([0, 1, 127, 128, 255, 256, rows // 2, rows - 2, rows - 1], device=dev)
    y_ref = _run(x[pick].contiguous(), packed, rn, cent, n, k, bias, native.KERNEL_TILED)
    _check_close(yb[pick], y_ref, ("full-size rows", rows, k, n))
    # column shards are independent: the second half of N computed alone equals the slice
    half = n // 2
    y_half = _run(x, packed[half * k // 2:], rn[half:], cent, n - half, k, bias[half:],
                  native.KERNEL_TCGEN05)
    _assert_status_clean()
    assert torch.equal(y_half, yb[:, half:])


def test_module_auto_dispatch_uses_tcgen05(oracle):
    dev = _dev()
    torch.manual_seed(8)
    cfg = OrbitQuantConfig(weight_bits=4, activation_bits=4, block_size=256, rotation_seed=0)
    lin = torch.nn.Linear(3072, 512)
    with torch.no_grad():
        lin.weight.mul_(0.02 / lin.weight.std())
    module = OrbitQuantLinear.from_linear(lin, config=cfg, module_name="t").to(dev)
    x = torch.randn(300, 3072)
    x[:, :8] *= 20
    x = x.to(torch.bfloat16)
    before = native.launch_count()
    y = module(x.to(dev))
    assert native.launch_count() - before == 2                       # prologue + GEMM
    _assert_status_clean()
    ref = oracle.linear_forward(
        x, module.packed_weight_indices.cpu(), module.row_norms.cpu(), module.bias.detach().cpu(),
        perm=module.rotation.permutation, signs=module.rotation.signs, block=256,
        act_boundaries=module.activation_codebook.boundaries,
        act_centroids=module.activation_codebook.centroids,
        w_centroids=module.weight_codebook.centroids, w_bits=4, out_features=512)
    _check_close(y, ref, "module W4A4 config-1 slice")


@pytest.mark.parametrize("bits,rows,k,n", [(4, 300, 1024, 1152), (4, 1000, 3072, 520), (3, 260, 768, 456),
                                           (2, 515, 768, 456)])
def test_tcgen05_bf16_scaled_operand(oracle, bits, rows, k, n):
    """The reference's other weight arithmetic on the tensor cores: operand
    bf16(centroid * row_norm) against the bf16 activations.  Same operands as the oracle's
    bf16 table mode, so only the fp32 summation order differs."""
    dev = _dev()
    idx, packed, rn, bias = _random_layer(k, n, bits, seed=bits * 7 + rows)
    cent = get_codebook(k, bits).centroids
    x = (torch.randn(rows, k) * 0.9).to(torch.bfloat16)
    native.gemm_clear_device_status()
    y = native.matmul_packed_weight(x.to(dev), packed.to(dev), rn, cent, bits=bits, out_features=n,
                                    in_features=k, bias=bias, kernel=native.KERNEL_TCGEN05,
                                    weight_mode=native.WEIGHT_BF16_SCALED)
    _assert_status_clean()
    ref = oracle.matmul_packed(x, packed, rn, cent, bits=bits, out_features=n, bias=bias,
                               mode=oracle.MM_BF16_LUT)
    _check_close(y, ref, ("bf16_scaled", bits, rows, k, n))
    assert rel_l2(y.float().cpu(), ref[0].float()) < 3e-4


@pytest.mark.parametrize("pair_width", [192, 256])
@pytest.mark.parametrize("bits,scaled", [(4, False), (3, False), (2, False), (4, True), (3, True)])
def test_tcgen05_cta_pair_kernel(oracle, pair_width, bits, scaled, tunables):
    """The cta_group::2 variant (two CTAs share every expanded weight tile): against the oracle
    on a shape that is ragged in M (the pair's second CTA is partly, then wholly, out of range)
    and in N, and bit for bit against the single-CTA kernel -- both accumulate the same products
    in the same order."""
    dev = _dev()
    rows, k, n = 1100, 768, 840
    idx, packed, rn, bias = _random_layer(k, n, bits, seed=bits * 5 + pair_width)
    cent = get_codebook(k, bits).centroids
    x = (torch.randn(rows, k) * 0.8).to(torch.bfloat16)
    mode = native.WEIGHT_BF16_SCALED if scaled else native.WEIGHT_CENTROID
    kw = dict(bits=bits, out_features=n, in_features=k, bias=bias, kernel=native.KERNEL_TCGEN05,
              weight_mode=mode)
    native.gemm_clear_device_status()
    tunables.set("pair", 0)
    single = native.matmul_packed_weight(x.to(dev), packed.to(dev), rn, cent, **kw)
    tunables.set("pair", pair_width)
    launches = native.launch_count()
    paired = native.matmul_packed_weight(x.to(dev), packed.to(dev), rn, cent, **kw)
    assert native.launch_count() > launches
    _assert_status_clean()
    assert torch.equal(single, paired)
    ref = oracle.matmul_packed(x, packed, rn, cent, bits=bits, out_features=n, bias=bias,
                               mode=oracle.MM_BF16_LUT if scaled else oracle.MM_FP32_CENTROIDS)
    _check_close(paired, ref, ("pair", pair_width, bits, scaled))


@pytest.mark.parametrize("pair", [0, 256])
def test_tcgen05_table_without_sign_symmetry(oracle, pair, tunables):
    """Lloyd-Max tables are sign-symmetric and take the short 4-bit decode; any other table
    must take the general one and give the same kind of answer."""
    dev = _dev()
    rows, k, n = 600, 512, 520
    idx, packed, rn, bias = _random_layer(k, n, 4, seed=77)
    cent = get_codebook(k, 4).centroids.clone()
    cent[3] *= 1.07              # breaks entry 3 = -entry 12
    cent = torch.sort(cent).values
    assert not torch.equal(cent, -cent.flip(0))
    x = (torch.randn(rows, k) * 0.8).to(torch.bfloat16)
    tunables.set("pair", pair)
    native.gemm_clear_device_status()
    y = native.matmul_packed_weight(x.to(dev), packed.to(dev), rn, cent, bits=4, out_features=n,
                                    in_features=k, bias=bias, kernel=native.KERNEL_TCGEN05)
    _assert_status_clean()
    ref = oracle.matmul_packed(x, packed, rn, cent, bits=4, out_features=n, bias=bias,
                               mode=oracle.MM_FP32_CENTROIDS)
    _check_close(y, ref, ("asymmetric table", pair))


def test_tcgen05_cta_pair_hand_over_under_load(tunables):
    """Several waves of pair tiles, launched back to back many times: every k step of every tile
    hands the peer CTA's half of the weight tile to the leader's MMAs; a hand-over that let the
    MMAs read a half-written tile would show as a difference from the single-CTA kernel's bits."""
    dev = _dev()
    rows, k, n = 2560, 1024, 4608
    g = torch.Generator().manual_seed(5)
    packed = torch.randint(0, 256, (k * n // 2,), generator=g, dtype=torch.uint8).to(dev)
    rn = (torch.rand(n, generator=g) + 0.5).to(torch.bfloat16).to(dev)
    cent = get_codebook(k, 4).centroids.to(dev)
    x = torch.randn(rows, k, generator=g).to(torch.bfloat16).to(dev)
    op, scale, table = native.rows_to_f16_operand(x, cent)
    native.gemm_clear_device_status()
    tunables.set("pair", 0)
    ref = torch.empty(rows, n, dtype=torch.bfloat16, device=dev)
    native.gemm_tcgen05_f16(op, scale, packed, rn, cent, out_features=n, out=ref, table_scale=table)
    for width in (256, 192):
        tunables.set("pair", width)
        outs = [torch.empty_like(ref) for _ in range(8)]
        for rep in range(40):
            native.gemm_tcgen05_f16(op, scale, packed, rn, cent, out_features=n, out=outs[rep % 8],
                                    table_scale=table)
            if rep % 8 == 7:
                torch.cuda.synchronize()
                assert all(torch.equal(o, ref) for o in outs), (width, rep)
    _assert_status_clean()
