"""Parity of the CUDA path (called through the C ABI) against the CPU oracle and the
reference's golden vectors.  Everything here needs a B200.

Tolerances (bf16 activations/outputs):
* bit streams, activation codes, token norms and quantised activations: bit-exact;
* matmul / forward outputs: rel-L2 <= 1e-3 on the bf16 outputs, and max-abs <= 2e-2 in units
  of the output RMS on the value BEFORE the final bf16 rounding, against the oracle
  evaluated with the SAME weight arithmetic (fp32 centroids for ``centroid`` mode,
  bf16(c*row_norm) for ``bf16_scaled``).  The oracle returns its fp32 value before that
  rounding; the kernels return bf16 only, so the assertion is
  ``|y_gpu - y_ref_f32| <= 2e-2 * rms + ulp_bf16(y_gpu) / 2`` (the half ulp is the most the
  device's own final rounding can add).  Where the reference side is rounded too (the
  compiled reference kernels return bf16), one whole ulp is allowed instead: one bf16 ulp
  at |y| >= 4 is 0.031, more than the tolerance itself.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import bf16_from_bits, bits_of, codebook_from_golden, rel_l2
from orbitquant_b200 import (OrbitQuantConfig, OrbitQuantLinear, RPBHRotation, get_codebook, native,
                             pack_lowbit, unpack_lowbit)

pytestmark = pytest.mark.gpu

REL_L2_TOL = 1e-3
MAX_ABS_TOL = 2e-2


def _dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)


def bf16_ulp(values: torch.Tensor) -> torch.Tensor:
    """Spacing of bf16 numbers at the magnitude of ``values`` (8 significant bits)."""
    mag = values.abs().double().clamp_min(2.0 ** -126)
    return torch.exp2(torch.floor(torch.log2(mag)) - 7)


def parity_errors(y_gpu: torch.Tensor, y_ref):
    """(rel-L2, max-abs of the rounded outputs, excess of the pre-rounding difference over the
    half ulp the final rounding may add), the last two in units of the reference's RMS.
    ``y_ref`` is the reference output, or the oracle's pair (rounded output, fp32 value
    before the final rounding)."""
    y_ref, y_ref_f32 = y_ref if isinstance(y_ref, tuple) else (y_ref, None)
    y_gpu = y_gpu.detach().float().cpu()
    y_ref = y_ref.detach().float().cpu()
    rms = y_ref.pow(2).mean().sqrt().clamp_min(1e-12).double()
    err = rel_l2(y_gpu, y_ref)
    max_abs = float(((y_gpu - y_ref).abs().double() / rms).max())
    if y_ref_f32 is not None:
        # the device rounds its own fp32 value to bf16 (at most half an ulp away from it)
        y32 = y_ref_f32.detach().double().cpu()
        excess = ((y_gpu.double() - y32).abs() - 0.5 * bf16_ulp(y_gpu)).clamp_min(0) / rms
    else:
        # both sides are rounded: two values that differ by less than the tolerance before
        # rounding can land one ulp apart
        excess = ((y_gpu - y_ref).abs().double() - bf16_ulp(torch.maximum(y_gpu.abs(), y_ref.abs()))
                  ).clamp_min(0) / rms
    return err, max_abs, float(excess.max())


def _check_close(y_gpu: torch.Tensor, y_ref, what):
    """rel-L2 <= 1e-3 on the bf16 outputs and max-abs <= 2e-2 (unit RMS) on the values before
    the final bf16 rounding; see the module docstring."""
    ref_out = y_ref[0] if isinstance(y_ref, tuple) else y_ref
    assert y_gpu.shape == ref_out.shape, what
    assert torch.isfinite(y_gpu.detach().float()).all(), what
    err, max_abs, pre_rounding = parity_errors(y_gpu, y_ref)
    assert err <= REL_L2_TOL, (what, "rel-L2", err)
    assert pre_rounding <= MAX_ABS_TOL, (what, "max-abs before rounding / rms", pre_rounding,
                                         "max-abs of the bf16 outputs / rms", max_abs)


def _random_layer(k, n, bits, seed, bias=True):
    g = torch.Generator().manual_seed(seed)
    idx = torch.randint(0, 2 ** bits, (n * k,), generator=g, dtype=torch.uint8)
    packed = pack_lowbit(idx, bits)
    row_norms = (torch.rand(n, generator=g) * 1.5 + 0.25).to(torch.bfloat16)
    b = torch.randn(n, generator=g) * 0.5 if bias else None
    return idx, packed, row_norms, b


# ---- bit stream ---------------------------------------------------------------------------

@pytest.mark.parametrize("bits", [1, 2, 3, 4, 5, 6, 7, 8])
def test_pack_unpack_bit_exact(bits, golden_bitpack):
    dev = _dev()
    for length in (1, 7, 64, 1003):
        values = torch.from_numpy(golden_bitpack[f"bits{bits}_len{length}_values"].copy())
        packed = torch.from_numpy(golden_bitpack[f"bits{bits}_len{length}_packed"].copy())
        assert torch.equal(native.pack_lowbit(values.to(dev), bits).cpu(), packed)
        assert torch.equal(native.unpack_lowbit(packed.to(dev), bits, length).cpu(), values)
    big = torch.randint(0, 2 ** bits, (1_000_003,), dtype=torch.uint8)
    packed = pack_lowbit(big, bits)
    assert torch.equal(native.pack_lowbit(big.to(dev), bits).cpu(), packed)
    assert torch.equal(native.unpack_lowbit(packed.to(dev), bits, big.numel()).cpu(), big)
    assert native.unpack_lowbit(packed.to(dev), bits, 0).numel() == 0
    with pytest.raises(ValueError):
        native.pack_lowbit(torch.full((4,), 2 ** bits, dtype=torch.int32, device=dev), bits)


def test_dequantize_weight_bit_exact(oracle):
    dev = _dev()
    for bits, k, n in ((4, 768, 40), (3, 256, 33), (2, 512, 16), (6, 256, 9), (8, 128, 5)):
        idx, packed, rn, _ = _random_layer(k, n, bits, seed=bits)
        cent = torch.linspace(-0.9, 0.9, 2 ** bits)
        w = native.dequantize_packed_weight(packed.to(dev), rn.to(dev), cent.to(dev), bits=bits,
                                            out_features=n, in_features=k, dtype=torch.float32)
        expect = rn.float()[:, None] * cent[idx.long().reshape(n, k)]
        assert torch.equal(w.cpu(), expect)


# ---- prologue -----------------------------------------------------------------------------

PROLOGUE_CASES = [
    # rows, dim, block, bits, seed
    (1, 768, 256, 6, 4), (4, 768, 256, 6, 4), (16, 768, 256, 6, 4),
    (37, 3072, 256, 4, 0), (64, 3072, 1024, 4, 1), (9, 5120, 1024, 4, 3),
    (5, 12288, 4096, 4, 1), (3, 13824, 512, 4, 3), (300, 3072, 1024, 3, 2),
    (17, 1024, 64, 2, 9), (8, 512, 512, 8, 6), (6, 2048, 2048, 4, 7), (5, 192, 64, 4, 8),
    (3, 16384, 16384, 4, 5), (2, 96, 32, 3, 1),
]


@pytest.mark.parametrize("rows,dim,block,bits,seed", PROLOGUE_CASES)
def test_prologue_bit_exact_vs_oracle(oracle, golden_codebooks, rows, dim, block, bits, seed):
    dev = _dev()
    rot = RPBHRotation(dim, seed, block)
    if bits == 8:
        cb = codebook_from_golden(golden_codebooks, 256, 8)  # any valid 8-bit table
    else:
        cb = get_codebook(dim, bits)
    g = torch.Generator().manual_seed(seed + 100)
    x = torch.randn(rows, dim, generator=g) * (torch.rand(rows, 1, generator=g) * 3 + 0.1)
    x[:, : max(1, dim // 200)] *= 20
    if rows > 2:
        x[rows // 2] = 0
    x = x.to(torch.bfloat16)
    xq_ref, codes_ref, norms_ref = oracle.quantize_activations(
        x, rot.permutation, rot.signs, block, cb.boundaries, cb.centroids, eps=1e-10,
        norm_order=oracle.NORM_AVX512)
    xq, codes, norms = native.quantize_activations(
        x.to(dev), rot.permutation, rot.signs, cb.centroids, cb.boundaries, eps=1e-10,
        block_size=block, return_codes=True, return_norms=True)
    assert torch.equal(norms.cpu(), norms_ref), "token norms differ"
    assert torch.equal(codes.cpu(), codes_ref), "activation codes differ"
    assert torch.equal(bits_of(xq), bits_of(xq_ref)), "quantised activations differ"
    if rows > 2:
        assert torch.all(xq[rows // 2] == 0)
    # without the side outputs the specialised kernel runs (bf16, dim % 256 == 0, block >= 256)
    xq_only = native.quantize_activations(x.to(dev), rot.permutation, rot.signs, cb.centroids,
                                          cb.boundaries, eps=1e-10, block_size=block)
    assert torch.equal(bits_of(xq_only), bits_of(xq_ref)), "specialised kernel differs"


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_prologue_other_dtypes(oracle, dtype):
    dev = _dev()
    rot = RPBHRotation(1024, 2, 256)
    cb = get_codebook(1024, 4)
    x = (torch.randn(11, 1024) * 2).to(dtype)
    ref, codes_ref, _ = oracle.quantize_activations(x, rot.permutation, rot.signs, 256,
                                                    cb.boundaries, cb.centroids)
    got, codes = native.quantize_activations(x.to(dev), rot.permutation, rot.signs, cb.centroids,
                                             cb.boundaries, eps=1e-10, block_size=256,
                                             return_codes=True)
    assert torch.equal(codes.cpu(), codes_ref)
    assert torch.equal(got.cpu(), ref)


def test_prologue_golden_reference_vectors(golden_layers, golden_codebooks):
    """Bit-exact against what the reference's own AVX-512 CPU kernel produced."""
    dev = _dev()
    for name in (str(n) for n in golden_layers["case_names"]):
        m, k, n, wb, ab, block, seed = (int(v) for v in golden_layers[f"{name}_meta"])
        rot = RPBHRotation(k, seed, block)
        cb = codebook_from_golden(golden_codebooks, k, ab) if ab == 8 else get_codebook(k, ab)
        x = bf16_from_bits(golden_layers[f"{name}_x"])
        xq = native.quantize_activations(x.to(dev), rot.permutation, rot.signs, cb.centroids,
                                         cb.boundaries, eps=1e-10, block_size=block)
        expect = golden_layers[f"{name}_xq_native_avx512"]
        assert np.array_equal(bits_of(xq).numpy().astype(np.uint16), expect), name


def test_prologue_empty_and_errors():
    dev = _dev()
    rot = RPBHRotation(256, 0, 256)
    cb = get_codebook(256, 4)
    out = native.quantize_activations(torch.empty(0, 256, dtype=torch.bfloat16, device=dev),
                                      rot.permutation, rot.signs, cb.centroids, cb.boundaries,
                                      eps=1e-10, block_size=256)
    assert out.shape == (0, 256)
    with pytest.raises(ValueError):
        native.quantize_activations(torch.zeros(2, 256, device=dev), rot.permutation, rot.signs,
                                    cb.centroids, cb.boundaries, eps=1e-10, block_size=96)
    with pytest.raises(RuntimeError):
        native.quantize_activations(torch.zeros(2, 256), rot.permutation, rot.signs,
                                    cb.centroids, cb.boundaries, eps=1e-10, block_size=256)


# ---- packed matmul kernels ------------------------------------------------------------------

def _oracle_matmul(oracle, x, packed, rn, cent, bits, n, bias, mode_name):
    mode = oracle.MM_BF16_LUT if mode_name == "bf16_scaled" else oracle.MM_FP32_CENTROIDS
    y = oracle.matmul_packed(x, packed, rn, cent, bits=bits, out_features=n, bias=bias, mode=mode)
    return y


@pytest.mark.parametrize("mode", ["centroid", "bf16_scaled"])
@pytest.mark.parametrize("bits,rows,k,n", [
    (4, 1, 768, 96), (4, 16, 768, 100), (4, 33, 200, 70), (3, 19, 768, 65), (2, 40, 512, 130),
    (6, 7, 256, 33), (8, 5, 128, 17), (5, 3, 96, 9),
])
def test_tiled_kernel_vs_oracle(oracle, mode, bits, rows, k, n):
    dev = _dev()
    idx, packed, rn, bias = _random_layer(k, n, bits, seed=bits * 7 + rows)
    cent = get_codebook(max(k, 32), bits).centroids if bits in (2, 3, 4, 6) else torch.linspace(-0.2, 0.2, 2 ** bits)
    x = torch.randn(rows, k).to(torch.bfloat16)
    y = native.matmul_packed_weight(x.to(dev), packed.to(dev), rn, cent, bits=bits, out_features=n,
                                    in_features=k, bias=bias,
                                    weight_mode=native.WEIGHT_MODE_NAMES[mode],
                                    kernel=native.KERNEL_TILED)
    _check_close(y, _oracle_matmul(oracle, x, packed, rn, cent, bits, n, bias, mode), (mode, bits, rows))


@pytest.mark.parametrize("mode", ["centroid", "bf16_scaled"])
@pytest.mark.parametrize("rows", [1, 2, 4, 7, 8, 9, 15, 16])
def test_small_rows_kernel_vs_oracle(oracle, mode, rows):
    dev = _dev()
    for k, n, with_bias in ((768, 2304, True), (768, 61, False), (3072, 520, True), (128, 8, True)):
        idx, packed, rn, bias = _random_layer(k, n, 4, seed=rows + n, bias=with_bias)
        cent = get_codebook(k, 4).centroids
        x = (torch.randn(rows, k) * 1.5).to(torch.bfloat16)
        y = native.matmul_packed_weight(x.to(dev), packed.to(dev), rn, cent, bits=4, out_features=n,
                                        in_features=k, bias=bias,
                                        weight_mode=native.WEIGHT_MODE_NAMES[mode],
                                        kernel=native.KERNEL_SMALL_ROWS)
        _check_close(y, _oracle_matmul(oracle, x, packed, rn, cent, 4, n, bias, mode), (mode, rows, k, n))


def test_small_rows_and_tiled_agree_and_are_deterministic():
    dev = _dev()
    idx, packed, rn, bias = _random_layer(768, 2304, 4, seed=5)
    cent = get_codebook(768, 4).centroids
    x = torch.randn(16, 768).to(torch.bfloat16).to(dev)
    a = native.matmul_packed_weight(x, packed.to(dev), rn, cent, bits=4, out_features=2304,
                                    in_features=768, bias=bias, kernel=native.KERNEL_SMALL_ROWS)
    b = native.matmul_packed_weight(x, packed.to(dev), rn, cent, bits=4, out_features=2304,
                                    in_features=768, bias=bias, kernel=native.KERNEL_SMALL_ROWS)
    c = native.matmul_packed_weight(x, packed.to(dev), rn, cent, bits=4, out_features=2304,
                                    in_features=768, bias=bias, kernel=native.KERNEL_TILED)
    assert torch.equal(a, b)
    _check_close(a, c, "small_rows vs tiled")


@pytest.mark.parametrize("mode", ["centroid", "bf16_scaled"])
@pytest.mark.parametrize("rows,k,n,with_bias", [
    (1, 3072, 3072, True),      # one k range, epilogue inside the kernel
    (16, 3072, 9216, True),
    (5, 12288, 1030, False),    # several k ranges, ragged last 8-row block
    (9, 4736, 1536, True),      # 37 k steps: the last range is shorter than the others
    (16, 13824, 1024, True),
])
def test_streaming_small_rows_kernel_vs_oracle(oracle, mode, rows, k, n, with_bias):
    """Layers of a few megabytes and more take the persistent weight-streaming kernel
    (same C entry point, chosen by size)."""
    dev = _dev()
    idx, packed, rn, bias = _random_layer(k, n, 4, seed=rows + n, bias=with_bias)
    cent = get_codebook(k, 4).centroids
    x = (torch.randn(rows, k) * 1.5).to(torch.bfloat16)
    args = dict(bits=4, out_features=n, in_features=k, bias=bias,
                weight_mode=native.WEIGHT_MODE_NAMES[mode], kernel=native.KERNEL_SMALL_ROWS)
    y = native.matmul_packed_weight(x.to(dev), packed.to(dev), rn, cent, **args)
    _check_close(y, _oracle_matmul(oracle, x, packed, rn, cent, 4, n, bias, mode), (mode, rows, k, n))
    again = native.matmul_packed_weight(x.to(dev), packed.to(dev), rn, cent, **args)
    assert torch.equal(y, again), "not deterministic"


def test_matmul_argument_errors():
    dev = _dev()
    x = torch.zeros(4, 64, dtype=torch.bfloat16, device=dev)
    packed = torch.zeros(8 * 64 // 2, dtype=torch.uint8, device=dev)
    rn = torch.ones(8, dtype=torch.bfloat16)
    cent = torch.zeros(16)
    with pytest.raises(ValueError, match="too short"):
        native.matmul_packed_weight(x, packed[:-1], rn, cent, bits=4, out_features=8, in_features=64)
    with pytest.raises(ValueError):
        native.matmul_packed_weight(x, packed, rn, cent, bits=4, out_features=8, in_features=32)
    with pytest.raises(ValueError):
        native.matmul_packed_weight(x, packed, rn, cent, bits=0, out_features=8, in_features=64)
    with pytest.raises(RuntimeError, match="tcgen05"):
        native.matmul_packed_weight(x.float(), packed, rn, cent, bits=4, out_features=8,
                                    in_features=64, kernel=native.KERNEL_TCGEN05)
    y = native.matmul_packed_weight(x[:0], packed, rn, cent, bits=4, out_features=8, in_features=64)
    assert y.shape == (0, 8)


# ---- the module, golden layers, compile, graphs -------------------------------------------------

def _module_from_golden(golden_layers, golden_codebooks, name, dev):
    m, k, n, wb, ab, block, seed = (int(v) for v in golden_layers[f"{name}_meta"])
    if wb == 8 or ab == 8:
        return None, None, None
    cfg = OrbitQuantConfig(weight_bits=wb, activation_bits=ab, block_size=block, rotation_seed=seed)
    bias = (torch.from_numpy(golden_layers[f"{name}_bias"].copy())
            if f"{name}_bias" in golden_layers else None)
    module = OrbitQuantLinear(
        in_features=k, out_features=n, config=cfg, module_name=name, source_weight_layout="out_in",
        bias=bias, packed_weight_indices=torch.from_numpy(golden_layers[f"{name}_packed"].copy()),
        row_norms=bf16_from_bits(golden_layers[f"{name}_row_norms"]), debug_weight=None).to(dev)
    x = bf16_from_bits(golden_layers[f"{name}_x"]).to(dev)
    return module, x, (m, k, n)


def test_module_forward_matches_reference_golden_outputs(golden_layers, golden_codebooks):
    """Against the reference's compiled CPU kernels (scalar ISA = fp32-centroid arithmetic)
    on the reference's own packed weights."""
    dev = _dev()
    for name in (str(n) for n in golden_layers["case_names"]):
        module, x, shape = _module_from_golden(golden_layers, golden_codebooks, name, dev)
        if module is None:
            continue
        y = module(x)
        ref = bf16_from_bits(golden_layers[f"{name}_y_native_scalar"])
        # the scalar reference reduced the token norm in sequential order; its activations
        # can differ from the AVX-512 order by a few bucket flips, which these tiny layers
        # (N <= 48) do not average out -> compare loosely here, tightly in the next test
        assert rel_l2(y.float().cpu(), ref.float()) < 2e-2, name
        if f"{name}_bias" in golden_layers:
            assert torch.equal(y[-1].float().cpu(),
                               torch.from_numpy(golden_layers[f"{name}_bias"].copy()).to(torch.bfloat16).float()), name
        else:
            assert torch.all(y[-1] == 0), name


def test_module_forward_vs_oracle_all_bit_pairs(oracle, golden_codebooks):
    dev = _dev()
    torch.manual_seed(3)
    for (wb, ab, k, n, m, block) in ((4, 4, 768, 256, 40, "paper"), (3, 3, 768, 128, 24, "paper"),
                                     (2, 4, 1024, 96, 17, 256), (4, 6, 768, 2304, 16, "paper"),
                                     (6, 6, 512, 64, 9, 128), (2, 3, 1536, 72, 12, "paper"),
                                     (4, 4, 3072, 512, 300, 256)):
        cfg = OrbitQuantConfig(weight_bits=wb, activation_bits=ab, block_size=block, rotation_seed=wb)
        lin = torch.nn.Linear(k, n)
        with torch.no_grad():
            lin.weight.mul_(0.02 / lin.weight.std())
        module = OrbitQuantLinear.from_linear(lin, config=cfg, module_name="t").to(dev)
        if m > 16:
            module.kernel = "tiled"  # the tcgen05 kernel has its own test file
        x = torch.randn(2, m // 2, k)
        x[..., :6] *= 20
        x = x.to(torch.bfloat16)
        y = module(x.to(dev))
        assert y.shape == (2, m // 2, n) and y.dtype == torch.bfloat16
        ref = oracle.linear_forward(
            x, module.packed_weight_indices.cpu(), module.row_norms.cpu(),
            None if module.bias is None else module.bias.detach().cpu(),
            perm=module.rotation.permutation, signs=module.rotation.signs,
            block=module.rotation.block_size, act_boundaries=module.activation_codebook.boundaries,
            act_centroids=module.activation_codebook.centroids,
            w_centroids=module.weight_codebook.centroids, w_bits=wb, out_features=n)
        _check_close(y, ref, (wb, ab, k, n, m))


def test_module_device_move_rebuilds_constants():
    dev = _dev()
    module = OrbitQuantLinear.from_linear(torch.nn.Linear(256, 64), config=OrbitQuantConfig(),
                                          module_name="t")
    assert module._rotation_permutation.device.type == "cpu"
    module = module.to(dev)
    y = module(torch.randn(3, 256, device=dev, dtype=torch.bfloat16))
    assert module._rotation_permutation.device.type == "cuda"
    assert module.last_effective_runtime_mode == "native_packed_matmul"
    assert y.shape == (3, 64)


def test_torch_compile_fullgraph_bit_equal_to_eager():
    dev = _dev()
    cfg = OrbitQuantConfig(weight_bits=4, activation_bits=4)
    module = OrbitQuantLinear.from_linear(torch.nn.Linear(768, 256), config=cfg, module_name="t").to(dev)

    class Block(torch.nn.Module):
        def __init__(self, inner):
            super().__init__()
            self.inner = inner

        def forward(self, x):
            y = self.inner(x)
            return y, torch.nn.functional.gelu(y.float())

    block = Block(module)
    compiled = torch.compile(block, fullgraph=True)
    for shape in ((4, 768), (2, 5, 768), (4, 768)):
        x = torch.randn(*shape, device=dev, dtype=torch.bfloat16)
        y_c, g_c = compiled(x)
        y_e, g_e = block(x)
        assert torch.equal(y_c, y_e)          # the custom op itself: bit-equal to eager
        assert torch.allclose(g_c, g_e, atol=1e-5)  # the surrounding graph is inductor's


def test_cuda_graph_capture_and_replay():
    dev = _dev()
    cfg = OrbitQuantConfig(weight_bits=4, activation_bits=6)
    blocks = [OrbitQuantLinear.from_linear(torch.nn.Linear(768, 768), config=cfg, module_name=f"b{i}").to(dev)
              for i in range(3)]
    x = torch.randn(4, 768, device=dev, dtype=torch.bfloat16)

    def run(inp):
        h = inp
        for b in blocks:
            h = b(h)
        return h

    eager = run(x)  # also builds the device constants before capture
    torch.cuda.synchronize()
    static_in = x.clone()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        run(static_in)
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(graph):
        static_out = run(static_in)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(static_out, eager)
    x2 = torch.randn(4, 768, device=dev, dtype=torch.bfloat16)
    static_in.copy_(x2)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(static_out, run(x2))
