"""RTN-INT4 group-64 linear (the AdaLN modulation layers): quantiser, oracle and kernel."""
from __future__ import annotations

import pytest
import torch

from orbitquant_b200 import OrbitQuantConfig, unpack_lowbit
from orbitquant_b200.adaln import RTNInt4Linear, quantize_adaln_weight


def _layer(k, n, seed, bias=True):
    g = torch.Generator().manual_seed(seed)
    lin = torch.nn.Linear(k, n, bias=bias)
    with torch.no_grad():
        lin.weight.copy_(torch.randn(n, k, generator=g) * 0.05)
        lin.weight[0, :5] *= 30.0
        if n > 3:
            lin.weight[3] = 0.0       # all-zero groups: scale clamps to 1e-12 / 7
        if bias:
            lin.bias.copy_(torch.randn(n, generator=g))
    return lin


def test_quantiser_codes_and_scales():
    lin = _layer(200, 9, 1)          # 200 = 3 groups + 8 values: padded to 256
    packed, scales = quantize_adaln_weight(lin.weight, group_size=64)
    assert packed.numel() == 9 * 256 // 2 and scales.shape == (9, 4)
    codes = unpack_lowbit(packed, 4, 9 * 256).reshape(9, 256).to(torch.int32) - 8
    w = torch.zeros(9, 256)
    w[:, :200] = lin.weight.detach()
    grouped = w.reshape(9, 4, 64)
    assert torch.equal(scales, grouped.abs().amax(-1).clamp_min(1e-12) / 7.0)
    expect = torch.round(grouped / scales[..., None]).clamp(-8, 7).to(torch.int32).reshape(9, 256)
    assert torch.equal(codes, expect)
    assert torch.all(codes[:, 200:] == 0)                       # padding quantises to zero
    assert codes.abs().max() <= 8 and torch.all(codes[3] == 0)
    # every group's largest magnitude lands on +-7
    assert torch.all(codes.reshape(9, 4, 64).abs().amax(-1)[[0, 1, 2, 4]] == 7)


def test_oracle_matches_reference_cpu_kernel(oracle):
    from oracle import ref_cpu
    if not ref_cpu.available():
        pytest.skip("oracle/_ref is not built")
    for (m, k, n, seed) in ((1, 64, 5, 0), (3, 200, 9, 1), (8, 768, 40, 2), (2, 3072, 33, 3)):
        lin = _layer(k, n, seed)
        packed, scales = quantize_adaln_weight(lin.weight)
        scales = scales.to(torch.bfloat16).float()      # what a module stores
        x = (torch.randn(m, k, generator=torch.Generator().manual_seed(seed + 50)) * 1.3).to(torch.bfloat16)
        mine = oracle.rtn_int4_matmul(x, packed, scales, out_features=n, in_features=k, bias=lin.bias.detach())
        for isa in ("scalar", "auto"):
            ref_cpu.set_isa(isa)
            ref = ref_cpu.matmul_packed_adaln_int4(x, packed, scales, out_features=n, in_features=k,
                                                   bias=lin.bias.detach())
            if isa == "scalar":
                assert torch.equal(mine, ref), (m, k, n, "scalar kernel is the oracle's definition")
            else:      # SIMD kernels reorder the fp32 sum: at most an occasional bf16 ulp
                diff = (mine.float() - ref.float()).abs()
                assert float(diff.max()) <= 2.0 ** -7 * float(ref.float().abs().max())
        ref_cpu.set_isa(None)


def test_module_state_dict_layout():
    cfg = OrbitQuantConfig()
    q = RTNInt4Linear.from_linear(_layer(200, 9, 4), config=cfg, module_name="mod")
    state = q.state_dict()
    assert set(state) == {"packed_weight", "scales", "bias"}
    assert state["packed_weight"].dtype == torch.uint8 and state["scales"].dtype == torch.bfloat16
    empty = RTNInt4Linear.empty_from_linear(torch.nn.Linear(200, 9), config=cfg, module_name="mod")
    empty.load_state_dict(state)
    assert torch.equal(empty.packed_weight, q.packed_weight) and torch.equal(empty.scales, q.scales)
    with pytest.raises(RuntimeError):
        q(torch.zeros(2, 200))          # no CPU path


@pytest.mark.gpu
@pytest.mark.parametrize("m,k,n,bias", [(1, 64, 8, True), (2, 3072, 18432, True), (5, 200, 9, True),
                                        (16, 1536, 520, False), (40, 768, 264, True), (128, 512, 130, True),
                                        (300, 256, 64, True)])
def test_kernel_vs_oracle(oracle, m, k, n, bias):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from orbitquant_b200 import native
    dev = torch.device("cuda", 0)
    native.gemm_clear_device_status()
    lin = _layer(k, n, m + k, bias=bias)
    q = RTNInt4Linear.from_linear(lin, config=OrbitQuantConfig(), module_name="mod").to(dev)
    x = (torch.randn(m, k, generator=torch.Generator().manual_seed(7)) * 1.1).to(torch.bfloat16)
    y = q(x.to(dev))
    torch.cuda.synchronize()
    assert native.gemm_device_status() == 0
    rows = min(m, 6)                      # the numpy oracle is slow: check a few rows of big layers
    ref = oracle.rtn_int4_matmul(x[:rows], q.packed_weight.cpu(), q.scales.cpu().float(), out_features=n,
                                 in_features=k, bias=None if lin.bias is None else lin.bias.detach())
    got = y[:rows].float().cpu()
    rel = float((got - ref.float()).norm() / ref.float().norm().clamp_min(1e-12))
    assert rel <= 1e-3, rel              # same bf16 operands, fp32 sums in a different order
    dense = torch.nn.functional.linear(x.float(), q.dequantize_weight(torch.float32),
                                       None if lin.bias is None else lin.bias.detach().float())
    rel_all = float((y.float().cpu() - dense).norm() / dense.norm())
    assert rel_all <= 4e-3, rel_all      # bf16 output rounding only
    again = q(x.to(dev))
    assert torch.equal(y, again)


@pytest.mark.gpu
def test_compile_fullgraph_with_both_layer_kinds():
    """A module holding an OrbitQuantLinear and an RTNInt4Linear traces without graph breaks:
    both go through the one custom op (the AdaLN layer with bf16_output=True) and the
    compiled result equals eager bit for bit."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from orbitquant_b200 import OrbitQuantConfig, OrbitQuantLinear
    from orbitquant_b200.adaln import RTNInt4Linear

    dev = torch.device("cuda", 0)
    torch.manual_seed(11)
    cfg = OrbitQuantConfig(weight_bits=4, activation_bits=4, rotation_seed=3)

    class Tiny(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.mod = RTNInt4Linear.from_linear(torch.nn.Linear(256, 512), config=cfg, module_name="mod")
            self.proj = OrbitQuantLinear.from_linear(torch.nn.Linear(256, 256), config=cfg, module_name="proj")

        def forward(self, x, c):
            # one elementwise op between the two layers: a chain of them would be fused by the
            # compiler without eager's intermediate bf16 roundings and differ for that reason
            shift = self.mod(c)[..., :256]
            return self.proj(x + shift)

    model = Tiny().to(dev)
    x = torch.randn(24, 256, device=dev).to(torch.bfloat16)
    c = torch.randn(24, 256, device=dev).to(torch.bfloat16)
    eager = model(x, c)
    compiled = torch.compile(model, fullgraph=True)(x, c)
    assert compiled.dtype == torch.bfloat16 and torch.equal(compiled, eager)
