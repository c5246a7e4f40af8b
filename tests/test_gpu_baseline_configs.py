"""Every benchmark configuration at its full K and N, through the DEFAULT module path, against
the reference's own compiled CPU kernels (``oracle/_ref``, built from the reference sources).

What each case pins (reference files are cited by their path inside the reference project):

* config 0 -- one OrbitLinear W4A4, M=1024, 3072 -> 3072, RPBH block 256, seed 0, columns 0..7
  scaled x20; the weight is a real fp32 matrix ~N(0, 0.02) quantised by ``from_weight``.
  Compared whole (all 1024 rows).
* config 1 -- DiT block projections W4A4, M=4608, the benchmark's own synthetic payloads and
  activations; 512 sampled token rows per projection (the sample always holds the first and
  the last row tile).
* config 2 -- mixed-bit layers at 3072 -> 3072, M=4096: W2A4 (Q/K projections) and W3A3.
* config 3 -- video-DiT W4A4, M=32760, hidden 5120 / FFN 13824; 512 sampled rows.
* config 4 -- ViT-base decode W4A6, M in {1, 4, 16}, all four projection shapes.

Reference arithmetic.  ``quantize_activations_cpu`` runs with ``ORBITQUANT_CPU_ISA=avx512``
(``quantize_activations_cpu.cpp:633-664``; the CUDA prologue follows that kernel's
operation order and is bit-identical to it).  ``matmul_packed_weight`` runs with the ISA
whose weight arithmetic matches the module's ``weight_mode``
(``packed_matmul_x86_avx512.cpp:767-823``): ``centroid`` = fp32 centroids, row norm applied
to the sum -> ``avx2`` for W4 (on an AVX512-BF16 host ``avx512`` would take the bf16 dot
kernel), ``avx512`` for the other widths; ``bf16_scaled`` = bf16(centroid * row_norm)
-> ``avx512`` on a host with AVX512-BF16.

Tolerances: as in test_gpu_parity.py (rel-L2 <= 1e-3; max-abs <= 2e-2 of the output RMS plus
one bf16 ulp, because both sides are rounded to bf16 here).  Where ``oracle/_ref`` is not
present the C restatement of the same kernels (``oracle/orbit_oracle.c``, bit-equal to them
in the CPU suite) checks a smaller row sample.
"""
from __future__ import annotations

import json
import os

import pytest
import torch

import bench
from oracle import ref_cpu
from orbitquant_b200 import OrbitQuantConfig, OrbitQuantLinear, native
from test_gpu_parity import _check_close, _dev, parity_errors

pytestmark = pytest.mark.gpu

SAMPLE_ROWS = 512 if ref_cpu.available() else 48


def _report(name: str, y_gpu, ref) -> None:
    """Optional record of the measured errors (path in ORBIT_B200_PARITY_REPORT)."""
    path = os.environ.get("ORBIT_B200_PARITY_REPORT")
    if not path:
        return
    err, max_abs, excess = parity_errors(y_gpu, ref)
    with open(path, "a") as fh:
        fh.write(json.dumps({"case": name, "rows": int(y_gpu.shape[0]), "rel_l2": err,
                             "max_abs_over_rms_bf16": max_abs,
                             "max_abs_over_rms_beyond_rounding": excess,
                             "reference": "oracle/_ref" if ref_cpu.available() else "oracle port"}) + "\n")


def _has_avx512_bf16() -> bool:
    return bool(ref_cpu.host_isa_report()["avx512_bf16"])


def reference_forward(x_cpu: torch.Tensor, module: OrbitQuantLinear, oracle, arithmetic: str):
    """The reference CPU forward of `module` on `x_cpu`; see the module docstring."""
    kw = dict(w_bits=module.weight_bits, out_features=module.out_features)
    packed = module.packed_weight_indices.detach().cpu()
    norms = module.row_norms.detach().cpu()
    bias = None if module.bias is None else module.bias.detach().cpu().float()
    rot, acb, wcb = module.rotation, module.activation_codebook, module.weight_codebook
    if not ref_cpu.available():
        mode = oracle.MM_BF16_LUT if arithmetic == "bf16_scaled" else oracle.MM_FP32_CENTROIDS
        return oracle.linear_forward(
            x_cpu, packed, norms, bias, perm=rot.permutation, signs=rot.signs, block=rot.block_size,
            act_boundaries=acb.boundaries, act_centroids=acb.centroids, w_centroids=wcb.centroids,
            eps=module.activation_eps, mode=mode, **kw)
    previous = os.environ.get("ORBITQUANT_CPU_ISA")
    try:
        ref_cpu.set_isa("avx512")
        x_q = ref_cpu.quantize_activations_cpu(
            x_cpu, rot.permutation, rot.signs, acb.centroids, acb.boundaries,
            eps=module.activation_eps, inv_sqrt_block=1.0 / (rot.block_size ** 0.5),
            block_size=rot.block_size)
        if arithmetic == "bf16_scaled":
            ref_cpu.set_isa("avx512")
        else:
            ref_cpu.set_isa("avx2" if module.weight_bits == 4 else "avx512")
        return ref_cpu.matmul_packed_weight(
            x_q, packed, norms, wcb.centroids, bits=module.weight_bits,
            out_features=module.out_features, in_features=module.in_features, bias=bias)
    finally:
        ref_cpu.set_isa(previous)


def _sample_rows(rows: int, count: int, seed: int) -> torch.Tensor:
    """Sorted row sample that always holds the first and last 128 rows' ends."""
    if rows <= count:
        return torch.arange(rows)
    g = torch.Generator().manual_seed(seed)
    fixed = torch.tensor([0, 1, 127, 128, 255, 256, rows - 257, rows - 256, rows - 2, rows - 1])
    rest = torch.randperm(rows, generator=g)[: count - fixed.numel()]
    return torch.unique(torch.cat([fixed, rest]))


def _synthetic_module(k, n, w_bits, a_bits, std, seed, payload_seed, block_size="paper"):
    cfg = OrbitQuantConfig(weight_bits=w_bits, activation_bits=a_bits, rotation_seed=seed,
                           block_size=block_size)
    packed, norms, bias = bench.synth_weight_payload(k, n, w_bits, std, payload_seed)
    return OrbitQuantLinear(in_features=k, out_features=n, config=cfg, module_name="parity",
                            source_weight_layout="out_in", bias=bias, packed_weight_indices=packed,
                            row_norms=norms, debug_weight=None)


def _run_case(name, module, x_dev, oracle, arithmetic="centroid", sample_seed=0):
    dev = x_dev.device
    module = module.to(dev)
    module.weight_mode = arithmetic
    native.gemm_clear_device_status()
    y = module(x_dev)
    torch.cuda.synchronize()
    assert native.gemm_device_status() == 0
    pick = _sample_rows(x_dev.shape[0], SAMPLE_ROWS, sample_seed)
    x_cpu = x_dev[pick.to(dev)].cpu()
    ref = reference_forward(x_cpu, module, oracle, arithmetic)
    got = y[pick.to(dev)]
    _report(name, got, ref)
    _check_close(got, ref, name)


def test_config0_single_layer_whole(oracle):
    dev = _dev()
    torch.manual_seed(0)
    weight = torch.randn(3072, 3072) * 0.02
    x = torch.randn(1024, 3072)
    x[:, :8] *= 20.0
    x = x.to(torch.bfloat16)
    cfg = OrbitQuantConfig(weight_bits=4, activation_bits=4, block_size=256, rotation_seed=0)
    module = OrbitQuantLinear.from_weight(weight, bias=None, in_features=3072, out_features=3072,
                                          source_weight_layout="out_in", config=cfg,
                                          module_name="config0").to(dev)
    y = module(x.to(dev))
    torch.cuda.synchronize()
    rows = 1024 if ref_cpu.available() else SAMPLE_ROWS
    ref = reference_forward(x[:rows], module, oracle, "centroid")
    _report("config0 M=1024 3072->3072 W4A4 block256", y[:rows], ref)
    _check_close(y[:rows], ref, "config 0")


@pytest.mark.parametrize("layer", range(4))
def test_config1_dit_block_projections(oracle, layer):
    dev = _dev()
    rows, specs, std, seed, w_bits, a_bits = bench.WORKLOADS["dit_block"]
    name, k, n, _gather = specs[layer]
    module = _synthetic_module(k, n, w_bits, a_bits, std, seed, seed * 100 + layer)
    x = bench.synth_activations(rows, k, seed * 1000 + layer).to(dev)
    _run_case(f"config1 {name} M={rows} {k}->{n} W4A4", module, x, oracle, sample_seed=layer)


@pytest.mark.parametrize("w_bits,a_bits,what", [(2, 4, "q/k projection"), (3, 3, "interior projection")])
def test_config2_mixed_bit_layers(oracle, w_bits, a_bits, what):
    dev = _dev()
    module = _synthetic_module(3072, 3072, w_bits, a_bits, 0.02, 2, 200 + w_bits)
    x = bench.synth_activations(4096, 3072, 2000 + w_bits).to(dev)
    _run_case(f"config2 {what} M=4096 3072->3072 W{w_bits}A{a_bits}", module, x, oracle,
              sample_seed=w_bits)


@pytest.mark.parametrize("layer", range(4))
def test_config3_video_dit_projections(oracle, layer):
    dev = _dev()
    rows, specs, std, seed, w_bits, a_bits = bench.WORKLOADS["video_dit"]
    name, k, n, _gather = specs[layer]
    module = _synthetic_module(k, n, w_bits, a_bits, std, seed, seed * 100 + layer)
    x = bench.synth_activations(rows, k, seed * 1000 + layer, device=dev)
    _run_case(f"config3 {name} M={rows} {k}->{n} W4A4", module, x, oracle, sample_seed=layer)
    del x
    torch.cuda.empty_cache()


@pytest.mark.parametrize("rows", [1, 4, 16])
def test_config4_vit_decode(oracle, rows):
    dev = _dev()
    _rows, specs, std, seed, w_bits, a_bits = bench.WORKLOADS["vit_decode"]
    for layer, (name, k, n, _gather) in enumerate(specs):
        module = _synthetic_module(k, n, w_bits, a_bits, std, seed, seed * 100 + layer)
        x = bench.synth_activations(rows, k, seed * 1000 + layer).to(dev)
        _run_case(f"config4 {name} M={rows} {k}->{n} W4A6", module, x, oracle)


def test_config1_bf16_scaled_arithmetic(oracle):
    """The reference's default arithmetic for W4 / bf16 on an AVX512-BF16 host (and of its CUDA
    kernels): operand bf16(centroid * row_norm).  Only compared where the host's reference
    kernels take that path."""
    if ref_cpu.available() and not _has_avx512_bf16():
        pytest.skip("the host's reference kernels have no bf16 dot path")
    dev = _dev()
    rows, specs, std, seed, w_bits, a_bits = bench.WORKLOADS["dit_block"]
    for layer in (1, 3):
        name, k, n, _gather = specs[layer]
        module = _synthetic_module(k, n, w_bits, a_bits, std, seed, seed * 100 + layer)
        x = bench.synth_activations(rows, k, seed * 1000 + layer).to(dev)
        _run_case(f"config1 {name} M={rows} {k}->{n} W4A4 bf16_scaled", module, x, oracle,
                  arithmetic="bf16_scaled", sample_seed=layer)
