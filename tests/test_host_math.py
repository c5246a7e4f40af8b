"""Host-side pieces (codebooks, RPBH constants, bit packing, weight quantisation, config,
module surface) against the golden vectors generated from the reference, plus the C-ABI
export check.  No GPU needed."""
from __future__ import annotations

import ctypes
import hashlib
import re

import numpy as np
import pytest
import torch

from conftest import REPO, bf16_from_bits, bits_of, codebook_from_golden
from orbitquant_b200 import (OrbitQuantConfig, OrbitQuantLinear, RPBHRotation, fwht, get_codebook,
                             native, pack_lowbit, unpack_lowbit)
from orbitquant_b200.layers import iter_aligned_row_tiles, quantize_weight
from orbitquant_b200.rotations import paper_block_size


# ---- codebooks ---------------------------------------------------------------------------

@pytest.mark.parametrize("dim", [32, 256, 768, 3072, 5120, 12288, 13824])
@pytest.mark.parametrize("bits", [2, 3, 4, 6])
def test_codebook_bit_equal_to_reference(golden_codebooks, dim, bits):
    cb = get_codebook(dim, bits, 2)
    assert np.array_equal(cb.centroids.numpy(), golden_codebooks[f"v2_dim{dim}_bits{bits}_centroids"])
    assert np.array_equal(cb.boundaries.numpy(), golden_codebooks[f"v2_dim{dim}_bits{bits}_boundaries"])


def test_codebook_reference_known_answer():
    # The reference's own known-answer vectors (tests/test_codebooks.py:33-62, :82-102):
    # dim 32, 3 bits, algorithm versions 2 and 1, tolerance 1e-6.
    cb = get_codebook(32, 3, 2)
    expected = torch.tensor([-0.36626825, -0.23246057, -0.13175610, -0.04285152,
                             0.04285152, 0.13175610, 0.23246057, 0.36626825])
    bounds = torch.tensor([-0.29936442, -0.18210834, -0.08730381, 0.0,
                           0.08730381, 0.18210834, 0.29936442])
    torch.testing.assert_close(cb.centroids, expected, atol=1e-6, rtol=0)
    torch.testing.assert_close(cb.boundaries, bounds, atol=1e-6, rtol=0)
    legacy = get_codebook(32, 3, 1)
    expected_v1 = torch.tensor([-0.36600566, -0.23213057, -0.13146324, -0.04273151,
                                0.04273151, 0.13146324, 0.23213057, 0.36600566])
    assert legacy.algorithm_version == 1
    torch.testing.assert_close(legacy.centroids, expected_v1, atol=1e-6, rtol=0)


def test_codebook_symmetry_and_order():
    for bits in (2, 3, 4, 6):
        cb = get_codebook(768, bits)
        assert cb.centroids.shape == (2 ** bits,) and cb.boundaries.shape == (2 ** bits - 1,)
        assert torch.equal(cb.centroids, -torch.flip(cb.centroids, dims=[0]))
        assert torch.all(cb.centroids[1:] > cb.centroids[:-1])
        assert cb.boundaries[2 ** (bits - 1) - 1] == 0.0


def test_legacy_grid_codebook(golden_codebooks):
    cb = get_codebook(32, 3, 1)
    assert np.allclose(cb.centroids.numpy(), golden_codebooks["v1_dim32_bits3_centroids"], atol=1e-7)
    with pytest.raises(ValueError):
        get_codebook(32, 3, 3)
    with pytest.raises(ValueError):
        get_codebook(32, 9)


def test_bucketize_ties_go_low():
    cb = get_codebook(256, 2)
    v = torch.tensor([cb.boundaries[1].item(), 1.0, -1.0])
    assert cb.quantize_indices(v).tolist() == [1, 3, 0]


# ---- rotations ---------------------------------------------------------------------------

def test_rotation_draws_match_reference(golden_rotations):
    for dim, seed, block in ((64, 0, 16), (768, 4, "paper"), (3072, 0, 256), (3072, 1, "paper")):
        rot = RPBHRotation(dim, seed, block)
        key = f"dim{dim}_seed{seed}"
        assert np.array_equal(rot.permutation.numpy().astype(np.int32), golden_rotations[key + "_perm"])
        assert np.array_equal(rot.signs.numpy(), golden_rotations[key + "_signs"])
        assert rot.block_size == int(golden_rotations[key + "_block"])
    for dim, seed in ((5120, 3), (12288, 1), (13824, 3)):
        rot = RPBHRotation(dim, seed, "paper")
        digest = hashlib.sha256(rot.permutation.numpy().astype(np.int32).tobytes()
                                + rot.signs.numpy().tobytes()).hexdigest()
        assert digest == bytes(golden_rotations[f"dim{dim}_seed{seed}_sha256"]).decode("ascii")


def test_paper_block_rule(golden_rotations):
    for dim, block in zip(golden_rotations["paper_dims"], golden_rotations["paper_blocks"]):
        assert paper_block_size(int(dim)) == int(block)
    # the table the reference pins (tests/test_paper_methodology.py:101-117)
    table = {1536: 512, 3072: 1024, 3840: 256, 8960: 256, 9216: 1024, 10240: 2048,
             12288: 4096, 15360: 1024}
    for dim, block in table.items():
        assert paper_block_size(dim) == block


def test_rotation_is_orthogonal_and_invertible():
    rot = RPBHRotation(96, 3, 32)
    x = torch.randn(5, 96, dtype=torch.float64)
    y = rot.apply_to_activations(x)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-12)
    assert torch.allclose(rot.apply_inverse_to_activations(y), x, atol=1e-12)
    w = torch.randn(7, 96, dtype=torch.float64)
    assert torch.allclose(x @ w.T, y @ rot.apply_to_weight(w).T, atol=1e-10)


def test_rotation_argument_errors():
    with pytest.raises(ValueError):
        RPBHRotation(0)
    with pytest.raises(ValueError):
        RPBHRotation(96, 0, 64)
    with pytest.raises(ValueError):
        RPBHRotation(96, 0, 24)
    with pytest.raises(TypeError):
        RPBHRotation(96, 0, "other")
    with pytest.raises(ValueError):
        RPBHRotation(96, 0, 32).apply_to_activations(torch.zeros(2, 95))


def test_fwht_matches_oracle_bitwise(oracle):
    x = torch.randn(3, 512)
    assert torch.equal(fwht(x), oracle.fwht(x))
    with pytest.raises(ValueError):
        fwht(torch.zeros(3, 12))


# ---- bit packing -------------------------------------------------------------------------

@pytest.mark.parametrize("bits", [1, 2, 3, 4, 5, 6, 7, 8])
def test_bitpack_matches_reference_vectors(golden_bitpack, oracle, bits):
    for length in (0, 1, 7, 64, 1003):
        values = torch.from_numpy(golden_bitpack[f"bits{bits}_len{length}_values"].copy())
        packed = torch.from_numpy(golden_bitpack[f"bits{bits}_len{length}_packed"].copy())
        assert torch.equal(pack_lowbit(values, bits), packed)
        assert torch.equal(unpack_lowbit(packed, bits, length), values)
        assert torch.equal(oracle.pack(values, bits), packed)
        assert torch.equal(oracle.unpack(packed, bits, length), values)


def test_bitpack_large_three_bit_roundtrip():
    # same size as the reference's ragged case (tests/test_bitpack.py)
    values = torch.randint(0, 8, (100_003,), dtype=torch.uint8)
    packed = pack_lowbit(values, 3)
    assert packed.numel() == (100_003 * 3 + 7) // 8
    assert torch.equal(unpack_lowbit(packed, 3, 100_003), values)


def test_bitpack_errors():
    with pytest.raises(ValueError):
        pack_lowbit(torch.tensor([4]), 2)
    with pytest.raises(ValueError):
        pack_lowbit(torch.tensor([1]), 0)
    with pytest.raises(ValueError):
        unpack_lowbit(torch.zeros(1, dtype=torch.uint8), 9, 1)
    with pytest.raises(ValueError):
        unpack_lowbit(torch.zeros(1, dtype=torch.uint8), 4, -1)


def test_row_tiles_end_on_byte_boundaries():
    tiles = list(iter_aligned_row_tiles(10, 5, 3, 3))  # 15 bits per row -> align to 8 rows
    assert tiles == [(0, 8), (8, 10)]
    assert list(iter_aligned_row_tiles(5, 768, 4, 2)) == [(0, 2), (2, 4), (4, 5)]


# ---- weight quantisation + module surface ------------------------------------------------

def _case(golden_layers, name):
    m, k, n, wb, ab, block, seed = (int(v) for v in golden_layers[f"{name}_meta"])
    return m, k, n, wb, ab, block, seed


def test_weight_quantisation_bit_equal_to_reference(golden_layers, golden_codebooks):
    for name in golden_layers["case_names"]:
        name = str(name)
        m, k, n, wb, ab, block, seed = _case(golden_layers, name)
        weight = torch.from_numpy(golden_layers[f"{name}_weight"].copy())
        rot = RPBHRotation(k, seed, block)
        cb = codebook_from_golden(golden_codebooks, k, wb) if wb == 8 else get_codebook(k, wb)
        packed, norms = quantize_weight(weight, rotation=rot, codebook=cb, bits=wb, eps=1e-10,
                                        row_tile_size=7)
        assert np.array_equal(packed.numpy(), golden_layers[f"{name}_packed"]), name
        assert np.array_equal(bits_of(norms).numpy().astype(np.uint16),
                              golden_layers[f"{name}_row_norms"]), name


def test_module_surface_and_state_dict():
    cfg = OrbitQuantConfig(weight_bits=4, activation_bits=6, rotation_seed=3)
    lin = torch.nn.Linear(256, 40)
    q = OrbitQuantLinear.from_linear(lin, config=cfg, module_name="proj")
    assert sorted(q.state_dict().keys()) == ["bias", "packed_weight_indices", "row_norms"]
    assert q.packed_weight_indices.dtype == torch.uint8
    assert q.packed_weight_indices.shape == (40 * 256 // 2,)
    assert q.row_norms.dtype == torch.bfloat16 and q.row_norms.shape == (40,)
    assert not q.packed_weight_indices.requires_grad
    assert q._rotation_permutation.dtype == torch.int32 and q._rotation_signs.dtype == torch.int8
    assert q.weight_bits == 4 and q.activation_bits == 6 and q.rotation.block_size == 256
    empty = OrbitQuantLinear.empty_from_linear(lin, config=cfg, module_name="proj")
    empty.load_state_dict(q.state_dict())
    assert torch.equal(empty.packed_weight_indices, q.packed_weight_indices)
    assert empty._derived_constants_valid is False
    nobias = OrbitQuantLinear.from_linear(torch.nn.Linear(256, 8, bias=False), config=cfg,
                                          module_name="x")
    assert sorted(nobias.state_dict().keys()) == ["packed_weight_indices", "row_norms"]


def test_module_rejects_cpu_input_and_bad_shapes():
    cfg = OrbitQuantConfig()
    q = OrbitQuantLinear.from_linear(torch.nn.Linear(256, 8), config=cfg, module_name="x")
    with pytest.raises(RuntimeError, match="CUDA"):
        q(torch.randn(2, 256))
    with pytest.raises(ValueError):
        OrbitQuantLinear.from_weight(torch.zeros(3, 4), bias=None, in_features=8, out_features=3,
                                     source_weight_layout="out_in", config=cfg, module_name="x")
    with pytest.raises(TypeError):
        OrbitQuantLinear.from_linear(torch.nn.Conv1d(4, 4, 1), config=cfg, module_name="x")


def test_compile_handle_registry_goes_stale():
    from orbitquant_b200 import layers
    q = OrbitQuantLinear.from_linear(torch.nn.Linear(256, 8), config=OrbitQuantConfig(),
                                     module_name="x")
    handle = q._compile_handle
    assert layers._registry_lookup(handle) is q
    del q
    import gc
    gc.collect()
    with pytest.raises(RuntimeError, match="stale"):
        layers._registry_lookup(handle)


def test_fake_op_shapes():
    x = torch.empty(2, 3, 256, device="meta", dtype=torch.float16)
    y = torch.ops.orbitquant.packed_linear_forward(x, 0, 40, False)
    assert y.shape == (2, 3, 40) and y.dtype == torch.float16
    y = torch.ops.orbitquant.packed_linear_forward(x, 0, 40, True)
    assert y.dtype == torch.bfloat16


def test_config_validation_and_roundtrip(tmp_path):
    cfg = OrbitQuantConfig(weight_bits=2, activation_bits=4, block_size=256)
    again = OrbitQuantConfig.from_dict(cfg.to_dict())
    assert again == cfg
    cfg.to_json_file(tmp_path / "c.json")
    assert '"weight_bits": 2' in (tmp_path / "c.json").read_text()
    assert OrbitQuantConfig.from_dict({"weight_bits": 4}).codebook_version == 1
    for bad in ({"weight_bits": 5}, {"activation_bits": 1}, {"rotation": "x"},
                {"row_norm_dtype": "float32"}, {"packed_matmul_block_m": 0},
                {"runtime_mode": "nope"}, {"lowbit_protected_bits": 9}):
        with pytest.raises(ValueError):
            OrbitQuantConfig(**bad)


# ---- the C ABI ----------------------------------------------------------------------------

def test_library_exports_every_declared_symbol():
    header = (REPO / "include" / "orbit_b200.h").read_text()
    declared = set(re.findall(r"\b(oq_[a-z0-9_]+)\s*\(", header))
    declared.discard("oq_status")
    assert declared, "no declarations found"
    lib = ctypes.CDLL(str(native.library_path()))
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/orbit_b200.h but not exported"
    assert declared == set(native.exported_symbols())
    assert native.load().oq_abi_version() == 1


def test_header_is_plain_c_and_links(tmp_path):
    """The boundary is a C ABI: the header must compile as C99 and a C program must link
    against the library without any C++ or torch symbol."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no gcc")
    source = tmp_path / "use.c"
    source.write_text('#include "orbit_b200.h"\n'
                      'int main(void) {\n'
                      '  if (oq_abi_version() != OQ_ABI_VERSION) return 1;\n'
                      '  if (oq_unpack_lowbit(0, 9, 4, 0, 0) != OQ_ERR_INVALID) return 2;\n'
                      '  return oq_last_error()[0] == 0 ? 3 : 0;\n'
                      '}\n')
    lib = native.library_path()
    exe = tmp_path / "use"
    subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", f"-I{REPO / 'include'}", str(source), str(lib),
                    f"-Wl,-rpath,{lib.parent}", "-o", str(exe)], check=True)
    assert subprocess.run([str(exe)]).returncode == 0


def test_argument_errors_surface_without_a_gpu():
    lib = native.load()
    assert lib.oq_unpack_lowbit(None, 9, 4, None, None) == -1
    assert b"bits" in lib.oq_last_error()
    assert lib.oq_matmul_packed_weight(None, None, 2, 4, 64, 8, None, 10, 4, None, None, None, 0,
                                       0, 0, None, 0, None) == -1
    assert b"too short" in lib.oq_last_error()
    assert lib.oq_linear_workspace_bytes(16, 768, 2304, 4, 2, 0, 0) == 16 * 768 * 2
    assert lib.oq_gemm_tcgen05_supported(4608, 3072, 9216, 4, 2, 0) == 1
    assert lib.oq_gemm_tcgen05_supported(4608, 3070, 9216, 4, 2, 0) == 0
    assert lib.oq_gemm_tcgen05_supported(4608, 3072, 9216, 3, 2, 0) == 1
    assert lib.oq_gemm_tcgen05_supported(4608, 3072, 9216, 5, 2, 0) == 0
    with pytest.raises(RuntimeError, match="CUDA"):
        native.matmul_packed_weight(torch.zeros(2, 64), torch.zeros(256, dtype=torch.uint8),
                                    torch.zeros(8), torch.zeros(16), bits=4, out_features=8,
                                    in_features=64)


def test_kernel_plan_by_shape_without_a_gpu():
    """`oq_linear_kernel_name` answers from the shape alone (no launch, no device): the dispatch
    rules of the forward -- one launch for a few tokens of a small layer, the CUDA-core GEMV for one
    to four tokens of a large W4 layer, the few-token tensor-core kernel up to 128 rows, the CTA-pair kernel where a 512-row pair tile fills the machine, the
    single-CTA kernel for 6- and 8-bit weights and for small grids, the general kernel otherwise."""
    from orbitquant_b200 import native

    plan = native.forward_kernel_name
    assert plan(1, 768, 2304, 4, 6, 256) == "decode_fused_kernel"
    assert plan(16, 768, 2304, 4, 6, 256) == "rotate_quantize + small_rows_w4_kernel"
    assert plan(1, 3072, 12288, 4, 4, 1024) == "rotate_quantize + gemv_w4_kernel"
    assert plan(4, 12288, 3072, 4, 4, 4096) == "rotate_quantize + gemv_w4_kernel"
    assert plan(5, 12288, 3072, 4, 4, 4096) == "rotate_quantize + skinny_tcgen05_kernel"
    assert plan(16, 3072, 9216, 4, 4, 1024) == "rotate_quantize + skinny_tcgen05_kernel"
    assert plan(128, 3072, 3072, 4, 4, 1024) == "rotate_quantize + skinny_tcgen05_kernel"
    assert plan(300, 768, 512, 4, 4, 256) == "rotate_quantize + gemm_w4_tcgen05_kernel"
    assert plan(4608, 3072, 9216, 4, 4, 1024) == "rotate_quantize + gemm_pair_tcgen05_kernel"
    assert plan(32760, 5120, 15360, 4, 4, 1024) == "rotate_quantize + gemm_pair_tcgen05_kernel"
    assert plan(4096, 3072, 3072, 3, 3, 1024) == "rotate_quantize + gemm_pair_tcgen05_kernel"
    assert plan(4608, 3072, 3072, 6, 6, 1024) == "rotate_quantize + gemm_w4_tcgen05_kernel"
    assert plan(40, 200, 96, 3, 3, 8) == "rotate_quantize + tiled_matmul_kernel"
    assert plan(0, 768, 768, 4, 4, 256) == "none"
