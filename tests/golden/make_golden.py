"""Generate the committed golden fixtures from the REFERENCE implementation.

Run where the reference checkout is present (it is imported read-only from
``$ORBITQUANT_REFERENCE_ROOT/src``) and where
``oracle/_ref`` has been built (``python oracle/build_ref.py``):

    python tests/golden/make_golden.py

Writes, next to this file:

* ``codebooks.npz``      -- fp32 centroids from the reference Lloyd-Max generator for every
                           ``(dim, bits)`` the benchmark configurations use, plus the
                           reference's own golden case (dim 32, 3 bits).
* ``rotations.npz``      -- RPBH permutation/sign draws (full arrays for small dims, SHA-256
                           for the large ones) and the "paper" block-size table.
* ``layer_cases.npz``    -- small OrbitQuantLinear cases: inputs, the reference's packed
                           weights / row norms, and the reference's outputs along every CPU
                           path (pure-torch definition, compiled kernels with the ISA
                           pinned to scalar and to avx512).
* ``bitpack.npz``        -- pack/unpack vectors for every bit width, ragged lengths.

Nothing here runs on the GPU box; the fixtures travel, this script does not need to.
"""
from __future__ import annotations

import hashlib
import os
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
REF_ROOT = Path(os.environ.get("ORBITQUANT_REFERENCE_ROOT") or REPO.parent / "reference")

# The reference derives 8-bit tables in minutes; let it keep its own disk cache in a
# scratch folder so that re-running this script is quick.
os.environ.setdefault("ORBITQUANT_CODEBOOK_CACHE_DIR",
                      str(Path(tempfile.gettempdir()) / "orbitquant_codebook_cache"))
sys.path.insert(0, str(REF_ROOT / "src"))
sys.path.insert(0, str(REPO))

from orbitquant.codebooks import get_codebook  # noqa: E402  (reference)
from orbitquant.config import OrbitQuantConfig  # noqa: E402
from orbitquant.functional import quantize_activations  # noqa: E402
from orbitquant.layers import OrbitQuantLinear  # noqa: E402
from orbitquant.packing import pack_lowbit, unpack_lowbit  # noqa: E402
from orbitquant.rotations import RPBHRotation  # noqa: E402

from oracle import ref_cpu  # noqa: E402  (the reference's compiled CPU kernels)

CODEBOOK_DIMS = (32, 256, 768, 3072, 5120, 12288, 13824)
BITS = (2, 3, 4, 6, 8)


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().astype(np.uint16)


def make_codebooks() -> None:
    if (HERE / "codebooks.npz").exists() and "--force" not in sys.argv:
        return
    out = {}
    for dim in CODEBOOK_DIMS:
        for bits in BITS:
            if bits == 8 and dim > 768:
                # minutes per table, and the reference's own iteration does not converge
                # for dim 12288 at 8 bits; 8-bit tables are pinned on the small dims only
                continue
            cb = get_codebook(dim, bits, 2)
            out[f"v2_dim{dim}_bits{bits}_centroids"] = cb.centroids.numpy()
            out[f"v2_dim{dim}_bits{bits}_boundaries"] = cb.boundaries.numpy()
    for dim, bits in ((32, 3), (768, 4), (3072, 2)):
        cb = get_codebook(dim, bits, 1)
        out[f"v1_dim{dim}_bits{bits}_centroids"] = cb.centroids.numpy()
        out[f"v1_dim{dim}_bits{bits}_boundaries"] = cb.boundaries.numpy()
    np.savez_compressed(HERE / "codebooks.npz", **out)


def make_rotations() -> None:
    out = {}
    for dim, seed, block in ((64, 0, 16), (768, 4, "paper"), (3072, 0, 256), (3072, 1, "paper")):
        rot = RPBHRotation(dim=dim, seed=seed, block_size=block)
        key = f"dim{dim}_seed{seed}"
        out[key + "_perm"] = rot.permutation.numpy().astype(np.int32)
        out[key + "_signs"] = rot.signs.numpy()
        out[key + "_block"] = np.int64(rot.block_size)
    for dim, seed in ((5120, 3), (12288, 1), (13824, 3)):
        rot = RPBHRotation(dim=dim, seed=seed, block_size="paper")
        key = f"dim{dim}_seed{seed}"
        digest = hashlib.sha256(rot.permutation.numpy().astype(np.int32).tobytes()
                                + rot.signs.numpy().tobytes()).hexdigest()
        out[key + "_sha256"] = np.frombuffer(digest.encode("ascii"), dtype=np.uint8)
        out[key + "_block"] = np.int64(rot.block_size)
    table_dims = (1536, 3072, 3840, 8960, 9216, 10240, 12288, 15360, 768, 5120, 13824)
    out["paper_dims"] = np.array(table_dims, dtype=np.int64)
    out["paper_blocks"] = np.array(
        [RPBHRotation(dim=d, seed=0, block_size="paper").block_size for d in table_dims],
        dtype=np.int64)
    np.savez_compressed(HERE / "rotations.npz", **out)


def make_bitpack() -> None:
    out = {}
    gen = torch.Generator().manual_seed(1234)
    for bits in (1, 2, 3, 4, 5, 6, 7, 8):
        for length in (0, 1, 7, 64, 1003):
            values = torch.randint(0, 1 << bits, (length,), generator=gen, dtype=torch.uint8)
            packed = pack_lowbit(values, bits)
            assert torch.equal(unpack_lowbit(packed, bits, length), values)
            out[f"bits{bits}_len{length}_values"] = values.numpy()
            out[f"bits{bits}_len{length}_packed"] = packed.numpy()
    np.savez_compressed(HERE / "bitpack.npz", **out)


LAYER_CASES = (
    # name, M, K, N, w_bits, a_bits, block, seed, bias
    ("w4a4_k256", 9, 256, 48, 4, 4, "paper", 0, True),
    ("w4a4_k768_b256", 6, 768, 40, 4, 4, 256, 0, False),
    ("w3a3_k768", 5, 768, 33, 3, 3, "paper", 2, True),
    ("w2a4_k768", 5, 768, 32, 2, 4, "paper", 2, True),
    ("w4a6_k768", 4, 768, 24, 4, 6, "paper", 4, True),
    ("w6a6_k512", 3, 512, 20, 6, 6, 128, 5, False),
    ("w8a8_k256", 3, 256, 17, 8, 8, "paper", 6, True),
    ("w2a3_k1536", 3, 1536, 16, 2, 3, "paper", 7, True),
)


def make_layer_cases() -> None:
    out = {}
    names = []
    for name, m, k, n, wb, ab, block, seed, with_bias in LAYER_CASES:
        torch.manual_seed(seed)
        weight = torch.randn(n, k) * 0.02
        weight[min(3, n - 1)] = 0.0  # a zero row dequantises to exact zeros
        bias = torch.randn(n) * 0.1 if with_bias else None
        x = torch.randn(m, k)
        x[:, :4] *= 20.0  # outlier channels
        x[m - 1] = 0.0  # a zero token must produce exactly the bias
        x = x.to(torch.bfloat16)
        config = OrbitQuantConfig(weight_bits=wb, activation_bits=ab, block_size=block,
                                  rotation_seed=seed, runtime_mode="dequant_bf16",
                                  activation_kernel_backend="cpu")
        layer = OrbitQuantLinear.from_weight(
            weight, bias=bias, in_features=k, out_features=n,
            source_weight_layout="out_in", config=config, module_name=name)
        rot = layer.rotation
        acb = layer.activation_codebook
        wcb = layer.weight_codebook
        xq_def = quantize_activations(x, rotation=rot, codebook=acb, eps=config.activation_eps)
        y_def = layer(x)
        out[f"{name}_meta"] = np.array([m, k, n, wb, ab, rot.block_size, seed], dtype=np.int64)
        out[f"{name}_x"] = bf16_bits(x)
        out[f"{name}_weight"] = weight.numpy()
        out[f"{name}_packed"] = layer.packed_weight_indices.detach().numpy()
        out[f"{name}_row_norms"] = bf16_bits(layer.row_norms.detach())
        if bias is not None:
            out[f"{name}_bias"] = bias.numpy()
        out[f"{name}_xq_definition"] = bf16_bits(xq_def)
        out[f"{name}_y_dequant_bf16"] = bf16_bits(y_def.detach())
        for isa in ("scalar", "avx512"):
            ref_cpu.set_isa(isa)
            xq = ref_cpu.quantize_activations_cpu(
                x, rot.permutation, rot.signs, acb.centroids, acb.boundaries,
                eps=config.activation_eps, inv_sqrt_block=rot.normalization,
                block_size=rot.block_size)
            y = ref_cpu.matmul_packed_weight(
                xq, layer.packed_weight_indices.detach(), layer.row_norms.detach(),
                wcb.centroids, bits=wb, out_features=n, in_features=k, bias=bias)
            out[f"{name}_xq_native_{isa}"] = bf16_bits(xq)
            out[f"{name}_y_native_{isa}"] = bf16_bits(y)
        ref_cpu.set_isa(None)
        names.append(name)
    out["case_names"] = np.array(names)
    out["host_isa"] = np.array(str(ref_cpu.host_isa_report()))
    np.savez_compressed(HERE / "layer_cases.npz", **out)


if __name__ == "__main__":
    make_codebooks()
    make_rotations()
    make_bitpack()
    make_layer_cases()
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size)
