"""Packed-artifact load (the reference's on-disk format, written by the reference itself:
tests/golden/artifact_tiny, produced by tests/golden/make_artifact.py)."""
from __future__ import annotations

import json
import shutil
from pathlib import Path

import numpy as np
import pytest
import torch

from orbitquant_b200 import OrbitQuantLinear
from orbitquant_b200.artifacts import load_orbitquant_artifact

ARTIFACT = Path(__file__).resolve().parent / "golden" / "artifact_tiny"


class TinyBlock(torch.nn.Module):
    def __init__(self, dim, hidden):
        super().__init__()
        self.to_q = torch.nn.Linear(dim, dim)
        self.proj = torch.nn.Linear(dim, dim, bias=False)
        self.fc1 = torch.nn.Linear(dim, hidden)
        self.fc2 = torch.nn.Linear(hidden, dim)
        self.norm = torch.nn.LayerNorm(dim)
        self.mod = torch.nn.Linear(dim, 6 * dim)


class TinyModel(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.blocks = torch.nn.ModuleList([TinyBlock(64, 192), TinyBlock(64, 192)])
        self.head = torch.nn.Linear(64, 10)


def test_load_replaces_modules_and_reads_bytes_exactly():
    from safetensors.torch import load_file

    model = TinyModel()
    manifest = load_orbitquant_artifact(model, ARTIFACT)
    stored = load_file(ARTIFACT / "model.safetensors")
    assert manifest["quantized_modules"] and isinstance(model.head, torch.nn.Linear)
    for name in manifest["quantized_modules"]:
        module = model.get_submodule(name)
        assert isinstance(module, OrbitQuantLinear)
        assert module.weight_bits == manifest["module_bits"].get(name, 4)
        assert torch.equal(module.packed_weight_indices, stored[f"{name}.packed_weight_indices"])
        assert module.row_norms.dtype == torch.bfloat16
        assert torch.equal(module.row_norms, stored[f"{name}.row_norms"])
        assert (module.bias is None) == (f"{name}.bias" not in stored)
        keys = {k for k in model.state_dict() if k.startswith(name + ".")}
        assert {k[len(name) + 1:] for k in keys} <= {"bias", "packed_weight_indices", "row_norms"}
    from orbitquant_b200.adaln import RTNInt4Linear
    for name in manifest["adaln_modules"]:
        module = model.get_submodule(name)
        assert isinstance(module, RTNInt4Linear)
        assert torch.equal(module.packed_weight, stored[f"{name}.packed_weight"])
        assert torch.equal(module.scales, stored[f"{name}.scales"])
    assert len(manifest["adaln_modules"]) == 2
    assert model.get_submodule("blocks.1.to_q").weight_bits == 2
    assert model.get_submodule("blocks.1.fc1").weight_bits == 3


def test_corrupt_or_inconsistent_artifacts_are_refused(tmp_path):
    broken = tmp_path / "artifact"
    shutil.copytree(ARTIFACT, broken)
    data = bytearray((broken / "model.safetensors").read_bytes())
    data[-1] ^= 0x01
    (broken / "model.safetensors").write_bytes(bytes(data))
    with pytest.raises(ValueError, match="checksum"):
        load_orbitquant_artifact(TinyModel(), broken)

    other_seed = tmp_path / "seed"
    shutil.copytree(ARTIFACT, other_seed)
    cfg = json.loads((other_seed / "quantization_config.json").read_text())
    cfg["rotation_seed"] = 4
    (other_seed / "quantization_config.json").write_text(json.dumps(cfg))
    with pytest.raises(ValueError, match="rotation_seed"):
        load_orbitquant_artifact(TinyModel(), other_seed, validate_checksums=False)
    manifest = json.loads((other_seed / "orbitquant_manifest.json").read_text())
    manifest["rotation_seed"] = 4
    (other_seed / "orbitquant_manifest.json").write_text(json.dumps(manifest))
    with pytest.raises(ValueError, match="rotation"):   # stored permutation is seed 3's
        load_orbitquant_artifact(TinyModel(), other_seed, validate_checksums=False)

    missing = tmp_path / "missing"
    shutil.copytree(ARTIFACT, missing)
    (missing / "orbitquant_rotations.safetensors").unlink()
    with pytest.raises(FileNotFoundError):
        load_orbitquant_artifact(TinyModel(), missing)

    class Wrong(TinyModel):
        def __init__(self):
            super().__init__()
            self.blocks[0].to_q = torch.nn.Identity()
    with pytest.raises(TypeError):
        load_orbitquant_artifact(Wrong(), ARTIFACT)


@pytest.mark.gpu
def test_loaded_modules_reproduce_the_reference_forward():
    """Outputs of the reference's own modules (CPU, dequantised-weight mode) on a fixed input,
    stored beside the artifact, against this package's kernels on the loaded modules."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    dev = torch.device("cuda", 0)
    model = TinyModel()
    manifest = load_orbitquant_artifact(model, ARTIFACT, device=dev)
    ref = np.load(ARTIFACT / "reference_forward.npz")
    x = torch.from_numpy(ref["x"].copy()).view(torch.bfloat16).to(dev)
    h = torch.from_numpy(ref["h"].copy()).view(torch.bfloat16).to(dev)
    for name in manifest["adaln_modules"]:
        y = model.get_submodule(name)(x).float().cpu()
        expect = torch.from_numpy(ref[name.replace(".", "__")])
        assert float((y - expect).norm() / expect.norm()) < 4e-3, name
    for name in manifest["quantized_modules"]:
        module = model.get_submodule(name)
        assert module.packed_weight_indices.device.type == "cuda"
        y = module(h if module.in_features == 192 else x).float().cpu()
        expect = torch.from_numpy(ref[name.replace(".", "__")])
        rel = float((y - expect).norm() / expect.norm())
        # the reference ran bf16 x dequantised-bf16-weight F.linear: bf16 weight rounding
        # (2^-9 relative) is the gap, not the kernels
        assert rel < 6e-3, (name, rel)
