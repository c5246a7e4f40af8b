"""Loading a packed OrbitQuant artifact into resident device modules.

Mirrors the reference's ``load_orbitquant_artifact`` (``src/orbitquant/artifacts/loader.py:54-116``)
for the files the quantized-linear forward needs, as its writer lays them out
(``src/orbitquant/artifacts/writer.py:117-137``):

* ``quantization_config.json`` -- the ``OrbitQuantConfig`` fields;
* ``orbitquant_manifest.json`` -- ``quantized_modules`` (dotted names of the ``nn.Linear``
  leaves that were replaced), ``module_bits`` (per-module weight bit widths that differ from
  the config), ``adaln_modules``, ``checksums`` (sha256 per file);
* ``model.safetensors`` -- the model's state dict; a quantized leaf contributes exactly
  ``<name>.packed_weight_indices`` (flat uint8 bit stream), ``<name>.row_norms`` (bf16) and,
  when present, ``<name>.bias``; an RTN-INT4 (AdaLN) leaf ``<name>.packed_weight``,
  ``<name>.scales`` (bf16 ``[out_features, groups]``) and ``<name>.bias``;
* ``orbitquant_rotations.safetensors`` / ``orbitquant_codebooks.safetensors`` -- the RPBH
  permutation / signs per ``(dim, seed, block)`` and the Lloyd-Max tables per ``(dim, bits)``.

The packed bytes are consumed as they are (no repacking).  The rotation and codebook files
are not needed to run -- both are functions of ``(dim, seed, block)`` / ``(dim, bits)`` --
but they are compared bit for bit with the constants this package regenerates, so that an
artifact written with different constants is refused instead of silently mis-decoded.
"""
from __future__ import annotations

import dataclasses
import hashlib
import json
from pathlib import Path

import torch

from .adaln import RTNInt4Linear
from .config import OrbitQuantConfig
from .layers import OrbitQuantLinear

READ_FILES = ("model.safetensors", "orbitquant_codebooks.safetensors",
              "orbitquant_rotations.safetensors", "quantization_config.json")
_SHARED_FIELDS = ("weight_bits", "activation_bits", "rotation_seed", "block_size", "codebook_version")


def sha256_file(path: Path) -> str:
    digest = hashlib.sha256()
    with Path(path).open("rb") as handle:
        for chunk in iter(lambda: handle.read(1 << 20), b""):
            digest.update(chunk)
    return digest.hexdigest()


def _parent_and_child(model: torch.nn.Module, name: str):
    parent_name, _, child = name.rpartition(".")
    parent = model.get_submodule(parent_name) if parent_name else model
    return parent, child


def _set_child(parent: torch.nn.Module, child: str, module: torch.nn.Module) -> None:
    if child.isdigit() and isinstance(parent, (torch.nn.ModuleList, torch.nn.Sequential)):
        parent[int(child)] = module
    elif isinstance(parent, torch.nn.ModuleDict):
        parent[child] = module
    else:
        setattr(parent, child, module)


def _verify_constants(model: torch.nn.Module, artifact: Path) -> None:
    from safetensors.torch import load_file

    rotations = load_file(artifact / "orbitquant_rotations.safetensors", device="cpu")
    codebooks = load_file(artifact / "orbitquant_codebooks.safetensors", device="cpu")
    for name, module in model.named_modules():
        if not isinstance(module, OrbitQuantLinear):
            continue
        rot = module.rotation
        prefix = f"dim{rot.dim}_seed{rot.seed}_block{rot.block_size}"
        for field in ("permutation", "signs"):
            stored = rotations.get(f"{prefix}.{field}")
            if stored is None:
                raise ValueError(f"{name}: the artifact holds no rotation {prefix}")
            mine = getattr(rot, field).cpu()
            if stored.shape != mine.shape or not torch.equal(stored.to(torch.int64), mine.to(torch.int64)):
                raise ValueError(f"{name}: rotation {prefix}.{field} differs from the regenerated one")
        for book in (module.weight_codebook, module.activation_codebook):
            prefix = f"dim{book.dim}_bits{book.bits}"
            for field in ("centroids", "boundaries"):
                stored = codebooks.get(f"{prefix}.{field}")
                if stored is None:
                    raise ValueError(f"{name}: the artifact holds no codebook {prefix}")
                mine = getattr(book, field).cpu()
                if stored.shape != mine.shape or not torch.equal(stored.float(), mine.float()):
                    raise ValueError(f"{name}: codebook {prefix}.{field} differs from the regenerated one")


def load_orbitquant_artifact(model: torch.nn.Module, artifact_dir, *, strict: bool = True,
                             validate_checksums: bool = True, verify_constants: bool = True,
                             device=None) -> dict:
    """Replace the ``nn.Linear`` leaves named in the artifact's manifest by ``OrbitQuantLinear``
    modules and load the packed tensors into them.  Returns the manifest as a dict.

    ``device``: where the tensors are read to (default: the model's first parameter's device);
    with a CUDA device safetensors reads straight into device memory and the modules are
    ready to run.  ``validate_checksums`` checks the sha256 of every file this loader reads
    against the manifest (the reference additionally insists on its model card and prompt
    files, which a runtime does not need).  The manifest's ``adaln_modules`` become
    ``RTNInt4Linear`` modules."""
    from safetensors.torch import load_file

    artifact = Path(artifact_dir)
    for required in READ_FILES + ("orbitquant_manifest.json",):
        if not (artifact / required).is_file():
            raise FileNotFoundError(f"artifact file missing: {artifact / required}")
    config = OrbitQuantConfig.from_dict(json.loads((artifact / "quantization_config.json").read_text("utf-8")))
    manifest = json.loads((artifact / "orbitquant_manifest.json").read_text("utf-8"))
    for field in _SHARED_FIELDS:
        if field in manifest and manifest[field] != getattr(config, field):
            raise ValueError(f"manifest and quantization_config disagree on {field}: "
                             f"{manifest[field]!r} vs {getattr(config, field)!r}")
    if validate_checksums:
        sums = manifest.get("checksums", {})
        for name in READ_FILES:
            if name not in sums:
                raise ValueError(f"manifest holds no checksum for {name}")
            if sha256_file(artifact / name) != sums[name]:
                raise ValueError(f"checksum mismatch for {name}")
    module_bits = manifest.get("module_bits", {})
    for name in manifest.get("quantized_modules", []):
        module = model.get_submodule(name)
        if not isinstance(module, torch.nn.Linear):
            raise TypeError(f"expected Linear at {name}, got {type(module).__name__}")
        module_config = config
        bits = module_bits.get(name)
        if bits is not None and bits != config.weight_bits:
            module_config = dataclasses.replace(config, weight_bits=int(bits))
        replacement = OrbitQuantLinear.empty_from_linear(module, config=module_config, module_name=name)
        parent, child = _parent_and_child(model, name)
        _set_child(parent, child, replacement)

    for name in manifest.get("adaln_modules", []):
        module = model.get_submodule(name)
        if not isinstance(module, torch.nn.Linear):
            raise TypeError(f"expected Linear at {name}, got {type(module).__name__}")
        replacement = RTNInt4Linear.empty_from_linear(module, config=config, module_name=name)
        parent, child = _parent_and_child(model, name)
        _set_child(parent, child, replacement)

    if device is None:
        first = next(iter(model.parameters()), None)
        device = first.device if first is not None else torch.device("cpu")
    device = torch.device(device)
    state = load_file(artifact / "model.safetensors", device=str(device) if device.type == "cuda" else "cpu")
    missing, unexpected = model.load_state_dict(state, strict=False)
    if strict and (missing or unexpected):
        raise RuntimeError(f"artifact state mismatch: missing={list(missing)}, unexpected={list(unexpected)}")
    if device.type == "cuda":
        model.to(device)
    if verify_constants:
        _verify_constants(model, artifact)
    return manifest
