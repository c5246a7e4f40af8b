"""Writes tests/golden/artifact_tiny/: a tiny OrbitQuant artifact produced by the REFERENCE's
own quantiser and artifact writer (imported from its source tree in the build container),
plus the forward outputs of the reference modules on a fixed input.

    python tests/golden/make_artifact.py /path/to/reference

The loader under test (orbitquant_b200/artifacts.py) must read these files as they are.
"""
from __future__ import annotations

import shutil
import sys
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
OUT = HERE / "artifact_tiny"


class TinyBlock(torch.nn.Module):
    def __init__(self, dim: int, hidden: int):
        super().__init__()
        self.to_q = torch.nn.Linear(dim, dim)
        self.proj = torch.nn.Linear(dim, dim, bias=False)
        self.fc1 = torch.nn.Linear(dim, hidden)
        self.fc2 = torch.nn.Linear(hidden, dim)
        self.norm = torch.nn.LayerNorm(dim)      # stays unquantised
        self.mod = torch.nn.Linear(dim, 6 * dim)  # AdaLN modulation: RTN-INT4


class TinyModel(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.blocks = torch.nn.ModuleList([TinyBlock(64, 192), TinyBlock(64, 192)])
        self.head = torch.nn.Linear(64, 10)      # skipped


QUANTIZED = ["blocks.0.to_q", "blocks.0.proj", "blocks.0.fc1", "blocks.0.fc2",
             "blocks.1.to_q", "blocks.1.proj", "blocks.1.fc1", "blocks.1.fc2"]
LOW_BITS = {"blocks.1.to_q": 2, "blocks.1.fc1": 3}
ADALN = ["blocks.0.mod", "blocks.1.mod"]


def main(reference_root: str) -> None:
    sys.path.insert(0, str(Path(reference_root) / "src"))
    import dataclasses

    from orbitquant.artifacts.writer import save_orbitquant_artifact
    from orbitquant.config import OrbitQuantConfig
    from orbitquant.adaln import RTNInt4Linear
    from orbitquant.layers import OrbitQuantLinear

    torch.manual_seed(11)
    model = TinyModel()
    config = OrbitQuantConfig(weight_bits=4, activation_bits=4, rotation_seed=3, target_policy="generic_dit",
                              runtime_mode="dequant_bf16", activation_kernel_backend="cpu")
    x = (torch.randn(5, 64, generator=torch.Generator().manual_seed(12)) * 1.5).to(torch.bfloat16)
    h = (torch.randn(5, 192, generator=torch.Generator().manual_seed(13)) * 1.5).to(torch.bfloat16)
    forward = {}
    for name in QUANTIZED:
        parent = model.get_submodule(name.rsplit(".", 1)[0])
        child = name.rsplit(".", 1)[1]
        linear = getattr(parent, child)
        module_config = config
        if name in LOW_BITS:
            module_config = dataclasses.replace(config, weight_bits=LOW_BITS[name])
        quantized = OrbitQuantLinear.from_linear(linear, config=module_config, module_name=name)
        setattr(parent, child, quantized)
        inp = h if linear.in_features == 192 else x
        with torch.no_grad():
            forward[name] = quantized(inp).float().numpy()
    for name in ADALN:
        parent = model.get_submodule(name.rsplit(".", 1)[0])
        child = name.rsplit(".", 1)[1]
        quantized = RTNInt4Linear.from_linear(getattr(parent, child), config=config, module_name=name)
        setattr(parent, child, quantized)
        with torch.no_grad():
            forward[name] = quantized(x).float().numpy()
    summary = SimpleNamespace(quantized_modules=list(QUANTIZED), skipped_modules=["head"],
                              adaln_modules=list(ADALN))
    if OUT.exists():
        shutil.rmtree(OUT)
    save_orbitquant_artifact(model, OUT, config=config, source_model_id="synthetic/tiny",
                             source_revision="0", source_license="none", summary=summary)
    # Only what a loader reads is kept as a fixture; the writer's model card, prompt list,
    # model index and benchmark stub are not needed (their checksums stay in the manifest).
    for extra in ("README.md", "prompts.json", "model_index.json"):
        (OUT / extra).unlink()
    shutil.rmtree(OUT / "benchmark")
    shutil.rmtree(OUT / "assets", ignore_errors=True)
    np.savez_compressed(OUT / "reference_forward.npz", x=x.view(torch.int16).numpy(),
                        h=h.view(torch.int16).numpy(), **{k.replace(".", "__"): v for k, v in forward.items()})
    for path in sorted(OUT.rglob("*")):
        if path.is_file():
            print(f"{path.relative_to(OUT)}  {path.stat().st_size} B")


if __name__ == "__main__":
    import os

    main(sys.argv[1] if len(sys.argv) > 1 else
         os.environ.get("ORBITQUANT_REFERENCE_ROOT") or str(Path(__file__).resolve().parents[3] / "reference"))
