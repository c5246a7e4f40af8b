"""Build ``orbitquant_b200/liborbit_b200.so`` (the C-ABI CUDA library) in-tree.

    python -m orbitquant_b200.build [-v] [--force]

One ``nvcc`` invocation per translation unit, sm_100a only (the kernels use tcgen05 /
TMEM / TMA instructions that exist on no other target), then one link.  The result sits
next to this file so that it travels with the source tree; nothing is installed.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB = HERE / "liborbit_b200.so"
OBJ_DIR = HERE / "csrc" / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    candidate = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(candidate).exists():
        raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")
    return candidate


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def needs_build() -> bool:
    if not LIB.exists():
        return True
    stamp = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "orbit_b200.h"]
    return any(p.stat().st_mtime > stamp for p in deps)


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    if not force and not needs_build():
        return LIB
    nvcc = _nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    flags = list(NVCC_FLAGS)
    if ptxas_info:
        flags += ["-Xptxas", "-v"]
    flags += os.environ.get("ORBIT_B200_NVCC_EXTRA", "").split()  # e.g. -DORBIT_TRACE
    # A host compiler that links libstdc++ statically breaks std::call_once in a shared
    # object; prefer the system one.
    if Path("/usr/bin/g++").exists():
        flags += ["-ccbin", "/usr/bin/g++"]

    def compile_one(src: Path) -> Path:
        obj = OBJ_DIR / (src.stem + ".o")
        cmd = [nvcc, *flags, "-c", str(src), "-o", str(obj)]
        if verbose:
            print(" ".join(cmd), flush=True)
        result = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or result.returncode != 0:
            sys.stderr.write(result.stdout + result.stderr)
        if result.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}")
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as pool:
        objects = list(pool.map(compile_one, sources()))
    link = [nvcc, "-shared", "-o", str(LIB), *map(str, objects),
            "-gencode", "arch=compute_100a,code=sm_100a"]
    if Path("/usr/bin/g++").exists():
        link += ["-ccbin", "/usr/bin/g++"]
    if verbose:
        print(" ".join(link), flush=True)
    subprocess.run(link, check=True)
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv,
                 ptxas_info="--ptxas" in sys.argv)
    print(path)
