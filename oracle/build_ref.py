"""Build the reference's own CPU packed-matmul kernels into ``oracle/_ref/``.

TEST INFRASTRUCTURE ONLY.  Nothing under ``oracle/`` is part of the product
path; it is the checker the GPU kernels are compared against and the timed CPU
baseline.

The reference ships its CPU path as C++17 sources that bind to torch through
the stable ABI (``native-kernels/orbitquant-packed-matmul/torch-ext/
torch_binding.cpp`` + ``orbitquant_packed_matmul_cpu/*.cpp``).  Its own JIT
recipe (``src/orbitquant/kernels/provision.py:394-412``) compiles exactly those
files with ``-O3 -DCPU_KERNEL``.  This script does the same with plain ``g++``
commands on the sources where they lie (no source is copied), and writes one
shared object:

    oracle/_ref/_orbitquant_ref_cpu.so

which registers the torch ops ``_orbitquant_ref_cpu::matmul_packed_weight``,
``::quantize_activations_cpu`` and ``::matmul_packed_adaln_int4_cpu``
(``torch-ext/torch_binding.cpp:7-31``).  ``oracle/ref_cpu.py`` loads it.

The system compiler ``/usr/bin/g++`` is used on purpose: a toolchain that links
libstdc++ statically produces a module that crashes inside the reference's
thread-count probe (``cpu_threads.cpp:35-64``).
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys
import sysconfig
from pathlib import Path

MODULE_NAME = "_orbitquant_ref_cpu"
HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"


def reference_root() -> Path:
    """The reference checkout: ``$ORBITQUANT_REFERENCE_ROOT``, else a directory named
    ``reference`` beside this repository."""
    env = os.environ.get("ORBITQUANT_REFERENCE_ROOT")
    return Path(env) if env else HERE.parent.parent / "reference"


def build(verbose: bool = False) -> Path | None:
    """Compile the reference CPU kernels; returns the .so path or None if the
    reference sources are not present (then a previously built file is kept)."""
    target = OUT_DIR / f"{MODULE_NAME}.so"
    root = reference_root() / "native-kernels" / "orbitquant-packed-matmul"
    if not root.is_dir():
        return target if target.exists() else None

    import torch
    from torch.utils import cpp_extension

    cxx = "/usr/bin/g++" if Path("/usr/bin/g++").exists() else "g++"
    sources = [root / "torch-ext" / "torch_binding.cpp"]
    sources += sorted((root / "orbitquant_packed_matmul_cpu").glob("*.cpp"))
    newest = max(p.stat().st_mtime for p in sources)
    if target.exists() and target.stat().st_mtime > max(newest, Path(__file__).stat().st_mtime):
        return target

    OUT_DIR.mkdir(parents=True, exist_ok=True)
    obj_dir = OUT_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    includes = [
        reference_root() / "src" / "orbitquant" / "kernels" / "_jit_support",
        root / "torch-ext",
        root / "orbitquant_packed_matmul_cpu",
        *map(Path, cpp_extension.include_paths()),
        Path(sysconfig.get_paths()["include"]),
    ]
    flags = [
        "-O3", "-std=c++17", "-fPIC", "-DCPU_KERNEL",
        f"-DTORCH_EXTENSION_NAME={MODULE_NAME}",
        f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
        "-Wno-ignored-attributes",
    ]
    for inc in includes:
        flags += ["-isystem" if "torch" in str(inc) and "torch-ext" not in str(inc) else "-I", str(inc)]

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        cmd = [cxx, *flags, "-c", str(src), "-o", str(obj)]
        if verbose:
            print(" ".join(cmd))
        subprocess.run(cmd, check=True)
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        objects = list(pool.map(compile_one, sources))

    lib_dirs = cpp_extension.library_paths()
    link = [cxx, "-shared", "-o", str(target), *map(str, objects)]
    for lib_dir in lib_dirs:
        link += [f"-L{lib_dir}", f"-Wl,-rpath,{lib_dir}"]
    link += ["-ltorch", "-ltorch_cpu", "-lc10", "-lpthread"]
    if verbose:
        print(" ".join(link))
    subprocess.run(link, check=True)
    return target


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv)
    print(path if path is not None else "reference sources not present; nothing built")
