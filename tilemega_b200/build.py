"""Build libtilemega_b200.so in-tree with nvcc for sm_100a.

The library is the product: nothing in the package falls back to another
implementation when it is missing.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB_DIR = ROOT / "lib"
LIBRARY = LIB_DIR / "libtilemega_b200.so"
SOURCES = ("megakernel.cu", "runtime.cu", "plan_spec.cpp", "static_probe.cu")
HEADERS = ("params.h", "ptx.cuh", "plan_spec.h", "json.h")


def nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return found


def _stale() -> bool:
    if not LIBRARY.exists():
        return True
    built = LIBRARY.stat().st_mtime
    inputs = [CSRC / name for name in SOURCES + HEADERS] + [ROOT.parent / "include" / "tilemega_b200.h"]
    return any(path.stat().st_mtime > built for path in inputs)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile the CUDA sources into lib/libtilemega_b200.so (no GPU needed)."""
    if not force and not _stale():
        return LIBRARY
    LIB_DIR.mkdir(exist_ok=True)
    objects = []
    common = ["-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-gencode", "arch=compute_100a,code=sm_100a",
              "-lineinfo"]
    if verbose:
        common += ["-Xptxas", "-v"]
    build_dir = ROOT / "build"
    build_dir.mkdir(exist_ok=True)
    for name in SOURCES:
        obj = build_dir / (Path(name).stem + ".o")
        cmd = [nvcc(), *common, "-x", "cu" if name.endswith(".cu") else "c++", "-c", str(CSRC / name), "-o", str(obj)]
        subprocess.run(cmd, check=True)
        objects.append(str(obj))
    tmp = LIBRARY.with_suffix(".so.tmp")
    subprocess.run([nvcc(), "-shared", "-o", str(tmp), *objects, "-gencode", "arch=compute_100a,code=sm_100a",
                    "-Xlinker", "--no-undefined", "-ldl"], check=True)
    os.replace(tmp, LIBRARY)
    return LIBRARY


if __name__ == "__main__":
    print(build_library(force=True, verbose=bool(os.environ.get("VERBOSE"))))
