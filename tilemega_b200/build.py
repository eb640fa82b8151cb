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
# (object name, source, extra flags). The kernel source is compiled twice, side by side:
# plain (unsharded dense plans), extended (tensor parallelism, mixture of experts, QK norm) and dense-batch
# (batch 16..64: GEMM stages on tcgen05 tiles) and e4m3 weights (the small-batch kernel with 8-bit weight pages).
UNITS = (("megakernel", "megakernel.cu", ()), ("megakernel_extended", "megakernel.cu", ("-DTMB_EXTENDED=1",)),
         ("megakernel_dense", "megakernel.cu", ("-DTMB_DENSE=1",)), ("megakernel_fp8", "megakernel.cu", ("-DTMB_FP8=1",)),
         ("runtime", "runtime.cu", ()), ("plan_spec", "plan_spec.cpp", ()), ("static_probe", "static_probe.cu", ()),
         ("pack", "pack.cu", ()), ("calibrate", "calibrate.cu", ()), ("encoder", "encoder.cu", ()))
# headers a source includes (directly or through another header): a unit is rebuilt when one of ITS headers changed
KERNEL_HEADERS = ("params.h", "ptx.cuh")
UNIT_HEADERS = {"megakernel.cu": KERNEL_HEADERS, "static_probe.cu": KERNEL_HEADERS, "calibrate.cu": ("ptx.cuh",), "pack.cu": (),
                "plan_spec.cpp": ("plan_spec.h", "json.h", "params.h")}
SOURCES = tuple(sorted({unit[1] for unit in UNITS}))
HEADERS = ("params.h", "ptx.cuh", "plan_spec.h", "json.h", "encoder.h")


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
              "-lineinfo", "-diag-suppress", "177"]   # 177: helpers one of the three kernel translation units does not use
    if verbose:
        common += ["-Xptxas", "-v"]
    build_dir = ROOT / "build"
    build_dir.mkdir(exist_ok=True)
    running = []
    for stem, name, flags in UNITS:
        obj = build_dir / (stem + ".o")
        objects.append(str(obj))
        inputs = [CSRC / name] + [CSRC / header for header in UNIT_HEADERS.get(name, HEADERS)] + [ROOT.parent / "include" / "tilemega_b200.h"]
        if not force and not verbose and obj.exists() and all(path.stat().st_mtime <= obj.stat().st_mtime for path in inputs):
            continue   # this unit's object is newer than its source and every header
        cmd = [nvcc(), *common, *flags, "-x", "cu" if name.endswith(".cu") else "c++", "-c", str(CSRC / name), "-o",
               str(obj)]
        running.append((cmd, subprocess.Popen(cmd)))
    for cmd, process in running:
        if process.wait() != 0:
            raise subprocess.CalledProcessError(process.returncode, cmd)
    tmp = LIBRARY.with_suffix(".so.tmp")
    subprocess.run([nvcc(), "-shared", "-o", str(tmp), *objects, "-gencode", "arch=compute_100a,code=sm_100a",
                    "-Xlinker", "--no-undefined", "-ldl"], check=True)
    os.replace(tmp, LIBRARY)
    return LIBRARY


if __name__ == "__main__":
    print(build_library(force=True, verbose=bool(os.environ.get("VERBOSE"))))
