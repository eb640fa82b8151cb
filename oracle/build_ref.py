"""Recipe for oracle/_ref/: the reference's own CPU forward, made importable where the
reference tree is not.

    python oracle/build_ref.py [/path/to/TileMega]

The reference's CPU implementation of the decode path is a PyTorch module,
python/tilemega/serving/export.py (`Decoder`, dense models) together with
python/tilemega/moe/export.py (`SparseMLP`, mixture of experts); they need nothing but
torch. This script places exactly those files, with the three package markers they are
imported through, under oracle/_ref/tilemega/ -- a folder that is git-ignored, so no
reference source enters this repository's history, but that travels with a checkout to
the machine that runs the GPU tests and the benchmark. There `bench.py --impl reference`
and the `cpu_baseline` leg time `Decoder.execute` itself (kind "reference"); without the
folder they fall back to the restatement in oracle/decoder_oracle.py (kind "port").

TEST / MEASUREMENT INFRASTRUCTURE ONLY: nothing on the product path imports oracle/.
"""
from __future__ import annotations

import os
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref"
FILES = ("__init__.py", "serving/__init__.py", "serving/export.py", "moe/__init__.py", "moe/export.py")


def reference_tree(explicit: str | None = None) -> Path | None:
    """The reference checkout: the argument, $TILEMEGA_REFERENCE, or a `reference` folder
    beside this repository."""
    for candidate in (explicit, os.environ.get("TILEMEGA_REFERENCE"), HERE.parents[1] / "reference"):
        if candidate and (Path(candidate) / "python" / "tilemega" / "serving" / "export.py").exists():
            return Path(candidate)
    return None


def build(explicit: str | None = None) -> Path | None:
    """Fill oracle/_ref/ from the reference tree; None (and nothing touched) when there is no tree."""
    tree = reference_tree(explicit)
    if tree is None:
        return None
    source = tree / "python" / "tilemega"
    for name in FILES:
        out = TARGET / "tilemega" / name
        out.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(source / name, out)
    return TARGET


def load_decoder():
    """The reference's `Decoder` class from oracle/_ref/, or None when the folder is absent."""
    if not (TARGET / "tilemega" / "serving" / "export.py").exists():
        return None
    if str(TARGET) not in sys.path:
        sys.path.insert(0, str(TARGET))
    from tilemega.serving.export import Decoder
    return Decoder


if __name__ == "__main__":
    made = build(sys.argv[1] if len(sys.argv) > 1 else None)
    print(made if made else "no reference tree found: oracle/_ref/ not built")
