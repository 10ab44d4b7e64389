"""Fill `baseline/_ref/` with an unmodified copy of the reference checkout.

    python baseline/make_ref.py [--reference <path-to-reference-checkout>]

The reference is pure Python (Triton kernels + an engine), has no build system and nothing to install: a plain copy
of its tree is the whole "installation".  `baseline/_ref/` is git-ignored - it is somebody else's source - but it
travels with the working tree to a GPU machine, where
  * `bench.py --impl reference-triton` runs the reference's own Triton operators and runner on the GPU, and
  * the tests that load the reference's `engine/` on top of this package's `triton_kernels` drop-in find it.
Without the directory those legs report "unavailable" / skip.  The default source is a directory called `reference`
next to this repository.
"""
from __future__ import annotations

import argparse
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEST = HERE / "_ref"
KEEP = ("engine", "triton_kernels", "tests", "tools", "demo.py", "smoke_test_runtime.py", "tokenize_text.py", "LICENSE",
        "README.md", "README-EN.md")


def make_ref(reference: Path | None = None, force: bool = False) -> Path | None:
    """Copy the reference tree; returns the destination, or None when there is no reference checkout to copy."""
    src = Path(reference) if reference is not None else HERE.parent.parent / "reference"
    if not (src / "triton_kernels").is_dir() or not (src / "engine").is_dir():
        return None
    if DEST.exists():
        if not force and (DEST / "engine" / "runner.py").exists():
            return DEST
        shutil.rmtree(DEST)
    DEST.mkdir(parents=True)
    for name in KEEP:
        item = src / name
        if item.is_dir():
            shutil.copytree(item, DEST / name, ignore=shutil.ignore_patterns("__pycache__", "*.pyc"))
        elif item.is_file():
            shutil.copy2(item, DEST / name)
    return DEST


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    dest = make_ref(a.reference, a.force)
    if dest is None:
        sys.exit("no reference checkout found (pass --reference)")
    print(dest)
