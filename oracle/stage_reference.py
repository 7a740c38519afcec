"""Stage the reference's own hot-path files for runs on a machine that has no reference checkout.

TEST INFRASTRUCTURE ONLY: nothing in the product package imports what this script stages.

    python oracle/stage_reference.py [--reference /path/to/WorldAttention] [--dest baseline/_ref]

Copies, byte for byte, the files of the reference project that implement or test the path this
repository replaces -- `wan/modules/hsa/`, `pipeline/hkv/`, `trainer/hsa_stage.py`, `tests/` -- into a
directory that version control ignores (reference sources are never committed) but that travels
with the working tree.  Two consumers:

* `tests/test_reference_suite_gpu.py` runs the reference's own tests from there against this
  package (the reference's import paths aliased onto it, default device set to CUDA);
* `bench.py` times the reference's PyTorch CPU path and its Triton kernel from there.

Both skip, saying so, when the directory is absent.  The reference checkout is found through
`--reference`, then `$WORLDATTENTION_REFERENCE`, then the default location in `DEFAULT_REFERENCE`.
"""
from __future__ import annotations

import argparse
import os
import shutil
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEFAULT_DEST = os.path.join(ROOT, "baseline", "_ref")
PARTS = ["wan/modules/hsa", "pipeline/hkv", "trainer/hsa_stage.py", "tests"]
DEFAULT_REFERENCE = "/root/reference"


def find_reference(explicit: str | None = None) -> str | None:
    for cand in (explicit, os.environ.get("WORLDATTENTION_REFERENCE"), DEFAULT_REFERENCE):
        if cand and os.path.isdir(os.path.join(cand, "wan", "modules", "hsa")):
            return cand
    return None


def stage(reference: str, dest: str = DEFAULT_DEST) -> list[str]:
    """Copy PARTS of `reference` under `dest`; returns the relative paths of the files written."""
    written = []
    for part in PARTS:
        src = os.path.join(reference, part)
        if os.path.isdir(src):
            for folder, _, files in os.walk(src):
                for name in sorted(files):
                    if name.endswith(".py"):
                        rel = os.path.relpath(os.path.join(folder, name), reference)
                        written.append(rel)
        elif os.path.isfile(src):
            written.append(part)
        else:
            raise FileNotFoundError(f"{src} is missing from the reference checkout")
    for rel in written:
        target = os.path.join(dest, rel)
        os.makedirs(os.path.dirname(target), exist_ok=True)
        shutil.copyfile(os.path.join(reference, rel), target)
    return written


def staged(dest: str = DEFAULT_DEST) -> bool:
    return os.path.isfile(os.path.join(dest, "wan", "modules", "hsa", "attention.py")) and \
        os.path.isdir(os.path.join(dest, "tests"))


def import_staged(dest: str = DEFAULT_DEST):
    """Import the staged reference modules without their package `__init__` chains (which pull in the whole
    model zoo): empty parent packages whose search path is the staged tree.  Returns `(hsa, hkv)` modules."""
    import importlib
    import types
    for name, sub in (("wan", "wan"), ("wan.modules", "wan/modules"), ("pipeline", "pipeline"), ("trainer", "trainer")):
        if name not in sys.modules:
            module = types.ModuleType(name)
            module.__path__ = [os.path.join(dest, sub)]
            sys.modules[name] = module
    return importlib.import_module("wan.modules.hsa"), importlib.import_module("pipeline.hkv")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None)
    ap.add_argument("--dest", default=DEFAULT_DEST)
    args = ap.parse_args()
    ref = find_reference(args.reference)
    if ref is None:
        sys.exit("no reference checkout found (pass --reference or set WORLDATTENTION_REFERENCE)")
    files = stage(ref, args.dest)
    print(f"staged {len(files)} files from {ref} into {args.dest}")
