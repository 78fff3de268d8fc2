#!/usr/bin/env python3
"""Copies the reference's own hot-path test programs and benchmark templates into the
git-ignored baseline/_ref/ so that they travel with the working tree to a machine that has
no reference checkout (the GPU tests run the reference's tests against their own CHECK
lines; bench_imex.py instantiates the reference's benchmark grid).

    python tests/golden/stage_reference_files.py [REFERENCE_CHECKOUT]

Nothing staged is committed: baseline/_ref/ is listed in .gitignore.  The reference
checkout is found through IMEX_REFERENCE_DIR, else a directory `reference` beside the
repository.
"""
import os
import shutil
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
STAGE = os.path.join(ROOT, "baseline", "_ref")

# (directory inside the reference, file suffixes kept, destination under baseline/_ref/)
TREES = [
    ("test/PlaidML", (".mlir", ".pp"), "reference_tests/PlaidML"),
    ("test/Jax", (".mlir", ".pp"), "reference_tests/Jax"),
    ("test/Gen/PlaidML", (".mlir.in", ".pp"), "reference_tests/Gen/PlaidML"),
    ("test/Integration/Dialect/XeGPU/WG", (".mlir", ".pp"), "reference_tests/XeGPU/WG"),
    ("test/Dialect/NDArray/Extensions", (".mlir",), "reference_tests/NDArray/Extensions"),
    ("benchmarks", (".in", ".pp", ".txt"), "benchmarks"),
]


def reference_dir(explicit=None):
    """The reference checkout, or None: the argument, $IMEX_REFERENCE_DIR, or ../reference."""
    for cand in (explicit, os.environ.get("IMEX_REFERENCE_DIR"),
                 os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "lib", "ExecutionEngine")):
            return os.path.abspath(cand)
    return None


def stage(reference=None):
    ref = reference_dir(reference)
    if ref is None:
        return 0
    n = 0
    for rel, suffixes, dest in TREES:
        src_root = os.path.join(ref, rel)
        for d, _, files in os.walk(src_root):
            for f in files:
                if not f.endswith(suffixes):
                    continue
                out_dir = os.path.join(STAGE, dest, os.path.relpath(d, src_root))
                os.makedirs(out_dir, exist_ok=True)
                shutil.copyfile(os.path.join(d, f), os.path.join(out_dir, f))
                n += 1
    return n


if __name__ == "__main__":
    count = stage(sys.argv[1] if len(sys.argv) > 1 else None)
    print("staged %d files under %s" % (count, STAGE))
