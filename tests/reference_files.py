"""Where the reference's own test programs and benchmark templates are read from.

A reference checkout (IMEX_REFERENCE_DIR, else a directory `reference` beside the
repository) is preferred; without one the copies that tests/golden/stage_reference_files.py
put under the git-ignored baseline/_ref/ are used (that is what a GPU machine sees).  A
test whose file is in neither place is skipped."""
import os

import pytest

from golden.stage_reference_files import STAGE, TREES, reference_dir

REFERENCE = reference_dir()


def find(rel):
    """Path of the reference file `rel` (e.g. "test/PlaidML/OpTest.Relu.mlir"), or None."""
    if REFERENCE and os.path.exists(os.path.join(REFERENCE, rel)):
        return os.path.join(REFERENCE, rel)
    for src, _, dest in TREES:
        if rel == src or rel.startswith(src + "/"):
            cand = os.path.join(STAGE, dest, rel[len(src):].lstrip("/"))
            if os.path.exists(cand):
                return cand
    return None


def need(rel):
    path = find(rel)
    if path is None:
        pytest.skip("reference file %s is neither in a checkout nor staged" % rel)
    return path
