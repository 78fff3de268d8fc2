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


def instantiate_gen_template(path, variant, out_dir):
    """One variant of a test/Gen template, by the rule of the reference's CMake function
    imex_gen_test (test/Gen/CMakeLists.txt:59-130): the header lines
    `// PLACEHOLDER NAME v0 v1 ...` list the values and variant i replaces every @NAME@ with
    its i-th value.  Returns (path of the written .mlir, {NAME: value}) or None when the
    template has fewer variants."""
    import re
    text = open(path).read()
    names = {}
    for m in re.finditer(r"^//\s*PLACEHOLDER\s+(\S+)\s+(.*)$", text, re.M):
        names[m.group(1)] = m.group(2).split()
    count = re.search(r"NUMVARIANTS\s+(\d+)", text)
    if not names or not count or variant >= int(count.group(1)):
        return None
    chosen = {k: v[variant] for k, v in names.items()}
    for k, v in chosen.items():
        text = text.replace("@" + k + "@", v)
    base = os.path.basename(path)[:-len(".mlir.in")]
    out = os.path.join(str(out_dir), "%s.%s.mlir" % (base, chosen.get("DTYPE", str(variant))))
    with open(out, "w") as f:
        f.write(text)
    return out, chosen
