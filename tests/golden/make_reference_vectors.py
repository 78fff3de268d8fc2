#!/usr/bin/env python3
"""Transcribe the golden vectors of the reference's own hot-path tests.

Reads the reference's lit tests AS TEXT (nothing is executed): the
`arith.constant dense<...>` / `memref.global ... dense<...>` inputs and the
values on the `// CHECK` lines, and writes them to
tests/golden/reference_vectors.json.  The CPU oracle (oracle/) must reproduce
every one of them; tests/test_oracle_golden.py checks that.

    python tests/golden/make_reference_vectors.py [--reference /path/to/imex]

The JSON is committed; this script only needs the reference checkout when the
fixture is regenerated.
"""
import argparse
import json
import os
import re

HERE = os.path.dirname(os.path.abspath(__file__))


def _strip_comments(text):
    return "\n".join(l for l in text.splitlines() if not l.lstrip().startswith("//"))


def _parse_shape(ty):
    # "tensor<10x20xf32>" / "memref<3x3xbf16>" / "tensor<f32>"
    m = re.search(r"<([^>]*)>", ty)
    parts = m.group(1).split("x")
    dims = [int(p) for p in parts[:-1]]
    return dims, parts[-1].strip()


def _expand(value, dims):
    """dense payload (python literal or scalar) -> flat list in row-major order."""
    n = 1
    for d in dims:
        n *= d
    if not isinstance(value, list):
        return [value] * n
    flat = []

    def walk(v):
        if isinstance(v, list):
            for e in v:
                walk(e)
        else:
            flat.append(v)

    walk(value)
    assert len(flat) == n, (len(flat), dims)
    return flat


def dense_constants(text):
    """All dense<...> : type constants of a file, in textual order."""
    body = _strip_comments(text)
    out = []
    for m in re.finditer(r"dense<((?:[^<>]|\n)*?)>\s*:\s*((?:tensor|memref)<[^>]*>)", body):
        payload, ty = m.group(1), m.group(2)
        dims, elt = _parse_shape(ty)
        value = json.loads(re.sub(r"\s+", " ", payload))
        out.append({"dims": dims, "dtype": elt, "data": _expand(value, dims)})
    # memref.global form: "memref<3x3xf32> = dense<...>"
    for m in re.finditer(r"(memref<[^>]*>)\s*=\s*dense<((?:[^<>]|\n)*?)>", body):
        ty, payload = m.group(1), m.group(2)
        dims, elt = _parse_shape(ty)
        value = json.loads(re.sub(r"\s+", " ", payload))
        out.append({"dims": dims, "dtype": elt, "data": _expand(value, dims)})
    return out


def check_rows(text):
    """Bracketed rows on CHECK lines -> list of lists of floats."""
    rows = []
    for l in text.splitlines():
        m = re.match(r"\s*//\s*CHECK(?:-NEXT|-SAME)?:\s*(.*)$", l)
        if not m:
            continue
        s = m.group(1).strip()
        if "Unranked Memref" in s or "rank =" in s or "ALLCLOSE" in s:
            continue
        nums = re.findall(r"-?\d+(?:\.\d+)?(?:[eE][-+]?\d+)?", s)
        if nums:
            rows.append([float(x) for x in nums])
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("IMEX_REFERENCE_DIR"),
                    required="IMEX_REFERENCE_DIR" not in os.environ,
                    help="checkout of intel/mlir-extensions (default: $IMEX_REFERENCE_DIR)")
    ap.add_argument("--out", default=os.path.join(HERE, "reference_vectors.json"))
    args = ap.parse_args()

    def read(rel):
        with open(os.path.join(args.reference, rel)) as f:
            return f.read()

    cases = []

    def add(name, rel, op, consts, expected, **extra):
        case = {"name": name, "source": rel, "op": op, "inputs": consts,
                "expected": expected}
        case.update(extra)
        cases.append(case)

    rel = "test/PlaidML/OpTest.Matmul.mlir"
    t = read(rel)
    c = dense_constants(t)
    add("matmul_5x3x2_f32", rel, "matmul_f32", c[:2], sum(check_rows(t), []),
        compare="exact")

    rel = "test/PlaidML/OpTest.GEMM_FLOAT32.mlir"
    t = read(rel)
    c = dense_constants(t)
    add("gemm_3x3_f32_cinit", rel, "matmul_f32_cinit", c[:3], sum(check_rows(t), []),
        compare="printed6")

    rel = "test/PlaidML/CppEdsl.Dot.mlir"
    t = read(rel)
    c = dense_constants(t)
    add("dot_8x16x32_f32", rel, "matmul_f32", c[:2], check_rows(t)[0],
        compare="exact", expected_rows="first")

    rel = "test/PlaidML/CppEdsl.BigDot.mlir"
    t = read(rel)
    c = dense_constants(t)
    # 2048^3 splats: keep the splat value only, the test expands it.
    add("bigdot_2048_f32", rel, "matmul_f32_splat",
        [{"dims": x["dims"], "dtype": x["dtype"], "splat": x["data"][0]} for x in c[:2]],
        sorted(set(sum(check_rows(t), []))), compare="exact_all_equal")

    rel = "test/PlaidML/CppEdsl.DotF16_AccF32.mlir"
    t = read(rel)
    c = dense_constants(t)
    add("dot_f16_accf32_8x16x32", rel, "matmul_f16_f32_truncf16", c[:2],
        sorted(set(check_rows(t)[0])), compare="exact_all_equal")

    rel = "test/SPIRV/OpTest.GEMM_BF16_ACC_F32.mlir"
    t = read(rel)
    c = dense_constants(t)
    by = {}
    for x in c:
        by.setdefault(x["dtype"], []).append(x)
    # order in file: C init (f32 splat 1.0), B (bf16), A (bf16), ref result (f32)
    add("gemm_3x3_bf16_accf32", rel, "matmul_bf16_f32_cinit",
        [by["bf16"][1], by["bf16"][0], by["f32"][0]], by["f32"][1]["data"],
        compare="allclose")

    rel = "test/PlaidML/OpTest.Softmax.mlir"
    t = read(rel)
    c = dense_constants(t)
    add("softmax_10x20_f32", rel, "softmax_plaidml", c[:1], sum(check_rows(t), []),
        compare="printed6")

    rel = "test/PlaidML/OpTest.Sum.mlir"
    t = read(rel)
    c = dense_constants(t)
    add("sum_10x20_f32", rel, "reduce_all", c[:1], sum(check_rows(t), []),
        compare="exact")

    rel = "test/PlaidML/OpTest.Transpose.mlir"
    t = read(rel)
    c = dense_constants(t)
    add("transpose_10x20_f32", rel, "transpose2d", c[:1], sum(check_rows(t), []),
        compare="exact")

    rel = "test/PlaidML/OpTest.Relu.mlir"
    t = read(rel)
    c = dense_constants(t)
    add("relu_4x5_f32", rel, "relu", c[:1], sum(check_rows(t), []),
        compare="printed6")

    rel = "test/Jax/qoc/jit_swapaxes.304_linalg.mlir"
    t = read(rel)
    c = dense_constants(t)
    add("swapaxes_2x1_i32", rel, "transpose2d", c[:1], sum(check_rows(t), []),
        compare="exact")

    with open(args.out, "w") as f:
        json.dump({"generated_by": "tests/golden/make_reference_vectors.py",
                   "cases": cases}, f, indent=1)
    print(f"wrote {len(cases)} cases to {args.out}")


if __name__ == "__main__":
    main()
