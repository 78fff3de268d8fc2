"""The benchmark driver (counterpart of the reference's benchmarks/bench_imex.in): template
instantiation rules of the reference's CMake files, option handling, report format."""
import os
import subprocess
import sys

import pytest

from __graft_entry__ import ROOT

SCRIPT = os.path.join(ROOT, "mlir-extensions_b200", "bench_imex.py")
import reference_files  # noqa: E402  (tests/reference_files.py: checkout or staged copies)


def _run(*args, cwd=None):
    return subprocess.run([sys.executable, SCRIPT, *args], capture_output=True, text=True, cwd=cwd)


def _fake_benchmarks(tmp_path):
    """A benchmarks/ folder with the file layout of the reference's and one-line templates."""
    root = tmp_path / "benchmarks"
    for name, shapes, dtypes, templates in [
            ("relu", ["1x2x3x4", "5x6"], ["f32", "f16"], {"relu_gpu.mlir.in": "@shape@|@dtype@|@affine_map@|@iterator_types@"}),
            ("softmax", ["16x2000", "2x3x4"], ["f32"], {"softmax_gpu.mlir.in": "@shape@|@batch_size@|@dtype@"}),
            ("transpose", ["128x136", "16x96x96"], ["f32"],
             {"transpose2d_gpu.mlir.in": "2d|@in_shape@|@out_shape@|@dtype@",
              "transpose3d_gpu.mlir.in": "3d|@in_shape@|@out_shape@|@dtype@"}),
            ("kLoopFusion", None, ["bf16"], {"kLoopFusion.mlir.in": "@dtype@"})]:
        d = root / name
        d.mkdir(parents=True)
        if shapes is not None:
            (d / (name + ".shapes.in")).write_text("\n".join(shapes) + "\n")
        (d / (name + ".dtypes.in")).write_text("\n".join(dtypes) + "\n")
        for fn, text in templates.items():
            (d / fn).write_text(text)
    return str(root)


def test_templates_are_filled_by_the_reference_rules(tmp_path):
    sys.path.insert(0, os.path.dirname(SCRIPT))
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench_imex", SCRIPT)
    bi = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bi)
    root, out = _fake_benchmarks(tmp_path), str(tmp_path / "gen")
    files = bi.instantiate(root, "relu", out)
    assert sorted(os.path.basename(f) for f in files) == ["relu_1x2x3x4_f16.mlir", "relu_1x2x3x4_f32.mlir",
                                                           "relu_5x6_f16.mlir", "relu_5x6_f32.mlir"]
    text = open(os.path.join(out, "relu", "gpu", "relu_1x2x3x4_f16.mlir")).read()
    assert text == '1x2x3x4|f16|d0, d1, d2, d3|"parallel", "parallel", "parallel", "parallel"'
    files = bi.instantiate(root, "softmax", out)                      # rank-3 shapes are skipped
    assert [os.path.basename(f) for f in files] == ["softmax_16x2000_f32.mlir"]
    assert open(files[0]).read() == "16x2000|16|f32"
    files = bi.instantiate(root, "transpose", out)
    assert open(files[0]).read() == "2d|128x136|136x128|f32"
    assert open(files[1]).read() == "3d|16x96x96|96x96x16|f32"
    files = bi.instantiate(root, "kLoopFusion", out)
    assert [os.path.basename(f) for f in files] == ["kLoopFusion_512x1024_bf16.mlir"]


def test_runtime_selection_follows_the_reference_script(tmp_path):
    r = _run()
    assert r.returncode != 0 and "Please select a runtime" in r.stderr
    r = _run("-c")
    assert r.returncode != 0 and "no CPU execution path" in r.stderr
    r = _run("-b")
    assert r.returncode != 0 and "--benchmarks" in r.stderr
    r = _run("-b", str(tmp_path / "nothing.mlir"))
    assert r.returncode != 0


def test_dry_run_of_a_single_file_writes_the_report(tmp_path):
    fixture = os.path.join(ROOT, "tests", "mlir", "fused_elementwise.mlir")
    report = tmp_path / "report.txt"
    r = _run("-b", "--emit-plan", "--report", str(report), fixture)
    assert r.returncode == 0, r.stdout + r.stderr
    lines = report.read_text().splitlines()
    assert any(l.startswith("================ Imex Perf (B200) @") for l in lines)
    kernels = [l for l in lines if l.startswith("fused_elementwise.mlir: kernel ")]
    assert len(kernels) == 3 and "+reduce_leading" in kernels[2]


def test_the_whole_reference_grid_becomes_kernels(tmp_path):
    """Every instance of the reference's benchmark grid (7 benchmarks x shapes x f32 / f16 / bf16)
    is recognised: one launch each."""
    report = tmp_path / "report.txt"
    benchmarks = os.path.dirname(os.path.dirname(reference_files.need("benchmarks/relu/relu.shapes.in")))
    r = _run("-b", "--emit-plan", "--benchmarks", benchmarks, "--out", str(tmp_path / "gen"),
             "--report", str(report))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    lines = [l for l in report.read_text().splitlines() if ": kernel " in l]
    assert len(lines) == 39 and not any("FAILED" in l for l in report.read_text().splitlines())
    per_file = {}
    for l in lines:
        per_file.setdefault(l.split(":")[0], []).append(l)
    assert all(len(v) == 1 for v in per_file.values())
