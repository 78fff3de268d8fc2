"""The MLIR-text front end (imex-b200-runner) and the imex-runner command line.

CPU: the recogniser is exercised with --emit-plan (no GPU call): which kernels
a program becomes, the ABI call order, the refusal of IR outside the hot path,
the FileCheck-style checker, and — when a reference checkout is present — the
reference's own test and benchmark files.  GPU: the fixtures under tests/mlir/
run end to end and their CHECK lines (values from the CPU oracle) must match."""
import os
import re
import subprocess
import sys

import pytest

from __graft_entry__ import ROOT, load_package

load_package()
from mlir_extensions_b200 import filecheck, imex_runner  # noqa: E402

RUNNER = os.path.join(ROOT, "mlir-extensions_b200", "bin", "imex-b200-runner")
MLIR = os.path.join(ROOT, "tests", "mlir")
import reference_files  # noqa: E402  (tests/reference_files.py: checkout or staged copies)


def plan(path, *extra):
    r = subprocess.run([RUNNER, path, "--emit-plan", *extra], capture_output=True, text=True)
    return r.returncode, r.stdout, r.stderr


def kernels(out):
    return [re.sub(r"^kernel \S+ = ", "", l) for l in out.splitlines() if l.startswith("kernel ")]


def test_plan_of_the_matmul_fixture_and_abi_call_order():
    rc, out, err = plan(os.path.join(MLIR, "matmul_f32.mlir"))
    assert rc == 0, err
    ks = kernels(out)
    assert ks == ["gemm f32->f32 dims=[4,2,3] epilogue=0 flags=0",
                  "gemm f32->f32 dims=[4,2,3] epilogue=0 flags=1"]  # flags=1: C is also an input
    # the call sequence of the reference's lowered host code, per launch
    # (lib/Conversion/GPUXToLLVM/GPUXToLLVMPass.cpp:456-713)
    calls = [l.split("(")[0] for l in out.splitlines() if l.startswith("gpu")]
    i = calls.index("gpuModuleLoad")
    assert calls[i:i + 4] == ["gpuModuleLoad", "gpuKernelGet", "gpuLaunchKernel", "gpuWait"]
    assert calls[0] == "gpuCreateStream" and calls[-1] == "gpuStreamDestroy"
    assert calls.count("gpuCreateStream") == calls.count("gpuStreamDestroy") == 3  # one per function call


def test_fusions():
    rc, out, err = plan(os.path.join(MLIR, "matmul_bf16_relu_silu.mlir"))
    assert rc == 0, err
    ks = kernels(out)
    assert ks[0].startswith("gemm bf16->f32 +relu dims=[256,16,64] epilogue=1")  # extf + matmul + relu
    assert ks[6].startswith("gemm bf16->f32 +silu dims=[256,16,64] epilogue=2")  # matmul + sigmoid + mul
    assert [k.split()[0] for k in ks[:3]] == ["gemm", "row_sum", "reduce_all"]
    rc, out, err = plan(os.path.join(MLIR, "softmax_silu_transpose.mlir"))
    assert rc == 0, err
    assert [k.split()[0] for k in kernels(out)] == ["softmax", "silu", "transpose2d", "reduce_leading"]
    assert "flags=0" in kernels(out)[0]  # -FLT_MAX / maximumf form


def test_transposed_operands_bias_and_16bit_result_fuse_into_one_launch():
    rc, out, err = plan(os.path.join(MLIR, "matmul_f16_transposed_bias.mlir"))
    assert rc == 0, err
    ks = kernels(out)
    # matmul(B stored [N,K]) + broadcast bias + add + relu + truncf: flags = BIAS | TRANS_B
    assert ks[0] == "gemm f16->f16 B^T +bias +relu dims=[8,16,64] epilogue=1 flags=18"
    assert ks[2] == "gemm f16->f32 A^T dims=[8,16,64] epilogue=0 flags=8"
    assert len(ks) == 3
    assert out.count("gpuLaunchKernel(4 pointer params)") == 2  # A, B, C, bias


def test_elementwise_chains_fuse_into_one_launch_each():
    rc, out, err = plan(os.path.join(MLIR, "fused_elementwise.mlir"))
    assert rc == 0, err
    ks = kernels(out)
    assert [k.split(" dims")[0] for k in ks] == ["expr[7 ops, 2 inputs] f32", "expr[7 ops, 2 inputs] f16",
                                                 "expr[4 ops, 2 inputs] f32 +reduce_leading"]
    assert out.count("deferred:") == 8  # the generics that joined a later kernel


def test_ir_outside_the_hot_path_is_refused():
    rc, out, err = plan(os.path.join(MLIR, "unrecognised.mlir"))
    assert rc == 1
    assert "line 9" in err and "math.ctlz" in err and "loop nest" in err and "no CPU fallback" in err


def test_linalg_ops_on_buffers_are_refused_not_dropped():
    rc, out, err = plan(os.path.join(MLIR, "buffer_form.mlir"))
    assert rc == 1 and "line 8" in err and "on buffers" in err


def test_parse_errors_name_the_line(tmp_path):
    p = tmp_path / "bad.mlir"
    p.write_text("module {\n  func.func @main() {\n    %0 = foo.bar : f32\n    return\n  }\n}\n")
    rc, out, err = plan(str(p))
    assert rc == 1 and "line 3" in err and "foo.bar" in err
    p.write_text("func.func @main() {\n  %t = tensor.empty() : tensor<?x4xf32>\n  return\n}\n")
    rc, out, err = plan(str(p))
    assert rc == 1 and "line 2" in err and "too few extents" in err


def test_dynamic_extents_are_taken_from_the_values(tmp_path):
    """tensor<?x?xf32> in a callee: tensor.dim reads the extent the value has, tensor.empty(%d0, %d1)
    allocates it, and the op runs as the loop nest for those extents
    (the reference's test/PlaidML/OpTest.EltwiseAdd.dynamic.mlir has this form)."""
    p = tmp_path / "dyn.mlir"
    p.write_text("""#map = affine_map<(d0, d1) -> (d0, d1)>
module {
  func.func @twice(%a: tensor<?x?xf32>) -> tensor<?x?xf32> {
    %c0 = arith.constant 0 : index
    %c1 = arith.constant 1 : index
    %d0 = tensor.dim %a, %c0 : tensor<?x?xf32>
    %d1 = tensor.dim %a, %c1 : tensor<?x?xf32>
    %0 = tensor.empty(%d0, %d1) : tensor<?x?xf32>
    %1 = linalg.generic {indexing_maps = [#map, #map], iterator_types = ["parallel", "parallel"]}
         ins(%a : tensor<?x?xf32>) outs(%0 : tensor<?x?xf32>) {
      ^bb0(%x: f32, %y: f32):
        %2 = arith.addf %x, %x : f32
        linalg.yield %2 : f32
    } -> tensor<?x?xf32>
    return %1 : tensor<?x?xf32>
  }
  func.func @main() {
    %0 = arith.constant dense<1.5> : tensor<3x5xf32>
    %1 = tensor.cast %0 : tensor<3x5xf32> to tensor<?x?xf32>
    %2 = call @twice(%1) : (tensor<?x?xf32>) -> tensor<?x?xf32>
    return
  }
}
""")
    rc, out, err = plan(str(p))
    assert rc == 0, err
    assert "loopnest[2 parallel, 0 reduction dims, 15 threads]" in out


def test_filecheck_semantics():
    text = ("// CHECK: Unranked Memref base@ = {{(0x)?[-9a-f]*}}\n// CHECK-SAME: sizes = [2, 2]\n"
            "// CHECK-NEXT: [1,   2],\n// CHECK-NEXT: [3, 4]\n// CHECK-NOT: ALLCLOSE: FALSE\n// CHECK: done\n")
    good = "Unranked Memref base@ = 0x55aa rank = 2 offset = 0 sizes = [2, 2] strides = [2, 1] data = \n[[1,   2], \n [3,   4]]\nnoise\ndone\n"
    assert filecheck.check(good, text) is None
    assert "CHECK-NEXT" in filecheck.check(good.replace("[3,   4]", "[3,   5]"), text)
    assert "CHECK-NOT" in filecheck.check(good.replace("noise", "[ALLCLOSE: FALSE]"), text)
    assert "not found" in filecheck.check(good.replace("done", "d0ne"), text)
    assert filecheck.check("x\n", "// nothing here\n").startswith("no CHECK")
    assert filecheck.check("a\nFOO: 1\n", "// FOO: a\n// FOO-NEXT: FOO", prefix="FOO") is None


def test_imex_runner_command_line(tmp_path, capsys):
    # a RUN line of the reference that needs a runtime this build does not have is skipped
    assert imex_runner.main(["--requires=l0-runtime", "-i", "whatever.mlir"]) == 0
    assert imex_runner.main(["--requires=no-such-feature", "-i", "x.mlir"]) == 1
    capsys.readouterr()
    pp = tmp_path / "p.pp"
    pp.write_text("// comment\nbuiltin.module(\n    func.func(a,\n  b)\n    c)\n// End\n")
    assert imex_runner.flatten_pipeline(str(pp)) == "builtin.module(func.func(a,b),c)"
    # -n (no runner): nothing is executed, the plan is printed
    rc = imex_runner.main(["-i", os.path.join(MLIR, "matmul_f32.mlir"), "-n", "-f",
                           os.path.join(MLIR, "linalg-to-gpu.pp"), "-e", "main",
                           "--entry-point-result=void", "-o", str(tmp_path / "plan.txt")])
    assert rc == 0 and "gpuLaunchKernel" in (tmp_path / "plan.txt").read_text()


@pytest.mark.parametrize("rel,expect", [
    ("test/PlaidML/OpTest.Matmul.mlir", ["gemm"]),
    ("test/PlaidML/OpTest.GEMM_FLOAT32.mlir", ["gemm"]),  # a plan lists a loop's body once
    ("test/PlaidML/CppEdsl.Dot.mlir", ["gemm"]),
    ("test/PlaidML/CppEdsl.BigDot.mlir", ["gemm"]),
    ("test/PlaidML/CppEdsl.DotF16_AccF32.mlir", ["gemm", "convert"]),  # extf, matmul, truncf: one launch,
    ("test/PlaidML/OpTest.Softmax.mlir", ["softmax"]),
    ("test/PlaidML/OpTest.Sum.mlir", ["reduce_all"]),
    ("test/PlaidML/OpTest.Transpose.mlir", ["transpose2d"]),
    ("test/Jax/qoc/jit_swapaxes.304_linalg.mlir", ["transpose2d"]),
])
def test_reference_tests_are_recognised(rel, expect):
    rc, out, err = plan(reference_files.need(rel))
    assert rc == 0, err
    assert [k.split()[0] for k in kernels(out)] == expect


def test_f16_multiply_add_is_not_sent_to_the_tensor_cores():
    # test/PlaidML/CppEdsl.DotF16.mlir multiplies and adds in f16: rounding at every
    # step, which an f32-accumulating GEMM would not reproduce; it runs as a loop nest
    # (one thread per output, k ascending, f16 rounding after the multiply and after the add)
    rc, out, err = plan(reference_files.need("test/PlaidML/CppEdsl.DotF16.mlir"))
    assert rc == 0, err
    ks = kernels(out)
    assert not any(k.startswith("gemm") for k in ks) and any(k.startswith("loopnest[2 parallel, 1 reduction") for k in ks), ks


@pytest.mark.parametrize("name,subst,expect", [
    ("softmax/softmax_gpu", {"shape": "64x2000", "batch_size": "64"}, ["softmax dims=[64,2000"]),
    ("softmax/softmax_gpu", {"shape": "1024x2000", "batch_size": "1024", "dtype": "f16"},
     ["softmax f16 dims=[1024,2000"]),
    ("relu/relu_gpu", {"shape": "512x640x20x15", "affine_map": "d0, d1, d2, d3",
                       "iterator_types": '"parallel", "parallel", "parallel", "parallel"'},
     ["relu dims=[98304000"]),
    ("silu/silu_gpu", {"shape": "1x16x56x56", "affine_map": "d0, d1, d2, d3",
                       "iterator_types": '"parallel", "parallel", "parallel", "parallel"'},
     ["silu dims=[50176"]),
    ("transpose/transpose2d_gpu", {"in_shape": "1024x512", "out_shape": "512x1024"},
     ["transpose2d dims=[1024,512"]),
    ("transpose/transpose3d_gpu", None, None),
    ("reduce/reduce_gpu", {}, ["reduce_leading dims=[32,4194304"]),
    # the grid's 16-bit dtypes go through the fused elementwise kernel (per-operation rounding)
    ("reduce/reduce_gpu", {"dtype": "bf16"}, ["expr[1 ops, 1 inputs] bf16 +reduce_leading dims=[32,4194304"]),
    ("relu/relu_gpu", {"shape": "50x640x20x15", "affine_map": "d0, d1, d2, d3", "dtype": "f16",
                       "iterator_types": '"parallel", "parallel", "parallel", "parallel"'},
     ["expr[2 ops, 1 inputs] f16 dims=[1,9600000"]),
    ("silu/silu_gpu", {"shape": "1x16x56x56", "affine_map": "d0, d1, d2, d3", "dtype": "bf16",
                       "iterator_types": '"parallel", "parallel", "parallel", "parallel"'},
     ["expr[9 ops, 1 inputs] bf16 dims=[1,50176"]),
    # four generics (log, absf, addf, subf) -> one launch; with the column reduce behind: still one
    ("kLoopFusion/kLoopFusion", {}, ["expr[7 ops, 2 inputs] f32 dims=[1,524288"]),  # walked as one long row
    ("kLoopFusion/kLoopFusion", {"dtype": "f16"}, ["expr[7 ops, 2 inputs] f16 dims=[1,524288"]),
    ("kInputFusion/kInputFusion", {}, ["expr[5 ops, 2 inputs] f32 +reduce_leading dims=[512,1024"]),
    ("kInputFusion/kInputFusion", {"dtype": "bf16"}, ["expr[5 ops, 2 inputs] bf16 +reduce_leading dims=[512,1024"]),
])
def test_reference_benchmark_templates_are_recognised(tmp_path, name, subst, expect):
    src = open(reference_files.need("benchmarks/" + name + ".mlir.in")).read()
    if subst is None:  # 3-D transpose: fill the template from the file's own placeholders
        subst = {"in_shape": "16x96x96", "out_shape": "96x16x96", "affine_map_in": "d0, d1, d2",
                 "affine_map_out": "d1, d0, d2", "perm": "1, 0, 2"}
        expect = ["transpose3d"]
    subst = dict({"dtype": "f32"}, **subst)
    for k, v in subst.items():
        src = src.replace("@" + k + "@", v)
    leftover = re.findall(r"@[a-z_]+@", src)
    if leftover:
        pytest.skip("template placeholders not known here: %s" % sorted(set(leftover)))
    p = tmp_path / "bench.mlir"
    p.write_text(src)
    rc, out, err = plan(str(p))
    assert rc == 0, err
    ks = kernels(out)
    assert len(ks) == len(expect) and all(k.startswith(e) for k, e in zip(ks, expect)), ks


# ---------------------------------------------------------------- on the GPU
@pytest.mark.gpu
@pytest.mark.parametrize("fixture", ["matmul_f32.mlir", "matmul_bf16_relu_silu.mlir",
                                     "softmax_silu_transpose.mlir", "matmul_f16_transposed_bias.mlir",
                                     "fused_elementwise.mlir"])
def test_fixture_runs_and_matches_its_check_lines(fixture):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "mlir-extensions_b200", "imex_runner.py"),
                        "-i", os.path.join(MLIR, fixture), "-f", os.path.join(MLIR, "linalg-to-gpu.pp"),
                        "-e", "main", "--entry-point-result=void", "--filecheck"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr


@pytest.mark.gpu
def test_trace_shows_the_reference_call_sequence_on_the_device():
    r = subprocess.run([RUNNER, os.path.join(MLIR, "matmul_f32.mlir"), "--trace"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    calls = [l[6:].split("(")[0] for l in r.stderr.splitlines() if l.startswith("[abi] gpu")]
    i = calls.index("gpuModuleLoad")
    assert calls[i:i + 4] == ["gpuModuleLoad", "gpuKernelGet", "gpuLaunchKernel", "gpuWait"]
    assert "[-2,   -2.75]" in r.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("rel", ["test/PlaidML/OpTest.Matmul.mlir", "test/PlaidML/OpTest.Softmax.mlir",
                                 "test/PlaidML/OpTest.Sum.mlir", "test/PlaidML/OpTest.Transpose.mlir",
                                 "test/PlaidML/CppEdsl.Dot.mlir", "test/PlaidML/CppEdsl.DotF16_AccF32.mlir"])
def test_reference_tests_pass_their_own_check_lines(rel):
    path = reference_files.need(rel)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "mlir-extensions_b200", "imex_runner.py"),
                        "-i", path, "-e", "main", "--entry-point-result=void",
                        "--filecheck"], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr
