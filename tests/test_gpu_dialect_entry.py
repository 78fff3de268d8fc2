"""GPU-dialect entry IR: host code written with memref.alloc / gpu.alloc / gpu.memcpy /
gpu.launch_func / gpu.wait around a gpu.module of XeGPU-dialect device code — the form of the
reference's integration tests (test/Integration/Dialect/XeGPU/WG/gemm_*.mlir).  The runner
recognises what each gpu.func computes from its data flow and serves it with its own GEMM;
the host-side scf.for nests run as compiled register programs."""
import os
import subprocess

import pytest

from __graft_entry__ import ROOT, load_package

load_package()
from mlir_extensions_b200 import filecheck  # noqa: E402

import reference_files  # noqa: E402

RUNNER = os.path.join(ROOT, "mlir-extensions_b200", "bin", "imex-b200-runner")
ORACLE_RUNNER = os.path.join(ROOT, "oracle", "_cpu", "imex-oracle-runner")
FIXTURE = os.path.join(ROOT, "tests", "mlir", "gpu_dialect_gemm.mlir")
WG = "test/Integration/Dialect/XeGPU/WG/"


def _kernels(path):
    r = subprocess.run([RUNNER, path, "--emit-plan"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr[-800:]
    return [l.split(" = ", 1)[1] for l in r.stdout.splitlines() if l.startswith("kernel ")], r.stdout


def test_fixture_kernels_are_recognised_from_their_data_flow():
    ks, out = _kernels(FIXTURE)
    assert ks[0].startswith("gemm f16->f32 B^T") and "dims=[384,512,256]" in ks[0] and "flags=16" in ks[0]
    assert ks[1].startswith("gemm f16->f32 +bias +C") and "flags=3" in ks[1]
    assert out.count("host loop nest") == 3 and "host call @gemmF16F16F32" in out
    # the launch's arguments reach the descriptor's pointer order: 3 pointers, then 4 with the bias
    assert "gpuLaunchKernel(3 pointer params)" in out and "gpuLaunchKernel(4 pointer params)" in out


@pytest.mark.parametrize("name,expect", [
    ("gemm_4kx4kx4k_f16_f16_f32_bias.mlir", "gemm f16->f32 +bias +C"),
    ("gemm_4kx4kx4k_f16_f16_f32_bias_large_GRF.mlir", "gemm f16->f32 +bias"),
    ("gemm_4kx4kx4k_f16_f16_f32.mlir", "gemm f16->f32 "),
    ("gemm_4kx4kx4k_f16_f16_f16.mlir", "gemm f16->f16 "),
    ("simple_gemm_4kx4kx4k_f16_f16_f16.mlir", "gemm f16->f16 "),
    ("gemm_4kx4kx4k_transpose_a.mlir", "gemm f16->f32 A^T"),
    ("gemm_4kx4kx4k_transpose_b.mlir", "gemm f16->f32 B^T"),
])
def test_the_reference_gemm_integration_tests_are_planned(name, expect):
    ks, _ = _kernels(reference_files.need(WG + name))
    assert ks and all(k.startswith(expect) and "dims=[4096,4096,4096]" in k for k in ks), ks[:2]


def test_a_gpu_func_that_is_no_matrix_product_is_refused():
    path = reference_files.need(WG + "softmax_intra_sg_cross_lane.mlir")
    r = subprocess.run([RUNNER, path, "--emit-plan"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 1 and "not a kernel this runtime can stand in for" in r.stderr and "xegpu.dpas" in r.stderr


@pytest.mark.skipif(not os.path.exists(ORACLE_RUNNER), reason="oracle/_cpu/imex-oracle-runner is not built")
def test_fixture_passes_its_check_lines_on_the_cpu_checker():
    r = subprocess.run([ORACLE_RUNNER, FIXTURE, "--all-loopnests"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-800:] + r.stderr[-800:]
    assert filecheck.check(r.stdout, open(FIXTURE).read()) is None


@pytest.mark.gpu
def test_fixture_passes_its_check_lines_on_the_gpu():
    r = subprocess.run([RUNNER, FIXTURE], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-800:] + r.stderr[-800:]
    assert filecheck.check(r.stdout, open(FIXTURE).read()) is None


@pytest.mark.gpu
def test_the_reference_bias_gemm_test_prints_allclose_true():
    """The reference's own file, unmodified: 4096^3 f16 GEMM + bias through gpu.launch_func, its
    in-file CPU GEMM (runner utilities, one host thread: the slow part) and printAllcloseF32."""
    path = reference_files.need(WG + "gemm_4kx4kx4k_f16_f16_f32_bias.mlir")
    r = subprocess.run([RUNNER, path], capture_output=True, text=True, timeout=1200)
    assert r.returncode == 0, r.stdout[-800:] + r.stderr[-800:]
    assert filecheck.check(r.stdout, open(path).read()) is None
    assert "[ALLCLOSE: TRUE]" in r.stdout and "Average time (ms)" in r.stdout
