"""CPU-side checks: the C-ABI library loads and exports every symbol the headers
declare, descriptor blobs round-trip, the partition rule and timing statistics
match the reference's definitions.  No CUDA call is made."""
import ctypes as C
import os
import re
import subprocess

import numpy as np
import pytest

from __graft_entry__ import ROOT, load_package
from oracle import oracle

pkg = load_package()
rt, B = pkg.runtime, pkg.blob


def _declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{]*\)\s*;", text)
    return sorted(set(n for n in names if n.startswith(("gpu", "mgpu", "imex", "_mlir_ciface", "print", "rtclock"))))


def test_runtime_library_exports_every_declared_symbol():
    names = _declared("imex_cuda_runtime.h")
    assert {"gpuCreateStream", "gpuStreamDestroy", "gpuMemAlloc", "gpuMemFree", "gpuMemCopy",
            "gpuModuleLoad", "gpuKernelGet", "gpuLaunchKernel", "gpuWait"} <= set(names)
    lib = C.CDLL(rt.LIB_PATH)
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    assert set(rt.EXPORTS) <= set(names)


def test_blob_layout_matches_header_and_round_trips():
    hdr = open(os.path.join(ROOT, "include", "imex_b200_blob.h")).read()
    magic = int(re.search(r"IMEX_BLOB_MAGIC\s+(0x[0-9A-Fa-f]+)", hdr).group(1), 16)
    assert magic == B.MAGIC and magic.to_bytes(8, "little") == b"IMXB200\0"
    for name, val in re.findall(r"(IMEX_OP_[A-Z0-9_]+)\s*=\s*(\d+)", hdr):
        assert getattr(B, name.replace("IMEX_", "")) == int(val)
    descs = [B.gemm("k0", 7, 8, 9, B.BF16, B.EPI_SILU, accumulate=True, bias=True, ldb=16, sm_margin=4),
             B.softmax("k1", 3, 5, True), B.transpose3d("k2", (2, 3, 4), (2, 0, 1)),
             B.fill_uniform("k3", 10, B.F32, 42, -1.0, 1.0, first=5)]
    data = B.pack_blob(descs)
    assert len(data) == 16 + 144 * len(descs)
    version, back = B.unpack_blob(data)
    assert version == 1
    for a, b in zip(descs, back):
        assert (a.name, a.op, a.in_dtype, a.out_dtype, a.epilogue, a.flags, a.sm_margin, a.dims,
                a.fparams) == (b.name, b.op, b.in_dtype, b.out_dtype, b.epilogue, b.flags,
                               b.sm_margin, b.dims, b.fparams)
    with pytest.raises(ValueError):
        B.unpack_blob(b"\x03\x02\x23\x07" + bytes(28))  # SPIR-V magic


def test_module_load_and_kernel_lookup_need_no_gpu():
    blob = B.Blob([B.gemm("test_kernel", 4, 8, 8), B.softmax("test_kernel_0", 2, 2)])
    mod = rt.gpuModuleLoad(None, blob.address, blob.size)
    assert mod and rt.gpuModuleLoad(None, blob.address, blob.size) == mod  # cached by address
    assert rt.gpuKernelGet(None, mod, b"test_kernel_0")


@pytest.mark.parametrize("code,msg", [
    ("buf = C.create_string_buffer(b'\\x03\\x02\\x23\\x07' + bytes(60)); "
     "rt.gpuModuleLoad(None, C.addressof(buf), 64)", "SPIR-V"),
    ("buf = C.create_string_buffer(bytes(64)); rt.gpuModuleLoad(None, C.addressof(buf), 64)",
     "bad blob magic"),
    ("b = B.Blob([B.gemm('a', 1, 8, 8)]); m = rt.gpuModuleLoad(None, b.address, b.size); "
     "rt.gpuKernelGet(None, m, b'nope')", "no kernel named"),
    ("b = B.Blob([B.KernelDesc('a', 99)]); rt.gpuModuleLoad(None, b.address, b.size)", "unknown op"),
])
def test_errors_follow_the_reference_convention(code, msg):
    """Failures print 'An exception was thrown: ...' to stdout and abort()
    (LevelZeroRuntimeWrappers.cpp:41-53)."""
    prog = ("import sys, ctypes as C; sys.path.insert(0, %r); from __graft_entry__ import load_package; "
            "p = load_package(); rt, B = p.runtime, p.blob; %s" % (ROOT, code))
    r = subprocess.run([os.sys.executable, "-c", prog], capture_output=True, text=True)
    assert r.returncode < 0  # killed by SIGABRT
    assert "An exception was thrown:" in r.stdout and msg in r.stdout


def test_partition_rule_matches_reference_formula():
    # lib/Dialect/NDArray/Extensions/MeshShardingExtensions.cpp:80-100: the LAST
    # extent % n shards get the extra element
    for n in (1, 2, 3, 4, 7, 8):
        for extent in (0, 1, 5, 8, 10, 1200, 32768, 65536, 65539):
            sizes = [rt.imexShardSize(s, n, extent) for s in range(n)]
            offs = [rt.imexShardOffset(s, n, extent) for s in range(n)]
            assert sum(sizes) == extent
            assert offs == [sum(sizes[:s]) for s in range(n)]
            assert sizes == [extent // n + (1 if s >= n - extent % n else 0) for s in range(n)]
    assert [rt.imexShardSize(s, 4, 10) for s in range(4)] == [2, 2, 3, 3]


STATS = ["avg", "min", "max", "median", "stddev", "variance", "P95", "P5", "middle_third"]


@pytest.mark.parametrize("n", [3, 4, 5, 10, 100, 101, 1000])
def test_statistics_match_reference_code(n):
    v = np.random.default_rng(n).gamma(2.0, 0.1, n).astype(np.float32)
    if oracle.ref_lib() is None:
        pytest.skip("oracle/_ref not built")
    for which, name in enumerate(STATS):
        ours = rt.stat(which, v.tolist())
        theirs = oracle.ref_stat(which, v)
        assert ours == pytest.approx(theirs, rel=1e-6), name


def test_statistics_definitions():
    v = [5.0, 1.0, 4.0, 2.0, 3.0]
    assert rt.stat(0, v) == 3.0 and rt.stat(1, v) == 1.0 and rt.stat(2, v) == 5.0
    assert rt.stat(3, v) == 4.0  # rank n/2 + 1 of the sorted values, as the reference takes it
    assert rt.stat(5, v) == pytest.approx(2.0) and rt.stat(4, v) == pytest.approx(2.0 ** 0.5)
    assert rt.stat(6, v) == 5.0 and rt.stat(7, v) == 1.0 and rt.stat(8, v) == pytest.approx(3.0)
    assert rt.stat(3, [7.0]) == 7.0  # clamped where the reference would read past the end


def test_expression_programs_assemble_and_pack():
    """Postfix text -> ImexExprCode bytes -> the four program words of the descriptor."""
    import struct
    code = B.assemble_expr("in0 log in1 abs add in0 sub")
    assert list(code) == [B.X_IN, B.X_UNARY["log"], B.X_IN + 1, B.X_UNARY["abs"], B.X_BINARY["add"],
                          B.X_IN, B.X_BINARY["sub"]]
    assert list(B.assemble_expr("row2 col3 mul c0 c1 max zero one min add")) == [
        B.X_ROWV + 2, B.X_COLV + 3, B.X_BINARY["mul"], B.X_C0, B.X_C1, B.X_BINARY["max"], B.X_ZERO, B.X_ONE,
        B.X_BINARY["min"], B.X_BINARY["add"]]
    d = B.expr("chain", 512, 1024, "in0 log in1 abs add in0 sub", B.F16, reduce_leading=True, consts=(0.5, 2.0))
    assert d.op == B.OP_EXPR and d.in_dtype == d.out_dtype == B.F16 and d.flags == B.FLAG_REDUCE_LEADING
    assert d.dims[:2] == (512, 1024)
    assert struct.pack("<4q", *d.dims[2:]).rstrip(b"\0") == code
    assert d.fparams == (0.5, 2.0)
    back = B.unpack_blob(B.pack_blob([d]))[1][0]
    assert back.dims == d.dims and back.flags == d.flags
    with pytest.raises(ValueError):
        B.assemble_expr("in0 frobnicate")
    with pytest.raises(ValueError):
        B.assemble_expr("in4")
    with pytest.raises(ValueError):
        B.assemble_expr(" ".join(["in0"] * 33))


def test_gemm_layout_and_attention_descriptors():
    d = B.gemm("g", 64, 128, 256, B.F16, B.EPI_RELU, bias=True, trans_a=True, trans_b=True, out_dtype=B.BF16)
    assert d.flags == B.FLAG_BIAS | B.FLAG_TRANS_A | B.FLAG_TRANS_B and d.out_dtype == B.BF16
    a = B.attention_fwd("a", 4, 4096, 64, B.F16, 0.5)
    assert a.op == B.OP_ATTENTION_FWD and a.dims[:3] == (4, 4096, 64) and a.fparams[0] == 0.5
    s = B.softmax("s", 16, 2000, dtype=B.BF16)
    assert s.in_dtype == s.out_dtype == B.BF16
