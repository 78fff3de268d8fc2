"""Host runner utilities (libimex_runner_utils.so): exported symbols, the memref
printer format the reference's CHECK lines pin, allclose / GEMM agreement with
the reference's own code (oracle/_ref) and with the oracle."""
import ctypes as C
import os
import re
import subprocess
import sys

import numpy as np
import pytest

from __graft_entry__ import ROOT
from oracle import oracle

LIB = os.path.join(ROOT, "mlir-extensions_b200", "lib", "libimex_runner_utils.so")


class Unranked(C.Structure):
    _fields_ = [("rank", C.c_int64), ("descriptor", C.c_void_p)]


def make_memref(arr):
    """(Unranked, keepalive) for a C-contiguous numpy array."""
    rank = arr.ndim
    words = (C.c_int64 * (3 + 2 * rank))()
    words[0] = words[1] = arr.ctypes.data
    words[2] = 0
    strides = [s // arr.itemsize for s in arr.strides]
    for d in range(rank):
        words[3 + d] = arr.shape[d]
        words[3 + rank + d] = strides[d]
    u = Unranked(rank, C.addressof(words))
    return u, (words, arr)


def test_exports_every_declared_symbol():
    text = open(os.path.join(ROOT, "include", "imex_runner_utils.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b([A-Za-z_][A-Za-z0-9_]*)\s*\([^;{]*\)\s*;", text))
    lib = C.CDLL(LIB)
    assert {"_mlir_ciface_gemmBF16BF16F32", "printMemrefF32", "rtclock",
            "_mlir_ciface_fillResource1DRandomBF16", "_mlir_ciface_printAllcloseF32"} <= names
    missing = [n for n in sorted(names) if not hasattr(lib, n)]
    assert not missing, missing


PRINT_PROG = r"""
import sys, numpy as np, ctypes as C
sys.path.insert(0, %r)
from tests.test_runner_utils import make_memref, LIB
lib = C.CDLL(LIB)
a = np.array([[14.1, 14.8, 14.6], [11, 13, 10.5]], np.float32)
u, k = make_memref(a); lib._mlir_ciface_printMemrefF32(C.byref(u))
lib.printMemrefI32.argtypes = [C.c_int64, C.c_void_p]
s = np.array(-10, np.int32); u, k = make_memref(s); lib.printMemrefI32(u.rank, u.descriptor)
t = np.arange(8, dtype=np.int32).reshape(2, 2, 2); u, k = make_memref(t); lib._mlir_ciface_printMemrefI32(C.byref(u))
x = np.array([[0.0715685, 0.11337]], np.float32); u, k = make_memref(x); lib._mlir_ciface_printMemrefF32(C.byref(u))
lib.printF64.argtypes = [C.c_double]; lib.printF64(0.125); lib.printNewline()
"""


def test_memref_printer_format():
    out = subprocess.run([sys.executable, "-c", PRINT_PROG % ROOT], capture_output=True, text=True,
                         check=True).stdout
    flat = re.sub(r"[ \t]+", " ", out)  # FileCheck canonicalises horizontal whitespace
    # test/PlaidML/OpTest.GEMM_FLOAT32.mlir:29-32, test/Integration/Dialect/Linalg/OpenCL/linalg_addf.mlir:24-27
    assert re.search(r"Unranked Memref base@ = 0x[0-9a-f]+ rank = 2 offset = 0 sizes = \[2, 3\] "
                     r"strides = \[3, 1\] data = \n\[\[14.1, 14.8, 14.6\], \n \[11, 13, 10.5\]\]", flat)
    # test/Jax/qoc/jit__reduce_sum.357_linalg.mlir:36-38
    assert "rank = 0 offset = 0 sizes = [] strides = [] data = \n[-10]" in flat
    # test/Jax/qoc/jit_matmul.338_linalg.mlir:46-49: rank 3, strides [4, 2, 1]
    assert "sizes = [2, 2, 2] strides = [4, 2, 1]" in flat and "[[[0, 1], \n [2, 3]], \n [[4, 5], \n [6, 7]]]" in flat
    assert "[[0.0715685, 0.11337]]" in flat  # six significant digits
    assert flat.rstrip().endswith("0.125")


def test_allclose_and_gemm_match_reference_code():
    lib = C.CDLL(LIB)
    lib._mlir_ciface_allcloseF32.restype = C.c_bool
    rng = np.random.default_rng(0)
    A = rng.uniform(-1, 1, (24, 40)).astype(np.float32)
    Bm = rng.uniform(-1, 1, (40, 16)).astype(np.float32)
    C0 = rng.uniform(-1, 1, (24, 16)).astype(np.float32)
    for is_bf16, fn in ((True, lib._mlir_ciface_gemmBF16BF16F32), (False, lib._mlir_ciface_gemmF16F16F32)):
        conv = oracle.to_bf16_bits if is_bf16 else oracle.to_f16_bits
        Ab, Bb, Cm = conv(A), conv(Bm), C0.copy()
        ua, ka = make_memref(Ab)
        ub, kb = make_memref(Bb)
        uc, kc = make_memref(Cm)
        fn(C.byref(ua), C.byref(ub), C.byref(uc))
        assert Cm.tobytes() == oracle.matmul_x16_f32(Ab, Bb, is_bf16, C_init=C0, loops=True).tobytes()
        if oracle.ref_lib() is not None:
            assert Cm.tobytes() == oracle.ref_gemm_x16_f32(Ab, Bb, is_bf16, C_init=C0).tobytes()
        ref = Cm.copy()
        ur, kr = make_memref(ref)
        assert lib._mlir_ciface_allcloseF32(C.byref(uc), C.byref(ur))
        ref[3, 3] += 0.5
        assert not lib._mlir_ciface_allcloseF32(C.byref(uc), C.byref(ur))
    # F16F16F16: result rounded through f16
    Ab, Bb, Cm = oracle.to_f16_bits(A), oracle.to_f16_bits(Bm), np.zeros((24, 16), np.float32)
    ua, ka = make_memref(Ab)
    ub, kb = make_memref(Bb)
    uc, kc = make_memref(Cm)
    lib._mlir_ciface_gemmF16F16F16(C.byref(ua), C.byref(ub), C.byref(uc))
    full = oracle.matmul_x16_f32(Ab, Bb, False, loops=True)
    assert np.array_equal(Cm, oracle.f16_bits_to_f32(oracle.to_f16_bits(full)))


def test_seeded_random_fill_is_reproducible():
    prog = ("import sys, numpy as np, ctypes as C; sys.path.insert(0, %r); "
            "from tests.test_runner_utils import make_memref, LIB; lib = C.CDLL(LIB); "
            "a = np.zeros(16, np.float32); u, k = make_memref(a); "
            "lib._mlir_ciface_fillResource1DRandomF32(C.byref(u), C.c_float(-1), C.c_float(1), C.c_bool(False)); "
            "b = np.zeros(8, np.uint16); u, k = make_memref(b); "
            "lib._mlir_ciface_fillResource1DBF16(C.byref(u), C.c_float(1.5)); "
            "print(a.tobytes().hex(), b.tolist())" % ROOT)
    env = dict(os.environ, IMEX_FILL_SEED="7")
    r1 = subprocess.run([sys.executable, "-c", prog], capture_output=True, text=True, env=env, check=True)
    r2 = subprocess.run([sys.executable, "-c", prog], capture_output=True, text=True, env=env, check=True)
    assert r1.stdout == r2.stdout and "16320" in r1.stdout  # 1.5 in bf16 = 0x3FC0
    vals = np.frombuffer(bytes.fromhex(r1.stdout.split()[0]), np.float32)
    assert vals.min() >= -1 and vals.max() < 1 and len(set(vals.tolist())) == 16
