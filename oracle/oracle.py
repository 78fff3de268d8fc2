"""ctypes door to the CPU oracle — TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Loads oracle/liblinalg_oracle.so (the C restatement of the reference's
linalg -> loops CPU pipeline, see linalg_oracle.h) and, when it was built,
oracle/_ref/libimex_ref_utils.so (the reference's own runner-utils and timing
statistics compiled from its source files).  Only tests/, the smoke check and
bench.py's CPU-baseline legs import this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "liblinalg_oracle.so")
REF_PATH = os.path.join(HERE, "_ref", "libimex_ref_utils.so")

EPI_NONE, EPI_RELU, EPI_SILU = 0, 1, 2
SOFTMAX_BENCH, SOFTMAX_PLAIDML = 0, 1

_i64 = C.c_int64
_fp = C.POINTER(C.c_float)
_u16p = C.POINTER(C.c_uint16)
_u32p = C.POINTER(C.c_uint32)


def reference_dir():
    """The reference checkout: $IMEX_REFERENCE_DIR, else a directory `reference` beside the
    repository; None when neither exists."""
    for cand in (os.environ.get("IMEX_REFERENCE_DIR"),
                 os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")):
        if cand and os.path.isdir(os.path.join(cand, "lib", "ExecutionEngine")):
            return os.path.abspath(cand)
    return None


def build(reference=None):
    """Compile the oracle; also oracle/_ref when a reference checkout is found."""
    subprocess.check_call(["make", "-C", HERE, "all"], stdout=subprocess.DEVNULL)
    reference = reference or reference_dir()
    if reference and os.path.isdir(reference):
        subprocess.check_call(["make", "-C", HERE, "ref", f"REFERENCE={reference}"],
                              stdout=subprocess.DEVNULL)


def _load():
    if not os.path.exists(LIB_PATH):
        build()
    lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
    sig = {
        "oracle_matmul_f32_loops": [_fp, _fp, _fp, _i64, _i64, _i64],
        "oracle_matmul_f32_fast": [_fp, _fp, _fp, _i64, _i64, _i64],
        "oracle_matmul_x16_f32_loops": [_u16p, _u16p, _fp, _i64, _i64, _i64, C.c_int],
        "oracle_matmul_x16_f32_fast": [_u16p, _u16p, _fp, _i64, _i64, _i64, C.c_int],
        "oracle_matmul_x16_f32_rows": [_u16p, _u16p, _fp, _i64, _i64, _i64, _i64, C.c_int],
        "oracle_bias_add_f32": [_fp, _fp, _i64, _i64],
        "oracle_relu_f32": [_fp, _fp, _i64],
        "oracle_silu_f32": [_fp, _fp, _i64],
        "oracle_epilogue_f32": [_fp, _i64, C.c_int],
        "oracle_softmax_f32": [_fp, _fp, _i64, _i64, C.c_int],
        "oracle_reduce_rows_f32": [_fp, _fp, _i64, _i64],
        "oracle_reduce_leading_f32": [_fp, _fp, _i64, _i64],
        "oracle_reduce_all_f32": [_fp, _fp, _i64],
        "oracle_transpose2d_b32": [_u32p, _u32p, _i64, _i64],
        "oracle_transpose2d_b16": [_u16p, _u16p, _i64, _i64],
        "oracle_transpose3d_b32": [_u32p, _u32p, C.POINTER(_i64), C.POINTER(C.c_int)],
        "oracle_fill_uniform_f32": [_fp, _i64, C.c_uint64, _i64, C.c_float, C.c_float],
        "oracle_round_to_bf16": [_fp, _u16p, _i64],
        "oracle_round_to_f16": [_fp, _u16p, _i64],
    }
    for name, args in sig.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = None
    lib.oracle_unary.argtypes = [C.c_int, C.c_int, _fp, _fp, _i64]
    lib.oracle_unary.restype = C.c_int
    lib.oracle_binary.argtypes = [C.c_int, C.c_int, _fp, _fp, _fp, _i64]
    lib.oracle_binary.restype = C.c_int
    lib.oracle_reduce_leading_as.argtypes = [C.c_int, _fp, _fp, _i64, _i64]
    lib.oracle_reduce_leading_as.restype = None
    lib.oracle_attention_fwd_x16.argtypes = [_u16p, _u16p, _u16p, _u16p, _i64, _i64, _i64, C.c_float, C.c_int]
    lib.oracle_attention_fwd_x16.restype = None
    lib.oracle_allclose_f32.argtypes = [_fp, _fp, _i64]
    lib.oracle_allclose_f32.restype = C.c_int
    lib.oracle_max_rel_err_f32.argtypes = [_fp, _fp, _i64, C.c_double]
    lib.oracle_max_rel_err_f32.restype = C.c_double
    lib.oracle_rel_frobenius_f32.argtypes = [_fp, _fp, _i64]
    lib.oracle_rel_frobenius_f32.restype = C.c_double
    lib.oracle_bf16_to_f32.argtypes = [C.c_uint16]
    lib.oracle_bf16_to_f32.restype = C.c_float
    lib.oracle_f16_to_f32.argtypes = [C.c_uint16]
    lib.oracle_f16_to_f32.restype = C.c_float
    return lib


_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        _lib = _load()
    return _lib


def ref_lib():
    """The reference-built library, or None when oracle/_ref was not built."""
    global _ref
    if _ref is None and os.path.exists(REF_PATH):
        lib()
        r = C.CDLL(REF_PATH)
        r.ref_stat.argtypes = [C.c_int, _fp, _i64]
        r.ref_stat.restype = C.c_float
        r.ref_gemm_x16_f32.argtypes = [_u16p, _u16p, _fp, _i64, _i64, _i64, C.c_int]
        r.ref_gemm_x16_f32.restype = None
        r.ref_allclose_f32.argtypes = [_fp, _fp, _i64]
        r.ref_allclose_f32.restype = C.c_int
        _ref = r
    return _ref


def _f(a):
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return a.ctypes.data_as(_fp)


def _h(a):
    assert a.dtype == np.uint16 and a.flags.c_contiguous
    return a.ctypes.data_as(_u16p)


def _w(a):
    assert a.dtype.itemsize == 4 and a.flags.c_contiguous
    return a.ctypes.data_as(_u32p)


def f32c(a):
    return np.ascontiguousarray(a, dtype=np.float32)


# ---- 16-bit helpers ------------------------------------------------------
def to_bf16_bits(a):
    a = f32c(a)
    out = np.empty(a.shape, np.uint16)
    lib().oracle_round_to_bf16(_f(a), _h(out), a.size)
    return out


def to_f16_bits(a):
    a = f32c(a)
    out = np.empty(a.shape, np.uint16)
    lib().oracle_round_to_f16(_f(a), _h(out), a.size)
    return out


def bf16_bits_to_f32(b):
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def f16_bits_to_f32(b):
    return np.ascontiguousarray(b, np.uint16).view(np.float16).astype(np.float32)


# ---- ops -----------------------------------------------------------------
def matmul_f32(A, B, C_init=None, loops=False):
    A, B = f32c(A), f32c(B)
    M, K = A.shape
    K2, N = B.shape
    assert K == K2
    Cm = np.zeros((M, N), np.float32) if C_init is None else f32c(C_init).copy()
    fn = lib().oracle_matmul_f32_loops if loops else lib().oracle_matmul_f32_fast
    fn(_f(A), _f(B), _f(Cm), M, N, K)
    return Cm


def matmul_x16_f32(A_bits, B_bits, is_bf16=True, C_init=None, loops=False):
    A_bits = np.ascontiguousarray(A_bits, np.uint16)
    B_bits = np.ascontiguousarray(B_bits, np.uint16)
    M, K = A_bits.shape
    K2, N = B_bits.shape
    assert K == K2
    Cm = np.zeros((M, N), np.float32) if C_init is None else f32c(C_init).copy()
    fn = lib().oracle_matmul_x16_f32_loops if loops else lib().oracle_matmul_x16_f32_fast
    fn(_h(A_bits), _h(B_bits), _f(Cm), M, N, K, 1 if is_bf16 else 0)
    return Cm


def matmul_x16_f32_rows(A_bits, B_bits, row0, nrows, is_bf16=True):
    A_bits = np.ascontiguousarray(A_bits, np.uint16)
    B_bits = np.ascontiguousarray(B_bits, np.uint16)
    K, N = B_bits.shape
    Cm = np.zeros((nrows, N), np.float32)
    lib().oracle_matmul_x16_f32_rows(_h(A_bits), _h(B_bits), _f(Cm), row0, nrows, N, K,
                                     1 if is_bf16 else 0)
    return Cm


def bias_add(Cm, bias):
    Cm = f32c(Cm).copy()
    bias = f32c(bias)
    lib().oracle_bias_add_f32(_f(Cm), _f(bias), Cm.shape[0], Cm.shape[1])
    return Cm


def epilogue(Cm, epi):
    Cm = f32c(Cm).copy()
    lib().oracle_epilogue_f32(_f(Cm), Cm.size, int(epi))
    return Cm


def relu(x):
    return epilogue(x, EPI_RELU)


def silu(x):
    return epilogue(x, EPI_SILU)


DT_F32, DT_BF16, DT_F16 = 1, 2, 3
UNARY = {"negf": 32, "absf": 33, "log": 34, "exp": 35, "sqrt": 36, "rsqrt": 37, "tanh": 38, "relu": 39}
BINARY = {"addf": 64, "subf": 65, "mulf": 66, "divf": 67, "maximumf": 68, "minimumf": 69}


def round_as(x, dtype):
    """f32 array holding the values of `x` rounded to dtype (DT_*)."""
    x = f32c(x)
    if dtype == DT_BF16:
        return bf16_bits_to_f32(to_bf16_bits(x))
    if dtype == DT_F16:
        return f16_bits_to_f32(to_f16_bits(x))
    return x


def unary(op, x, dtype=DT_F32):
    """One elementwise generic `op` (IR mnemonic) in element type dtype; f32 array in and out."""
    x = f32c(x)
    y = np.empty_like(x)
    if lib().oracle_unary(UNARY[op], dtype, _f(x), _f(y), x.size):
        raise ValueError(op)
    return y


def binary(op, a, b, dtype=DT_F32):
    a, b = f32c(a), f32c(b)
    assert a.shape == b.shape
    y = np.empty_like(a)
    if lib().oracle_binary(BINARY[op], dtype, _f(a), _f(b), _f(y), a.size):
        raise ValueError(op)
    return y


def reduce_leading_as(x, dtype=DT_F32, init=None):
    """y[j] = init[j] + sum_i x[i,j] with every add rounded to dtype."""
    x = f32c(x)
    lead, inner = x.shape[0], int(np.prod(x.shape[1:]))
    y = np.zeros(x.shape[1:], np.float32) if init is None else f32c(init).copy()
    lib().oracle_reduce_leading_as(dtype, _f(x), _f(y), lead, inner)
    return y


def attention_fwd(q_bits, k_bits, v_bits, heads, sm_scale, is_bf16=False):
    """O bits [heads * n_ctx, d_head] of the reference test's CPU attention; inputs are
    uint16 arrays of that shape."""
    q, k, v = (np.ascontiguousarray(a, dtype=np.uint16) for a in (q_bits, k_bits, v_bits))
    rows, d = q.shape
    assert rows % heads == 0 and k.shape == q.shape == v.shape
    o = np.empty_like(q)
    lib().oracle_attention_fwd_x16(_h(q), _h(k), _h(v), _h(o), heads, rows // heads, d, sm_scale, int(is_bf16))
    return o


def softmax(x, flavour=SOFTMAX_BENCH):
    x = f32c(x)
    rows = int(np.prod(x.shape[:-1])) if x.ndim > 1 else 1
    cols = x.shape[-1] if x.ndim else 1
    y = np.empty_like(x)
    lib().oracle_softmax_f32(_f(x), _f(y), rows, cols, flavour)
    return y


def reduce_rows(x, init=None):
    x = f32c(x)
    rows, cols = x.shape
    y = np.zeros(rows, np.float32) if init is None else f32c(init).copy()
    lib().oracle_reduce_rows_f32(_f(x), _f(y), rows, cols)
    return y


def reduce_leading(x, init=None):
    x = f32c(x)
    lead = x.shape[0]
    inner = x.size // lead if lead else 0
    y = np.zeros(x.shape[1:], np.float32) if init is None else f32c(init).copy()
    lib().oracle_reduce_leading_f32(_f(x), _f(y), lead, inner)
    return y


def reduce_all(x, init=0.0):
    x = f32c(x)
    y = np.array([init], np.float32)
    lib().oracle_reduce_all_f32(_f(x), _f(y), x.size)
    return y[0]


def transpose2d(x):
    x = np.ascontiguousarray(x)
    rows, cols = x.shape
    y = np.empty((cols, rows), x.dtype)
    if x.dtype.itemsize == 4:
        lib().oracle_transpose2d_b32(_w(x), _w(y), rows, cols)
    elif x.dtype.itemsize == 2:
        lib().oracle_transpose2d_b16(x.view(np.uint16).ctypes.data_as(_u16p),
                                     y.view(np.uint16).ctypes.data_as(_u16p), rows, cols)
    else:
        raise TypeError(x.dtype)
    return y


def transpose3d(x, perm):
    x = np.ascontiguousarray(x)
    assert x.ndim == 3 and x.dtype.itemsize == 4
    y = np.empty(tuple(x.shape[p] for p in perm), x.dtype)
    dims = (_i64 * 3)(*x.shape)
    pp = (C.c_int * 3)(*perm)
    lib().oracle_transpose3d_b32(_w(x), _w(y), dims, pp)
    return y


def fill_uniform(shape, seed, lo, hi, first=0):
    v = np.empty(shape, np.float32)
    lib().oracle_fill_uniform_f32(_f(v), v.size, seed, first, lo, hi)
    return v


# ---- comparisons -----------------------------------------------------------
def allclose(got, ref):
    got, ref = f32c(got), f32c(ref)
    return bool(lib().oracle_allclose_f32(_f(got), _f(ref), got.size))


def max_rel_err(got, ref, floor_abs=1e-30):
    got, ref = f32c(got), f32c(ref)
    return float(lib().oracle_max_rel_err_f32(_f(got), _f(ref), got.size, floor_abs))


def rel_frobenius(got, ref):
    got, ref = f32c(got), f32c(ref)
    return float(lib().oracle_rel_frobenius_f32(_f(got), _f(ref), got.size))


# ---- the reference's own code (oracle/_ref) ------------------------------
def ref_gemm_x16_f32(A_bits, B_bits, is_bf16=True, C_init=None):
    r = ref_lib()
    A_bits = np.ascontiguousarray(A_bits, np.uint16)
    B_bits = np.ascontiguousarray(B_bits, np.uint16)
    M, K = A_bits.shape
    _, N = B_bits.shape
    Cm = np.zeros((M, N), np.float32) if C_init is None else f32c(C_init).copy()
    r.ref_gemm_x16_f32(_h(A_bits), _h(B_bits), _f(Cm), M, N, K, 0 if is_bf16 else 1)
    return Cm


def ref_stat(which, values):
    v = f32c(values)
    return float(ref_lib().ref_stat(which, _f(v), v.size))
