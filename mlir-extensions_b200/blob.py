"""Kernel-descriptor blobs (include/imex_b200_blob.h) built from Python.

A blob is what the front end attaches to a gpu.module in place of the
reference's serialised SPIR-V (lib/Transforms/SerializeSPIRV.cpp:64-69) and
what gpuModuleLoad receives."""
import ctypes as C
import struct

MAGIC = 0x0030303242584D49
VERSION = 1
NAME_MAX = 64

OP_GEMM, OP_SOFTMAX, OP_REDUCE_ROWS, OP_REDUCE_LEADING, OP_REDUCE_ALL = 1, 2, 3, 4, 5
OP_TRANSPOSE2D, OP_TRANSPOSE3D, OP_ELTWISE, OP_FILL_UNIFORM, OP_FILL_NORMAL = 6, 7, 8, 9, 10
OP_EXPR, OP_ATTENTION_FWD, OP_LOOPNEST = 11, 12, 13
F32, BF16, F16, I32 = 1, 2, 3, 4
EPI_NONE, EPI_RELU, EPI_SILU = 0, 1, 2
FLAG_ACCUMULATE, FLAG_BIAS, FLAG_SOFTMAX_NEG_INF, FLAG_TRANS_A, FLAG_TRANS_B = 1, 2, 4, 8, 16
FLAG_REDUCE_LEADING = 32

DTYPE_BYTES = {F32: 4, I32: 4, BF16: 2, F16: 2}
_DESC = struct.Struct("<64s6I6q2f")  # ImexKernelDesc, 144 bytes
_HEADER = struct.Struct("<QII")      # ImexBlobHeader, 16 bytes
assert _DESC.size == 144 and _HEADER.size == 16


class KernelDesc:
    def __init__(self, name, op, in_dtype=F32, out_dtype=F32, epilogue=EPI_NONE, flags=0,
                 dims=(), fparams=(0.0, 0.0), sm_margin=0):
        if len(name.encode()) >= NAME_MAX:
            raise ValueError("kernel name too long")
        if len(dims) > 6:
            raise ValueError("at most 6 dims")
        self.name, self.op = name, op
        self.in_dtype, self.out_dtype = in_dtype, out_dtype
        self.epilogue, self.flags = epilogue, flags
        self.sm_margin = int(sm_margin)
        self.dims = tuple(int(d) for d in dims) + (0,) * (6 - len(dims))
        self.fparams = tuple(float(f) for f in fparams)
        self.payload = b""  # OP_LOOPNEST: the kernel's text; placed behind the table by pack_blob

    def pack(self):
        return _DESC.pack(self.name.encode(), self.op, self.in_dtype, self.out_dtype,
                          self.epilogue, self.flags, self.sm_margin, *self.dims, *self.fparams)


def pack_blob(descs):
    """bytes of a blob holding `descs` (list of KernelDesc): header, descriptor table, then
    the payloads (kernel text of OP_LOOPNEST descriptors, addressed by offset and length
    in dims[1], dims[2])."""
    table_end = _HEADER.size + len(descs) * _DESC.size
    payload = b""
    for d in descs:
        if d.payload:
            d.dims = (d.dims[0], table_end + len(payload), len(d.payload)) + tuple(d.dims[3:])
            payload += d.payload
    return _HEADER.pack(MAGIC, VERSION, len(descs)) + b"".join(d.pack() for d in descs) + payload


def unpack_blob(data):
    magic, version, n = _HEADER.unpack_from(data, 0)
    if magic != MAGIC:
        raise ValueError("bad blob magic")
    out = []
    for i in range(n):
        f = _DESC.unpack_from(data, _HEADER.size + i * _DESC.size)
        out.append(KernelDesc(f[0].split(b"\0")[0].decode(), f[1], f[2], f[3], f[4], f[5],
                              f[7:13], f[13:15], sm_margin=f[6]))
    return version, out


def gemm(name, M, N, K, in_dtype=BF16, epilogue=EPI_NONE, accumulate=False, bias=False,
         lda=0, ldb=0, ldc=0, sm_margin=0, trans_a=False, trans_b=False, out_dtype=F32):
    """lda/ldb/ldc: row pitches of the arrays as stored, in elements (0 = dense);
    sm_margin: SMs the persistent kernel leaves free (for a collective running
    beside it); trans_a: A is stored [K,M]; trans_b: B is stored [N,K]; out_dtype
    BF16/F16: f32 accumulation, one rounding at the end."""
    flags = ((FLAG_ACCUMULATE if accumulate else 0) | (FLAG_BIAS if bias else 0)
             | (FLAG_TRANS_A if trans_a else 0) | (FLAG_TRANS_B if trans_b else 0))
    return KernelDesc(name, OP_GEMM, in_dtype, out_dtype, epilogue, flags, (M, N, K, lda, ldb, ldc),
                      sm_margin=sm_margin)


# postfix code of OP_EXPR (ImexExprCode)
X_END, X_IN, X_ROWV, X_COLV, X_C0, X_C1, X_ZERO, X_ONE = 0, 1, 5, 9, 13, 14, 15, 16
X_UNARY = {"neg": 32, "abs": 33, "log": 34, "exp": 35, "sqrt": 36, "rsqrt": 37, "tanh": 38, "relu": 39}
X_BINARY = {"add": 64, "sub": 65, "mul": 66, "div": 67, "max": 68, "min": 69}
EXPR_MAX_CODE = 32


def assemble_expr(text):
    """Postfix text -> code bytes.  Tokens: in0..in3 (full tensors), row0..row3 (row
    vectors [cols]), col0..col3 (column vectors [rows]), c0, c1 (fparams), zero, one,
    and the operation names of X_UNARY / X_BINARY.  "in0 log in1 abs add in0 sub" is
    (log(x0) + |x1|) - x0."""
    code = []
    for tok in text.split():
        if tok[:-1] in ("in", "row", "col") and tok[-1].isdigit() and int(tok[-1]) < 4:
            code.append({"in": X_IN, "row": X_ROWV, "col": X_COLV}[tok[:-1]] + int(tok[-1]))
        elif tok in ("c0", "c1", "zero", "one"):
            code.append({"c0": X_C0, "c1": X_C1, "zero": X_ZERO, "one": X_ONE}[tok])
        elif tok in X_UNARY:
            code.append(X_UNARY[tok])
        elif tok in X_BINARY:
            code.append(X_BINARY[tok])
        else:
            raise ValueError("unknown token %r in expression" % tok)
    if not 0 < len(code) <= EXPR_MAX_CODE:
        raise ValueError("expression programs hold 1..%d operations" % EXPR_MAX_CODE)
    return bytes(code)


def expr(name, rows, cols, program, dtype=F32, out_dtype=None, reduce_leading=False,
         accumulate=False, consts=(0.0, 0.0)):
    """Fused elementwise chain: pointers = the inputs in order, then Y.  `program` is
    postfix text (assemble_expr) or code bytes."""
    code = assemble_expr(program) if isinstance(program, str) else bytes(program)
    words = struct.unpack("<4q", code.ljust(EXPR_MAX_CODE, b"\0"))
    flags = (FLAG_REDUCE_LEADING if reduce_leading else 0) | (FLAG_ACCUMULATE if accumulate else 0)
    return KernelDesc(name, OP_EXPR, dtype, dtype if out_dtype is None else out_dtype, 0, flags,
                      (rows, cols) + words, fparams=consts)


def loopnest(name, source, threads, n_pointers):
    """A loop-nest kernel given as CUDA C++ text: one `extern "C" __global__ void
    imex_loopnest(pointers...)` written against the runtime's loop-nest prelude (element-type
    helpers, IMX_THREAD_INDEX); compiled for sm_100a at first launch and run over `threads`
    points.  Pointers = the kernel's arguments in order."""
    d = KernelDesc(name, OP_LOOPNEST, 0, 0, 0, 0, (threads, 0, 0, n_pointers))
    d.payload = source.encode() if isinstance(source, str) else bytes(source)
    return d


def attention_fwd(name, heads, n_ctx, d_head=64, dtype=F16, sm_scale=0.5):
    """Pointers Q, K, V, O: [heads * n_ctx, d_head] arrays of dtype, heads one after the other."""
    return KernelDesc(name, OP_ATTENTION_FWD, dtype, dtype, 0, 0, (heads, n_ctx, d_head),
                      fparams=(sm_scale, 0.0))


def softmax(name, rows, cols, neg_inf_init=False, dtype=F32):
    """dtype F16 / BF16: every operation of the chain rounds to the element type."""
    return KernelDesc(name, OP_SOFTMAX, dtype, dtype, 0, FLAG_SOFTMAX_NEG_INF if neg_inf_init else 0,
                      (rows, cols))


def reduce_rows(name, rows, cols, accumulate=False):
    return KernelDesc(name, OP_REDUCE_ROWS, F32, F32, 0, FLAG_ACCUMULATE if accumulate else 0,
                      (rows, cols))


def reduce_leading(name, lead, inner, accumulate=False):
    return KernelDesc(name, OP_REDUCE_LEADING, F32, F32, 0, FLAG_ACCUMULATE if accumulate else 0,
                      (lead, inner))


def reduce_all(name, n, accumulate=False):
    return KernelDesc(name, OP_REDUCE_ALL, F32, F32, 0, FLAG_ACCUMULATE if accumulate else 0, (n,))


def transpose2d(name, rows, cols, dtype=F32):
    return KernelDesc(name, OP_TRANSPOSE2D, dtype, dtype, 0, 0, (rows, cols))


def transpose3d(name, dims, perm, dtype=F32):
    return KernelDesc(name, OP_TRANSPOSE3D, dtype, dtype, 0, 0, tuple(dims) + tuple(perm))


def eltwise(name, n, epilogue):
    return KernelDesc(name, OP_ELTWISE, F32, F32, epilogue, 0, (n,))


def convert(name, n, in_dtype, out_dtype):
    """arith.extf / arith.truncf between f32 and bf16 / f16."""
    return KernelDesc(name, OP_ELTWISE, in_dtype, out_dtype, EPI_NONE, 0, (n,))


def fill_uniform(name, n, dtype, seed, lo, hi, first=0):
    return KernelDesc(name, OP_FILL_UNIFORM, dtype, dtype, 0, 0, (n, seed, first), (lo, hi))


def fill_normal(name, n, dtype, seed, mean, stddev, first=0):
    return KernelDesc(name, OP_FILL_NORMAL, dtype, dtype, 0, 0, (n, seed, first), (mean, stddev))


_KEEP = []


class Blob:
    """Owns the bytes at a fixed address for the life of the process.

    gpuModuleLoad caches parsed modules by blob ADDRESS until exit (in the
    reference the blob is a global constant of the compiled host module), so a
    blob must never be freed and its address reused for other contents."""

    def __init__(self, descs):
        _KEEP.append(self)
        self.descs = list(descs)
        data = pack_blob(self.descs)
        self.buffer = C.create_string_buffer(data, len(data))
        self.size = len(data)

    @property
    def address(self):
        return C.addressof(self.buffer)
