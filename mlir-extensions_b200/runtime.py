"""Host-side mirror of the reference's GPU runtime-wrapper interface.

The functions keep the reference's names and argument meaning
(lib/ExecutionEngine/LEVELZERORUNTIME/LevelZeroRuntimeWrappers.cpp:606-671):
gpuCreateStream, gpuMemAlloc, gpuMemCopy, gpuModuleLoad, gpuKernelGet,
gpuLaunchKernel, gpuWait, ... and are thin ctypes calls into
lib/libimex_cuda_runtime.so.  There is no fallback: if the library is missing
the import raises."""
import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "lib", "libimex_cuda_runtime.so")


class ParamDesc(C.Structure):
    _fields_ = [("data", C.c_void_p), ("size", C.c_size_t)]


class EventDesc(C.Structure):
    _fields_ = [("event", C.c_void_p)]


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: run `python mlir-extensions_b200/build.py` (needs nvcc). "
            "This package has no CPU or PyTorch fallback.")
    lib = C.CDLL(LIB_PATH)
    vp, sz = C.c_void_p, C.c_size_t
    sig = {
        "gpuCreateStream": (vp, [vp, vp]),
        "gpuStreamDestroy": (None, [vp]),
        "gpuMemAlloc": (vp, [vp, sz, sz, C.c_bool]),
        "gpuMemFree": (None, [vp, vp]),
        "gpuMemCopy": (None, [vp, vp, vp, sz]),
        "gpuMemcpy": (None, [vp, vp, vp, sz]),
        "gpuModuleLoad": (vp, [vp, vp, sz]),
        "gpuKernelGet": (vp, [vp, vp, C.c_char_p]),
        "gpuLaunchKernel": (vp, [vp, vp, sz, sz, sz, sz, sz, sz, sz, vp, vp]),
        "gpuWait": (None, [vp]),
        "gpuModuleUnload": (None, [vp]),
        "mgpuStreamCreate": (vp, []),
        "mgpuStreamSynchronize": (None, [vp]),
        "mgpuStreamDestroy": (None, [vp]),
        "mgpuMemAlloc": (vp, [sz, vp, C.c_bool]),
        "mgpuMemFree": (None, [vp, vp]),
        "mgpuModuleLoad": (vp, [vp, sz]),
        "mgpuModuleGetFunction": (vp, [vp, C.c_char_p]),
        "mgpuModuleUnload": (None, [vp]),
        "mgpuLaunchKernel": (None, [vp, sz, sz, sz, sz, sz, sz, sz, vp, C.POINTER(vp),
                                    C.POINTER(vp), sz]),
        "imexStreamNative": (vp, [vp]),
        "imexEventRecord": (vp, [vp]),
        "imexEventElapsedMs": (C.c_float, [vp, vp]),
        "imexLaunchCount": (C.c_uint64, []),
        "imexLastKernelName": (C.c_char_p, [vp]),
        "imexShardSize": (C.c_int64, [C.c_int64, C.c_int64, C.c_int64]),
        "imexShardOffset": (C.c_int64, [C.c_int64, C.c_int64, C.c_int64]),
        "imexStat": (C.c_float, [C.c_int, C.POINTER(C.c_float), sz]),
        "imexSelfTestWaitTimeout": (None, [vp]),
        "imexStreamStatusWord": (vp, [vp]),
        "imexNoteLaunches": (None, [C.c_uint64]),
        "imexIpcExport": (C.c_int, [vp, vp]),
        "imexIpcOpen": (vp, [vp]),
        "imexIpcClose": (None, [vp]),
        "imexMemCopyAsync": (None, [vp, vp, vp, sz]),
        "imexPeerBarrier": (None, [vp, C.POINTER(vp), C.c_int, C.c_int, C.c_uint32]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib, sorted(sig)


_lib, EXPORTS = _load()

gpuCreateStream = _lib.gpuCreateStream
gpuStreamDestroy = _lib.gpuStreamDestroy
gpuMemAlloc = _lib.gpuMemAlloc
gpuMemFree = _lib.gpuMemFree
gpuMemCopy = _lib.gpuMemCopy
gpuModuleLoad = _lib.gpuModuleLoad
gpuKernelGet = _lib.gpuKernelGet
gpuWait = _lib.gpuWait
imexStreamNative = _lib.imexStreamNative
imexEventRecord = _lib.imexEventRecord
imexEventElapsedMs = _lib.imexEventElapsedMs
imexLaunchCount = _lib.imexLaunchCount
imexShardSize = _lib.imexShardSize
imexShardOffset = _lib.imexShardOffset


def library():
    return _lib


def make_params(values):
    """ParamDesc array the way the lowered host code builds it
    (lib/Conversion/GPUXToLLVM/GPUXToLLVMPass.cpp:540-623): each entry points
    at a slot holding the value, {NULL,0} terminates.  Returns (array, keepalive)."""
    slots = (C.c_void_p * max(len(values), 1))(*[C.c_void_p(int(v)) for v in values])
    arr = (ParamDesc * (len(values) + 1))()
    for i in range(len(values)):
        arr[i].data = C.addressof(slots) + i * C.sizeof(C.c_void_p)
        arr[i].size = C.sizeof(C.c_void_p)
    arr[len(values)].data = None
    arr[len(values)].size = 0
    return arr, slots


_NO_EVENTS = (EventDesc * 1)()


def gpuLaunchKernel(stream, kernel, grid, block, shared_mem_bytes, pointer_args, dep_events=()):
    """gpuLaunchKernel with the argument lists built from Python sequences."""
    params, keep = make_params(pointer_args)
    if dep_events:
        deps = (EventDesc * (len(dep_events) + 1))()
        for i, e in enumerate(dep_events):
            deps[i].event = e
    else:
        deps = _NO_EVENTS
    gx, gy, gz = grid
    bx, by, bz = block
    ev = _lib.gpuLaunchKernel(stream, kernel, gx, gy, gz, bx, by, bz, shared_mem_bytes,
                              C.cast(params, C.c_void_p), C.cast(deps, C.c_void_p))
    del keep
    return ev


def last_kernel_name(stream):
    return _lib.imexLastKernelName(stream).decode()


def stat(which, values):
    arr = (C.c_float * len(values))(*values)
    return float(_lib.imexStat(which, arr, len(values)))
