"""A small host-side driver that issues exactly the call sequence the
reference's lowered host code issues per gpu.launch_func
(lib/Conversion/GPUXToLLVM/GPUXToLLVMPass.cpp:456-713):

    gpuCreateStream -> gpuMemAlloc -> gpuMemCopy(in) -> gpuModuleLoad(blob) ->
    gpuKernelGet(name) -> gpuLaunchKernel(bare pointers) -> gpuWait ->
    gpuMemCopy(out) -> gpuMemFree -> gpuStreamDestroy

Tests and bench.py use it so that everything they measure goes through the
C ABI."""
import ctypes as C

import numpy as np

from . import blob as B
from . import runtime as rt

_NP_TO_DTYPE = {np.dtype(np.float32): B.F32, np.dtype(np.int32): B.I32}


class Session:
    def __init__(self, device=None, adopt_stream=None):
        dev = None
        if device is not None:
            self._dev = C.c_int32(int(device))
            dev = C.addressof(self._dev)
        self.stream = rt.gpuCreateStream(dev, adopt_stream)
        self._blobs = []
        self._allocs = []

    # ---- memory -------------------------------------------------------------
    def alloc(self, nbytes, shared=False):
        p = rt.gpuMemAlloc(self.stream, int(nbytes), 64, bool(shared))
        self._allocs.append(p)
        return p

    def free(self, ptr):
        self._allocs.remove(ptr)
        rt.gpuMemFree(self.stream, ptr)

    def upload(self, array, shared=False):
        a = np.ascontiguousarray(array)
        p = self.alloc(a.nbytes, shared)
        if a.nbytes:
            rt.gpuMemCopy(self.stream, p, a.ctypes.data, a.nbytes)
        return p

    def download(self, ptr, shape, dtype):
        out = np.empty(shape, dtype)
        if out.nbytes:
            rt.gpuMemCopy(self.stream, out.ctypes.data, ptr, out.nbytes)
        return out

    # ---- kernels ------------------------------------------------------------
    def kernel(self, desc):
        """Module with one descriptor -> kernel handle."""
        blob = B.Blob([desc])
        self._blobs.append(blob)  # the module cache is keyed by this address
        mod = rt.gpuModuleLoad(self.stream, blob.address, blob.size)
        return rt.gpuKernelGet(self.stream, mod, desc.name.encode())

    def launch(self, kernel, pointer_args, wait=True, deps=()):
        # grid/block: what the reference's one-work-item-per-element lowering
        # would pass; the runtime picks its own geometry
        ev = rt.gpuLaunchKernel(self.stream, kernel, (1, 1, 1), (1, 1, 1), 0, pointer_args, deps)
        if wait:
            rt.gpuWait(self.stream)
        return ev

    def wait(self):
        rt.gpuWait(self.stream)

    def run(self, desc, pointer_args):
        self.launch(self.kernel(desc), pointer_args)

    def last_kernel(self):
        return rt.last_kernel_name(self.stream)

    def close(self):
        for p in list(self._allocs):
            rt.gpuMemFree(self.stream, p)
        self._allocs.clear()
        if self.stream:
            rt.gpuStreamDestroy(self.stream)
            self.stream = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
