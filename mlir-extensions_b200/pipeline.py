"""Host-buffer GEMM with the copies overlapped, through the C ABI only.

The reference's lowered host code copies inputs in, launches, waits and copies
the result out, one after the other (lib/Transforms/InsertGPUAllocs.cpp:437-469,
lib/Conversion/GPUXToLLVM/GPUXToLLVMPass.cpp:691-707); gpuMemCopy blocks, as in
both reference back-ends.  For operands that start and end in host memory that
order leaves the GPU idle during the transfers and the PCIe link idle in one
direction at a time.  Here the rows of A are cut into chunks and three host
threads and the B loader, each with its own stream handle, run a pipeline:

    B loader    gpuMemCopy(B) — or, when the ranks of a node share the upload of B
                (b_gather): gpuMemCopy(this rank's rows of B), then the other rows
                from the peers over NVLink                            host -> device
    uploader    gpuMemCopy(A chunk i)                                 host -> device
    launcher    gpuLaunchKernel(GEMM on chunk i); gpuWait
    downloader  gpuMemCopy(C chunk i)                                device -> host

A chunk is handed from one thread to the next only after the blocking call that
produced it has returned, so no cross-stream events are needed.  Uploads of
chunk i+1 and downloads of chunk i-1 overlap the GEMM of chunk i and each other
(PCIe is full duplex).
"""
import queue
import threading

from . import blob as B
from . import runtime as rt


class HostPipelinedGemm:
    """C_host[rows, n] = epilogue(A_host[rows, k] . B_host[k, n]) for host arrays given by address."""

    def __init__(self, device, rows, n, k, in_dtype=B.BF16, epilogue=B.EPI_NONE, chunks=8, b_gather=None):
        """b_gather: None, or a dist.PeerAllGather over B's k rows of n elements shared by the
        ranks of the node: this process then uploads only its own block of rows of B and
        fetches the other blocks from the ranks that uploaded them (NVLink, copy engines)."""
        import ctypes as C
        self._dev = C.c_int32(int(device))
        self.rows, self.n, self.k = rows, n, k
        self.esz = B.DTYPE_BYTES[in_dtype]
        chunks = max(1, min(chunks, rows))
        self.bounds = [(rows * i // chunks, rows * (i + 1) // chunks) for i in range(chunks)]
        dev = C.addressof(self._dev)
        self.s_up = rt.gpuCreateStream(dev, None)
        self.s_b = rt.gpuCreateStream(dev, None)
        self.s_run = rt.gpuCreateStream(dev, None)
        self.s_down = rt.gpuCreateStream(dev, None)
        self.b_gather = b_gather
        self.dA = rt.gpuMemAlloc(self.s_run, rows * k * self.esz, 64, False)
        self.dB = b_gather.array if b_gather is not None else rt.gpuMemAlloc(self.s_run, k * n * self.esz, 64, False)
        self.dC = rt.gpuMemAlloc(self.s_run, rows * n * 4, 64, False)
        self.kernels = []
        self._blobs = []
        for i, (r0, r1) in enumerate(self.bounds):
            desc = B.gemm(f"host_pipelined_gemm_{i}", r1 - r0, n, k, in_dtype, epilogue)
            blob = B.Blob([desc])
            self._blobs.append(blob)
            mod = rt.gpuModuleLoad(self.s_run, blob.address, blob.size)
            self.kernels.append(rt.gpuKernelGet(self.s_run, mod, desc.name.encode()))

    def __call__(self, a_host_ptr, b_host_ptr, c_host_ptr):
        """Runs one GEMM; returns when C is complete in host memory."""
        uploaded, computed = queue.Queue(), queue.Queue()
        errors = []

        def guard(fn):
            def run():
                try:
                    fn()
                except BaseException as e:  # noqa: BLE001 - surfaced to the caller below
                    errors.append(e)
                    uploaded.put(None)
                    computed.put(None)
            return run

        b_ready = threading.Event()

        def upload_b():
            if self.b_gather is None:
                rt.gpuMemCopy(self.s_b, self.dB, b_host_ptr, self.k * self.n * self.esz)
            else:  # this rank's rows of B from the host, the rest from the peers
                off, nbytes = self.b_gather.own_block()
                if nbytes:
                    rt.gpuMemCopy(self.s_b, self.dB + off, b_host_ptr + off, nbytes)
                self.b_gather.exchange(self.s_b)
                rt.gpuWait(self.s_b)
            b_ready.set()

        def upload():
            for i, (r0, r1) in enumerate(self.bounds):
                off = r0 * self.k * self.esz
                rt.gpuMemCopy(self.s_up, self.dA + off, a_host_ptr + off, (r1 - r0) * self.k * self.esz)
                uploaded.put(i)
            uploaded.put(None)

        def launch():
            while True:
                i = uploaded.get()
                if i is None:
                    break
                while not b_ready.wait(0.05) and not errors:  # B travels beside the first chunks of A
                    pass
                if errors:
                    break
                r0, _ = self.bounds[i]
                rt.gpuLaunchKernel(self.s_run, self.kernels[i], (1, 1, 1), (1, 1, 1), 0,
                                   [self.dA + r0 * self.k * self.esz, self.dB, self.dC + r0 * self.n * 4])
                rt.gpuWait(self.s_run)
                computed.put(i)
            computed.put(None)

        def download():
            while True:
                i = computed.get()
                if i is None:
                    break
                r0, r1 = self.bounds[i]
                off = r0 * self.n * 4
                rt.gpuMemCopy(self.s_down, c_host_ptr + off, self.dC + off, (r1 - r0) * self.n * 4)

        threads = [threading.Thread(target=guard(f)) for f in (upload_b, upload, launch, download)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if errors:
            raise errors[0]

    def close(self):
        for p in (self.dA, self.dC) + (() if self.b_gather is not None else (self.dB,)):
            rt.gpuMemFree(self.s_run, p)
        for s in (self.s_up, self.s_b, self.s_run, self.s_down):
            rt.gpuStreamDestroy(s)
