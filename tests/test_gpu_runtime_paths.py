"""Runtime paths of the C ABI that the parity tests do not reach: the profiling loop, the
upstream-style `mgpu*` launch sequence, the event ring, kernel-handle reuse and scalar
parameters standing between memrefs.  Everything goes through libimex_cuda_runtime.so and
is checked against the CPU oracle."""
import ctypes as C
import os
import re
import subprocess
import sys

import numpy as np
import pytest

from __graft_entry__ import load_package
from oracle import oracle

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def pkg():
    return load_package()


def _child(code, env=None):
    prog = ("import sys, numpy as np; sys.path.insert(0, %r)\n"
            "from __graft_entry__ import load_package\npkg = load_package(); rt, B = pkg.runtime, pkg.blob\n"
            % ROOT) + code
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run([sys.executable, "-c", prog], capture_output=True, text=True, env=e)


# the line of lib/ExecutionEngine/LEVELZERORUNTIME/LevelZeroRuntimeWrappers.cpp:587-596, with
# "CUDA" where the reference names its own runtime
_NUM = r"-?\d+\.\d+"
PROFILE_LINE = re.compile(
    r"^the kernel execution time is \(ms, on CUDA runtime\):avg: (%s), min: (%s), max: (%s), "
    r"median: (%s), std_deviation: (%s), variance: (%s), P95: (%s), P5: (%s), "
    r"median_one_third_avg: (%s) \(over (\d+) runs\)$" % ((_NUM,) * 9), re.M)


@pytest.mark.parametrize("flush", [True, False])
def test_profiling_loop_prints_the_reference_statistics_line(flush):
    """IMEX_ENABLE_PROFILING repeats the launch (warm-ups, then IMEX_PROFILING_RUNS timed
    runs, the last-level cache overwritten before each when IMEX_ENABLE_CACHE_FLUSHING is
    set), prints one statistics line and then launches once more for the result."""
    env = {"IMEX_ENABLE_PROFILING": "1", "IMEX_PROFILING_RUNS": "5", "IMEX_PROFILING_WARMUPS": "2"}
    if flush:
        env["IMEX_ENABLE_CACHE_FLUSHING"] = "1"
    r = _child("s = pkg.Session(device=0)\n"
               "x = np.random.default_rng(0).normal(0, 3, (256, 1024)).astype(np.float32)\n"
               "dx, dy = s.upload(x), s.alloc(x.nbytes)\n"
               "before = rt.imexLaunchCount()\n"
               "s.run(B.softmax('sm', 256, 1024), [dx, dy])\n"
               "print('launches', rt.imexLaunchCount() - before)\n"
               "y = s.download(dy, x.shape, np.float32)\n"
               "print('rowsum', float(abs(y.sum(axis=1) - 1).max()))\n", env)
    assert r.returncode == 0, r.stdout + r.stderr
    m = PROFILE_LINE.search(r.stdout)
    assert m, r.stdout
    avg, mn, mx, med, sd, var, p95, p5, mid, runs = [float(g) for g in m.groups()]
    eps = 1e-4  # avg / min / max are printed with four decimals, the others with six
    assert runs == 5 and 0 < mn <= med + eps and med <= mx + eps and mn <= avg + eps and avg <= mx + eps
    assert p5 <= p95 + eps
    assert abs(var - sd * sd) <= 1e-4 + 0.02 * var
    assert "launches 8" in r.stdout          # 2 warm-ups + 5 timed + the launch itself
    assert float(re.search(r"rowsum (\S+)", r.stdout).group(1)) < 1e-5


def test_upstream_style_mgpu_sequence_runs_a_kernel(pkg):
    """mgpuStreamCreate -> mgpuMemAlloc -> mgpuModuleLoad -> mgpuModuleGetFunction ->
    mgpuLaunchKernel(void **params) -> mgpuStreamSynchronize, the sequence upstream's
    gpu-to-llvm host code issues (LevelZeroRuntimeWrappers.cpp:673-741)."""
    rt, B = pkg.runtime, pkg.blob
    lib = rt.library()
    stream = lib.mgpuStreamCreate()
    X = oracle.fill_uniform((96, 640), 11, -1.0, 1.0)
    dx = lib.mgpuMemAlloc(X.nbytes, stream, False)
    dy = lib.mgpuMemAlloc(X.nbytes, None, False)     # null stream: the thread's default queue
    rt.gpuMemCopy(stream, dx, X.ctypes.data, X.nbytes)
    blob = B.Blob([B.transpose2d("mgpu_transpose", 96, 640)])
    mod = lib.mgpuModuleLoad(blob.address, blob.size)
    fn = lib.mgpuModuleGetFunction(mod, b"mgpu_transpose")
    assert fn == lib.mgpuModuleGetFunction(mod, b"mgpu_transpose")   # handles belong to the module
    slots = (C.c_void_p * 2)(dx, dy)
    params = (C.c_void_p * 2)(C.addressof(slots), C.addressof(slots) + 8)
    before = rt.imexLaunchCount()
    lib.mgpuLaunchKernel(fn, 1, 1, 1, 1, 1, 1, 0, stream, params, None, 2)
    lib.mgpuStreamSynchronize(stream)
    assert rt.imexLaunchCount() - before == 1
    out = np.empty((640, 96), np.float32)
    rt.gpuMemCopy(stream, out.ctypes.data, dy, out.nbytes)
    assert np.array_equal(out, oracle.transpose2d(X))
    lib.mgpuModuleUnload(mod)
    lib.mgpuMemFree(stream, dx)
    lib.mgpuMemFree(stream, dy)
    lib.mgpuStreamDestroy(stream)


def test_index_scalars_between_memrefs_are_not_operands(pkg):
    """The lowering appends loop bounds as 8-byte index values; wherever they stand in the
    parameter list they must not displace the memref pointers."""
    rt, B = pkg.runtime, pkg.blob
    with pkg.Session(device=0) as s:
        X = oracle.fill_uniform((64, 512), 5, 0.0, 1.0)
        dx, dy = s.upload(X), s.upload(np.full(64, np.nan, np.float32))
        k = s.kernel(B.reduce_rows("r", 64, 512))
        s.launch(k, [64, dx, 512, 1, dy, 0])      # scalars before, between and after
        got = s.download(dy, (64,), np.float32)
        assert oracle.max_rel_err(got, oracle.reduce_rows(X)) <= 1e-5


def test_launch_events_come_from_a_ring_and_stay_usable(pkg):
    """More launches than the ring has slots: handles repeat after 256 launches, a recent
    handle still orders a dependent launch."""
    rt, B = pkg.runtime, pkg.blob
    with pkg.Session(device=0) as s:
        X = oracle.fill_uniform((8, 128), 3, -1.0, 1.0)
        dx, dy, dz = s.upload(X), s.alloc(X.nbytes), s.alloc(X.nbytes)
        relu = s.kernel(B.eltwise("relu", X.size, B.EPI_RELU))
        events = [s.launch(relu, [dx, dy], wait=False) for _ in range(300)]
        assert len(set(events)) == 256 and events[0] == events[256]
        s.launch(relu, [dy, dz], wait=False, deps=[events[-1]])
        s.wait()
        assert np.array_equal(s.download(dz, X.shape, np.float32), oracle.relu(X))


def test_launches_captured_into_a_cuda_graph_replay_with_the_same_results(pkg):
    """gpuLaunchKernel on a stream that is being captured: the launches become graph nodes (no
    event record between them; the softmax of a few rows per SM is launched with programmatic
    stream serialisation, the second launch reads what the first wrote), and a replay gives the
    bits of the direct launches.  A handle returned under capture may be passed as a dependency
    on the same stream."""
    import torch
    B = pkg.blob
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    stream = torch.cuda.Stream(device=dev)
    torch.cuda.set_stream(stream)
    sess = pkg.Session(device=0, adopt_stream=stream.cuda_stream)
    x = torch.empty((4096, 1024), dtype=torch.float32, device=dev).normal_(0.0, 3.0)
    y1, y2 = torch.empty_like(x), torch.empty_like(x)
    k = sess.kernel(B.softmax("sm", 4096, 1024))
    sess.launch(k, [x.data_ptr(), y1.data_ptr()], wait=False)   # everything lazy happens before the capture
    sess.launch(k, [y1.data_ptr(), y2.data_ptr()], wait=True)
    want1, want2 = y1.clone(), y2.clone()
    y1.zero_()
    y2.zero_()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        first = sess.launch(k, [x.data_ptr(), y1.data_ptr()], wait=False)
        sess.launch(k, [y1.data_ptr(), y2.data_ptr()], wait=False, deps=(first,))
    assert float(y2.abs().sum()) == 0.0          # captured, not run
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    assert torch.equal(y1, want1) and torch.equal(y2, want2)
    torch.cuda.set_stream(torch.cuda.default_stream(dev))
    sess.close()
