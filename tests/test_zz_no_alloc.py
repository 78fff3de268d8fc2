"""imexReduceAllF32Static: the full-sum entry point for callers that cannot let
the library allocate (hosts that own all device memory, loops that cannot take
cudaMalloc's synchronisation).  Its scratch is an array inside the library, so
the checks here are: same answer as the regular gpuLaunchKernel path, twice in
a row with different sizes (the array keeps the first call's partials), and a
clean refusal beyond the built-in limit.  Collected last on purpose."""
import ctypes as C

import numpy as np
import pytest

from __graft_entry__ import load_package
from oracle import oracle

pytestmark = pytest.mark.gpu

TOL = 1e-5  # the tolerance of the other sum-reduction tests


def _static_entry(pkg):
    fn = pkg.runtime.library().imexReduceAllF32Static
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p]
    return fn


def test_static_scratch_sum_matches_regular_path_twice_in_a_row():
    pkg = load_package()
    rt, B = pkg.runtime, pkg.blob
    fn = _static_entry(pkg)
    with pkg.Session(device=0) as s:
        stream = rt.imexStreamNative(s.stream)
        # second call is smaller than the first: partials left over from call 1 must not leak in
        for n, acc, seed in ((3_000_017, False, 1), (40_001, True, 2)):
            X = np.random.default_rng(seed).uniform(0, 1, n).astype(np.float32)
            init = np.array([1.25], np.float32)
            dX = s.upload(X)
            d_ref, d_new = s.upload(init), s.upload(init)
            s.run(B.reduce_all("sum", n, accumulate=acc), [dX, d_ref])      # existing entry point
            assert fn(dX, d_new, n, int(acc), stream) == 0                   # the one under test
            s.wait()
            ref = s.download(d_ref, (1,), np.float32)[0]
            new = s.download(d_new, (1,), np.float32)[0]
            assert abs(float(new) - float(ref)) <= TOL * abs(float(ref))
            truth = X.astype(np.float64).sum() + (1.25 if acc else 0.0)
            assert abs(float(new) - truth) <= TOL * truth
            assert abs(float(new) - float(oracle.reduce_all(X, 1.25 if acc else 0.0))) <= 4 * TOL * truth
        # n = 0: the sum of nothing
        d0 = s.upload(np.array([7.0], np.float32))
        assert fn(None, d0, 0, 1, stream) == 0
        s.wait()
        assert s.download(d0, (1,), np.float32)[0] == 7.0


def test_static_scratch_refuses_sizes_beyond_its_array(capfd):
    pkg = load_package()
    fn = _static_entry(pkg)
    with pkg.Session(device=0) as s:
        y = s.upload(np.array([3.0], np.float32))
        x = s.alloc(16)
        too_many = 65536 * 16384 + 1
        assert fn(x, y, too_many, 0, None) == 2     # refused before anything is launched
        assert fn(x, None, 4, 0, None) == 1
        s.wait()
        assert s.download(y, (1,), np.float32)[0] == 3.0
    err = capfd.readouterr().err
    assert "block partials" in err and "invalid argument" in err
