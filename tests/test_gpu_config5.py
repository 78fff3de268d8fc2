"""The headline workload (BASELINE config 5) as a test: bf16 A[65536,8192] . B[8192,8192] -> f32 C
with the fused silu, inputs N(0, 0.02) from seeds 7 and 8, on one GPU at full shape; and the
launch plans the row-sharded modes cut one rank's GEMM into, against one plain launch."""
import numpy as np
import pytest

from __graft_entry__ import load_package
from oracle import oracle

pytestmark = pytest.mark.gpu
N, K = 8192, 8192


@pytest.fixture(scope="module")
def pkg():
    return load_package()


def _fill(pkg, sess, rows, row0=0):
    B = pkg.blob
    dA, dB = sess.alloc(rows * K * 2), sess.alloc(K * N * 2)
    sess.run(B.fill_normal("a", rows * K, B.BF16, 7, 0.0, 0.02, first=row0 * K), [dA])
    sess.run(B.fill_normal("b", K * N, B.BF16, 8, 0.0, 0.02), [dB])
    return dA, dB


def _rows(pkg, sess, base, rows, width, dtype):
    """Selected rows of a device array [*, width] of dtype."""
    rt = pkg.runtime
    out = np.empty((len(rows), width), dtype)
    step = width * out.itemsize
    for i, r in enumerate(rows):
        rt.gpuMemCopy(sess.stream, out[i].ctypes.data, base + int(r) * step, step)
    return out


def test_config5_full_shape_sampled_rows_against_the_oracle(pkg):
    B = pkg.blob
    M = 65536
    with pkg.Session(device=0) as s:
        dA, dB = _fill(pkg, s, M)
        dC = s.alloc(M * N * 4)
        s.run(B.gemm("config5", M, N, K, B.BF16, B.EPI_SILU), [dA, dB, dC])
        assert s.last_kernel() == "gemm_tcgen05_2cta"
        rng = np.random.default_rng(5)
        # first and last row, the last 256-row block (where a k-split tail would land), random rows
        rows = sorted({0, M - 1, *range(M - 256, M, 37), *rng.choice(M, 256, replace=False).tolist()})
        assert len(rows) >= 256
        a = _rows(pkg, s, dA, rows, K, np.uint16)
        b = s.download(dB, (K, N), np.uint16)
        got = _rows(pkg, s, dC, rows, N, np.float32)
    ref = oracle.silu(oracle.matmul_x16_f32(a, b, True))
    assert np.isfinite(got).all()
    assert oracle.rel_frobenius(got, ref) <= 1e-3            # the tolerance the task states; measured ~1e-5
    assert np.abs(got - ref).max() <= 1e-4 * np.abs(ref).max()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("no_splitk", [True, False])
def test_row_sharded_launch_plans_equal_one_launch(pkg, monkeypatch, world, no_splitk):
    """One rank's rows of config 5, cut the way overlap="calls" (two column ranges, the first
    leaving 32 SMs free) and overlap="slabs" (column slabs, 8 SMs free) cut them, against ONE
    launch on all SMs (what overlap="ce" runs).  Without the k-split tail every element is one
    ascending-k chain whatever the launch: bit for bit.  With it (default) a split tile sums its
    parts in another order: equal to 1e-5 of the largest value."""
    from mlir_extensions_b200 import dist
    B = pkg.blob
    if no_splitk:
        monkeypatch.setenv("IMEX_GEMM_NO_SPLITK", "1")
    else:
        monkeypatch.delenv("IMEX_GEMM_NO_SPLITK", raising=False)
    rows = 65536 // world
    row0 = (world - 1) * rows                                   # the last rank's block
    with pkg.Session(device=0) as s:
        dA, dB = _fill(pkg, s, rows, row0)
        dC1, dC2 = s.alloc(rows * N * 4), s.alloc(rows * N * 4)
        s.run(B.gemm("whole", rows, N, K, B.BF16, B.EPI_SILU), [dA, dB, dC1])
        one = s.download(dC1, (rows, N), np.float32)
        plans = {"calls": [(c0, w, m) for (c0, w), m in zip(
                     [(0, dist.plan_two_parts(rows, N, K)[0]), (dist.plan_two_parts(rows, N, K)[0],
                                                                dist.plan_two_parts(rows, N, K)[1])], (32, 0)) if w],
                 "slabs": [(c0, w, 8) for c0, w in dist.plan_slabs(rows, N, world, sm_margin=8)]}
        for name, launches in plans.items():
            assert sum(w for _, w, _ in launches) == N
            rt = pkg.runtime
            poison = np.full(1 << 20, np.nan, np.float32)
            for off in range(0, rows * N * 4, poison.nbytes):      # every element must be written
                rt.gpuMemCopy(s.stream, dC2 + off, poison.ctypes.data, min(poison.nbytes, rows * N * 4 - off))
            for j, (c0, w, margin) in enumerate(launches):
                desc = B.gemm("%s_%d" % (name, j), rows, w, K, B.BF16, B.EPI_SILU, ldb=N, ldc=N, sm_margin=margin)
                s.run(desc, [dA, dB + 2 * c0, dC2 + 4 * c0])
            cut = s.download(dC2, (rows, N), np.float32)
            if no_splitk:
                assert cut.tobytes() == one.tobytes(), name
            else:
                assert np.abs(cut - one).max() <= 1e-5 * np.abs(one).max(), name
