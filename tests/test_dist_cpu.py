"""Host side of the row-sharded path, on CPU: slab planning, and the pack +
broadcast of B's column slabs over a world_size-2 gloo group."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from __graft_entry__ import ROOT, load_package

load_package()
from mlir_extensions_b200 import dist as rows  # noqa: E402


@pytest.mark.parametrize("world,rows_per_rank", [(2, 32768), (4, 16384), (8, 8192), (3, 21846), (8, 100)])
def test_slab_plan_covers_b_in_whole_tiles(world, rows_per_rank):
    slabs = rows.plan_slabs(rows_per_rank, 8192, world)
    assert slabs[0][0] == 0 and sum(w for _, w in slabs) == 8192
    assert all(c % 256 == 0 and w % 256 == 0 and w > 0 for c, w in slabs)
    assert all(slabs[i][0] + slabs[i][1] == slabs[i + 1][0] for i in range(len(slabs) - 1))
    assert 1 < len(slabs) <= 8


def test_slab_plan_fills_whole_waves_for_the_benchmark_shapes():
    clusters = (148 - 4) // 2
    for world in (2, 4, 8):
        r = 65536 // world
        slabs = rows.plan_slabs(r, 8192, world)
        for _, w in slabs[1:]:  # all but the short first slab
            assert ((r // 256) * (w // 256)) % clusters == 0
    assert rows.plan_slabs(65536, 8192, 1) == [(0, 8192)]
    assert rows.plan_slabs(512, 200, 4) == [(0, 200)]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import sys
    sys.path.insert(0, ROOT)
    from __graft_entry__ import load_package
    load_package()
    from mlir_extensions_b200 import dist as rows
    dist.init_process_group("gloo", rank=rank, world_size=world)
    k, n, m_total = 64, 1024, 10
    g = torch.Generator().manual_seed(5)
    b_true = torch.randn((k, n), generator=g)
    b_full = b_true.clone() if rank == 0 else torch.full((k, n), float("nan"))
    slabs = [(0, 256), (256, 512), (768, 256)]
    bufs = [torch.empty((k, w)) for _, w in slabs]
    works = rows.replicate_slabs(b_full, bufs, slabs, src=0, is_src=rank == 0)
    a_all = torch.randn((m_total, k), generator=g)
    row0, nrows = rows.shard_rows(rank, world, m_total)
    c = torch.empty((nrows, n))
    for (c0, w), buf, work in zip(slabs, bufs, works):
        work.wait()
        c[:, c0:c0 + w] = a_all[row0:row0 + nrows] @ buf  # stands in for the GPU launch
    ok = torch.allclose(c, a_all[row0:row0 + nrows] @ b_true, atol=1e-5)
    gathered = [None] * world
    dist.all_gather_object(gathered, (row0, nrows, bool(ok)))
    if rank == 0:
        np.save(os.path.join(tmp, "result.npy"), np.array(gathered, dtype=np.int64))
    dist.destroy_process_group()


def test_world2_gloo_slab_replication(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    res = np.load(tmp_path / "result.npy")
    assert res[:, 2].all()                       # every rank reproduced its rows of A.B
    assert res[:, :2].tolist() == [[0, 5], [5, 5]]  # block rows of a 10-row A over 2 ranks


def _gather_worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import sys
    sys.path.insert(0, ROOT)
    from __graft_entry__ import load_package
    load_package()
    from mlir_extensions_b200 import dist as rows
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ok = True
    for extent in (10, 11, 1):  # even blocks, ragged blocks, a rank with no rows
        truth = torch.arange(extent * 3, dtype=torch.float32).reshape(extent, 3)
        row0, nrows = rows.shard_rows(rank, world, extent)
        full = torch.full((extent, 3), float("nan"))
        rows.all_gather_rows(truth[row0:row0 + nrows].clone(), full, rank, world, extent)
        ok = ok and bool(torch.equal(full, truth))
    gathered = [None] * world
    dist.all_gather_object(gathered, ok)
    if rank == 0:
        np.save(os.path.join(tmp, "gather.npy"), np.array(gathered, dtype=np.int64))
    dist.destroy_process_group()


def test_world2_gloo_all_gather_rows(tmp_path):
    world = 2
    mp.spawn(_gather_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert np.load(tmp_path / "gather.npy").all()


def test_overlap_across_calls_uses_one_full_width_slab():
    from mlir_extensions_b200 import dist as rows

    class _NoSession:
        def kernel(self, blob):
            return blob

    import pytest
    with pytest.raises(ValueError):
        rows.RowShardedGemm(_NoSession(), 0, 1, 512, 512, 64, overlap="sometimes")
    g = rows.RowShardedGemm(_NoSession(), 0, 1, 512, 512, 64, overlap="calls")
    assert g.slabs == [(0, 512)]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_two_part_plan_for_the_benchmark_gemm(world):
    """overlap="calls": the first launch (NCCL beside it) covers whole 256-column blocks and
    about half a millisecond of work, the second the rest of the width."""
    from mlir_extensions_b200 import dist as rows
    n = k = 8192
    w1, w2 = rows.plan_two_parts(65536 // world, n, k)
    assert w1 + w2 == n and w1 % 256 == 0 and w1 > 0 and w2 > 0
    est_ms = 2.0 * (65536 // world) * n * k / 1.4e12
    first_ms = est_ms * (w1 / n) * 148 / 116
    assert 0.4 <= first_ms <= 0.75
    # a GEMM shorter than the replication keeps one launch with the margin
    assert rows.plan_two_parts(1024, 8192, 1024) == (8192, 0)
    assert rows.plan_two_parts(4096, 512, 512) == (512, 0)


def test_copy_engine_replication_slices_cover_b_once():
    """Row slices of B for the copy-engine replication: one block per rank other than the source,
    by the reference's partition rule over world-1 parts; together they cover every row once."""
    from mlir_extensions_b200.dist import plan_peer_slices
    for world in (2, 3, 4, 8):
        for src in (0, world - 1):
            for rows in (8192, 1000, 7, 1):
                slices = plan_peer_slices(rows, world, src)
                assert sorted(slices) == [r for r in range(world) if r != src]
                covered = []
                for r in sorted(slices):
                    r0, nr = slices[r]
                    covered += list(range(r0, r0 + nr))
                assert covered == list(range(rows))
                sizes = [n for _, n in slices.values()]
                assert max(sizes) - min(sizes) <= 1
    assert plan_peer_slices(8192, 8, 0)[1] == (0, 1170) and plan_peer_slices(8192, 8, 0)[7] == (7021, 1171)


def _leaving_worker(rank, world, port, tmp):
    """Two steps of slab replication; rank 1 leaves between the steps (no collective of its in
    flight).  Rank 0 must come out of its next replication with an error within the group's
    timeout, not hang."""
    import datetime
    import sys
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    sys.path.insert(0, ROOT)
    from __graft_entry__ import load_package
    load_package()
    from mlir_extensions_b200 import dist as rows
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    k, n = 16, 512
    b_full = torch.ones((k, n)) if rank == 0 else torch.zeros((k, n))
    slabs = [(0, 256), (256, 256)]
    bufs = [torch.empty((k, w)) for _, w in slabs]
    for w in rows.replicate_slabs(b_full, bufs, slabs, src=0, is_src=rank == 0):
        w.wait()
    step1_ok = all(bool((b == 1).all()) for b in bufs)
    if rank == 1:
        with open(os.path.join(tmp, "rank1.txt"), "w") as f:
            f.write("left after step 1, step1_ok=%s" % step1_ok)
        os._exit(0)  # between steps: nothing of this rank is in flight
    t0 = time.time()
    outcome = "no error"
    try:
        for w in rows.replicate_slabs(b_full, bufs, slabs, src=0, is_src=True):
            w.wait()
        dist.barrier()  # a broadcast's sender may complete locally; the barrier needs the peer
    except Exception as e:  # noqa: BLE001 - the error is what the test is about
        outcome = "error: " + type(e).__name__
    with open(os.path.join(tmp, "rank0.txt"), "w") as f:
        f.write("%s after %.1f s, step1_ok=%s" % (outcome, time.time() - t0, step1_ok))
    os._exit(0)


def test_a_rank_that_leaves_between_steps_ends_the_next_replication_with_an_error(tmp_path):
    """Failure detection on the host side (no GPU involved): the surviving rank learns of the
    loss through the process group (connection closed, or the group's short timeout) and gets
    an exception instead of waiting for ever."""
    port = _free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_leaving_worker, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert not p.is_alive(), "a rank hung after its peer left"
    r0 = (tmp_path / "rank0.txt").read_text()
    assert "left after step 1, step1_ok=True" in (tmp_path / "rank1.txt").read_text()
    assert r0.startswith("error: ") and "step1_ok=True" in r0, r0
    assert float(r0.split("after ")[1].split(" s")[0]) < 30
