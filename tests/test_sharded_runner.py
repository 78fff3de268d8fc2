"""Row sharding through the reference's annotation surface: shard.grid / shard.sharding
split_axes = [[0]] / shard.shard (test/Dialect/NDArray/Extensions/sharding_propagation.mlir:4-12)
on func/linalg programs.  Each rank of the grid runs the program on its own block of rows
(partition rule of lib/Dialect/NDArray/Extensions/MeshShardingExtensions.cpp:74-100); the
ranks' outputs put together must be the output of the unsharded run."""
import os
import re
import subprocess

import pytest

from __graft_entry__ import ROOT

RUNNER = os.path.join(ROOT, "mlir-extensions_b200", "bin", "imex-b200-runner")
ORACLE_RUNNER = os.path.join(ROOT, "oracle", "_cpu", "imex-oracle-runner")
FIXTURE = os.path.join(ROOT, "tests", "mlir", "sharded_rows.mlir")


def _memrefs(text):
    """[(sizes, flat list of numbers)] for every printed memref."""
    out = []
    for m in re.finditer(r"sizes = \[([^\]]*)\] strides = \[[^\]]*\] data =\s*\n((?:[ \[].*\n?)+)", text):
        sizes = [int(x) for x in m.group(1).split(",") if x.strip()]
        nums = [float(x) for x in re.findall(r"-?(?:\d+\.?\d*(?:e[-+]?\d+)?|inf|nan)", m.group(2))]
        out.append((sizes, nums))
    return out


def _run(runner, *args):
    r = subprocess.run([runner, FIXTURE, "-e", "main", *args], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-800:] + r.stderr[-800:]
    return _memrefs(r.stdout)


def _ranks_together_equal_the_whole(runner, extra):
    whole = _run(runner, *extra)
    assert [s for s, _ in whole] == [[9, 2], [9]]
    parts = [_run(runner, *extra, "--shard-rank", str(r), "--shard-count", "4") for r in range(4)]
    # blocks of 2, 2, 2 and 3 rows: the last 9 % 4 ranks hold one row more
    assert [p[0][0] for p in parts] == [[2, 2], [2, 2], [2, 2], [3, 2]]
    assert [p[1][0] for p in parts] == [[2], [2], [2], [3]]
    for k in range(2):
        joined = [x for p in parts for x in p[k][1]]
        assert joined == whole[k][1]


@pytest.mark.skipif(not os.path.exists(ORACLE_RUNNER), reason="oracle/_cpu/imex-oracle-runner is not built")
def test_ranks_together_equal_the_whole_on_the_cpu_checker():
    _ranks_together_equal_the_whole(ORACLE_RUNNER, ["--all-loopnests"])


def test_plan_of_a_rank_shows_its_rows_and_local_kernel_shapes():
    r = subprocess.run([RUNNER, FIXTURE, "--emit-plan", "--shard-rank", "3", "--shard-count", "4"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    assert "shard: rows [6, 9) of 9 on rank 3 of 4" in r.stdout
    kernels = [l for l in r.stdout.splitlines() if l.startswith("kernel ")]
    assert "gemm f32->f32 +bias +relu dims=[3,2,3]" in kernels[0]      # 3 of the 9 rows of A and C
    assert "row_sum dims=[3,3" in kernels[1]
    # a single rank (the default) runs the whole arrays
    r = subprocess.run([RUNNER, FIXTURE, "--emit-plan"], capture_output=True, text=True)
    assert r.returncode == 0 and "dims=[9,2,3]" in r.stdout and "shard: rows" not in r.stdout


def test_what_needs_an_exchange_between_ranks_is_refused(tmp_path):
    """A reduction over the split dimension (column sums of a row-sharded array) would need the
    ranks to exchange partial results: refused, by name, instead of computing on one block."""
    text = open(FIXTURE).read()
    text = text.replace("indexing_maps = [#id, #row], iterator_types = [\"parallel\", \"reduction\"]} "
                        "ins(%as : tensor<9x3xf32>) outs(%y0 : tensor<9xf32>)",
                        "indexing_maps = [affine_map<(d0, d1) -> (d1, d0)>, #row], iterator_types = "
                        "[\"parallel\", \"reduction\"]} ins(%as : tensor<9x3xf32>) outs(%y0 : tensor<9xf32>)")
    p = tmp_path / "colsum.mlir"
    p.write_text(text)
    r = subprocess.run([RUNNER, str(p), "--emit-plan", "--shard-rank", "1", "--shard-count", "4"],
                       capture_output=True, text=True)
    assert r.returncode == 1 and "exchange between them" in r.stderr
    # and a grid of another size than the run
    r = subprocess.run([RUNNER, FIXTURE, "--emit-plan", "--shard-rank", "1", "--shard-count", "2"],
                       capture_output=True, text=True)
    assert r.returncode == 1 and "--shard-count 2" in r.stderr


@pytest.mark.gpu
@pytest.mark.parametrize("mode", [[], ["--all-loopnests"]])
def test_ranks_together_equal_the_whole_on_the_gpu(mode):
    _ranks_together_equal_the_whole(RUNNER, mode)
