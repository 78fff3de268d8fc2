"""Row-sharded execution over the GPUs of one box (one process per GPU).

The reference shards arrays with `shard.grid` / `shard.sharding split_axes =
[[0]]` annotations (test/Dialect/NDArray/Extensions/sharding_propagation.mlir:4-12)
and a block partition rule in which the LAST extent % n shards get one extra
element (lib/Dialect/NDArray/Extensions/MeshShardingExtensions.cpp:74-100); its
lowering exchanges data through MPI.  Here rank r owns a block of rows of A
(and of C / X / Y), `torch.distributed` over NCCL is the transport, and the
only exchange step of the GEMM is the replication of B:

    B lives on rank 0.  It is cut into column slabs; rank 0 packs slab j
    into a contiguous [K, w_j] buffer and NCCL-broadcasts it on a side stream
    while the GEMM for slab j-1 runs; every rank multiplies its rows of A with
    slab j as soon as that slab has landed in its own HBM (stream events, no
    device-side spinning) and writes columns [c_j, c_j + w_j) of its rows of C.

Slabs are sized in whole waves of the persistent GEMM (tiles per slab a
multiple of the CTA pairs in flight) so that cutting B costs no tail.  The
GEMM leaves `sm_margin` SMs free so that the NCCL kernel of the next slab can
run beside it.  Softmax and row-reduce shard by rows with no exchange at all.

Two ways to hide the replication (`overlap=`):

    "slabs"  inside one call, as above: several GEMM launches per call.
    "calls"  across calls: B travels as ONE slab into one of two replica
             buffers, the GEMM is a single launch over the whole width, and
             the replication for call i+1 runs beside the GEMM of call i
             (the host enqueues ahead).  Every extra GEMM launch costs a
             pipeline ramp and an un-overlapped drain, so this is the faster
             form for back-to-back calls; a lone call pays the whole
             replication up front.
"""
from . import blob as B
from . import runtime as rt

PAIR_TILE = 256  # the 2-CTA GEMM works on 256 x 256 output tiles


def shard_rows(rank, world, extent):
    """(offset, size) of rank's block — the reference's partition rule."""
    return rt.imexShardOffset(rank, world, extent), rt.imexShardSize(rank, world, extent)


def plan_slabs(rows, n_cols, world, sm_count=148, sm_margin=4, max_slabs=8):
    """Column slabs [(col0, width), ...] of B for a rank that owns `rows` rows.

    world == 1: one slab (nothing to overlap).  Otherwise widths are multiples
    of 256 columns chosen so that (row blocks x column blocks) of a slab fills
    whole waves of the (sm_count - sm_margin)/2 CTA pairs, first slab smallest
    so the first GEMM starts early."""
    if world <= 1 or n_cols <= PAIR_TILE:
        return [(0, n_cols)]
    clusters = max(1, (sm_count - sm_margin) // 2)
    row_blocks = max(1, -(-rows // PAIR_TILE))
    col_blocks = -(-n_cols // PAIR_TILE)
    # smallest number of column blocks whose tile count is a whole number of waves
    unit = 1
    while unit < col_blocks and (row_blocks * unit) % clusters:
        unit += 1
    if (row_blocks * unit) % clusters:  # no exact fit: four near-equal slabs
        widths = [col_blocks // 4 + (1 if i < col_blocks % 4 else 0) for i in range(4)]
        widths = [w for w in widths if w]
    else:
        full = min(col_blocks // unit, max_slabs - 1)
        rest = col_blocks - full * unit
        widths = ([rest] if rest else []) + [unit] * full  # the short slab goes first
    slabs, c = [], 0
    for w in widths:
        width = min(w * PAIR_TILE, n_cols - c)
        slabs.append((c, width))
        c += width
    return slabs


def replicate_slabs(b_full, slab_bufs, slabs, src, is_src, comm_stream=None):
    """Pack (on the source rank) and broadcast every slab; returns the work
    handles in slab order.  Device-agnostic torch code: runs over NCCL on GPUs
    and over gloo on CPU tensors (tests)."""
    import torch
    import torch.distributed as dist
    works = []
    ctx = torch.cuda.stream(comm_stream) if comm_stream is not None else _NullCtx()
    with ctx:
        for (c0, w), buf in zip(slabs, slab_bufs):
            if is_src:
                buf.copy_(b_full[:, c0:c0 + w])
            works.append(dist.broadcast(buf, src=src, async_op=True))
    return works


class _NullCtx:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


class RowShardedGemm:
    """C[rows of this rank, :] = epilogue(A[rows of this rank, :] . B), B replicated
    from rank `src` inside every call."""

    def __init__(self, session, rank, world, m_total, n, k, in_dtype=B.BF16, epilogue=B.EPI_NONE,
                 src=0, sm_margin=4, slabs=None, device=None, overlap="slabs"):
        import torch
        self.torch = torch
        self.sess, self.rank, self.world, self.src = session, rank, world, src
        self.m_total, self.n, self.k = m_total, n, k
        self.row0, self.rows = shard_rows(rank, world, m_total)
        self.margin = sm_margin if world > 1 else 0
        if overlap not in ("slabs", "calls"):
            raise ValueError("overlap must be 'slabs' or 'calls'")
        self.overlap = overlap
        if slabs is None:
            slabs = [(0, n)] if overlap == "calls" else plan_slabs(self.rows, n, world, sm_margin=sm_margin)
        self.slabs = slabs
        self.device = device
        self.comm_stream = torch.cuda.Stream(device=device) if world > 1 else None
        elt = torch.bfloat16 if in_dtype == B.BF16 else torch.float16
        # two sets of slab buffers: the broadcast of call i+1 may run while the GEMMs of
        # call i still read theirs, so back-to-back calls hide the replication entirely
        self.slab_sets = None
        self.calls = 0
        self.done_events = [None, None]
        if world > 1:
            self.slab_sets = [[torch.empty((k, w), dtype=elt, device=device) for _, w in self.slabs]
                              for _ in range(2)]
            self.slab_bufs = self.slab_sets[0]
        self.kernels = []
        for j, (c0, w) in enumerate(self.slabs):
            ldb = w if world > 1 else 0
            self.kernels.append(session.kernel(B.gemm(
                f"row_sharded_gemm_slab{j}", self.rows, w, k, in_dtype, epilogue,
                ldb=ldb, ldc=n if w != n else 0, sm_margin=self.margin)))

    def __call__(self, a_shard, b_full, c_shard, b_ready=None):
        """a_shard [rows,k], c_shard [rows,n] on this rank; b_full [k,n] valid on `src`
        (a scratch tensor of that shape elsewhere).  Enqueues on the current stream.

        b_ready: None  -> the broadcast waits for everything queued so far on the
                          current stream (b_full may be produced there); safe default;
                 True  -> b_full is already complete in memory (resident weights): the
                          broadcast starts at once and overlaps earlier GEMMs;
                 event -> the broadcast waits for that CUDA event only."""
        torch = self.torch
        if self.world == 1:
            self.sess.launch(self.kernels[0], [a_shard.data_ptr(), b_full.data_ptr(),
                                               c_shard.data_ptr()], wait=False)
            return 1
        cur = torch.cuda.current_stream()
        which = self.calls & 1
        self.calls += 1
        bufs = self.slab_bufs = self.slab_sets[which]
        if b_ready is None:
            self.comm_stream.wait_stream(cur)
        elif b_ready is not True:
            self.comm_stream.wait_event(b_ready)
        # this set of slab buffers was last read by the GEMMs of two calls ago
        if self.done_events[which] is not None:
            self.comm_stream.wait_event(self.done_events[which])
        works = replicate_slabs(b_full, bufs, self.slabs, self.src, self.rank == self.src,
                                self.comm_stream)
        for (c0, w), buf, work, kern in zip(self.slabs, bufs, works, self.kernels):
            work.wait()  # the current stream waits for this slab only
            self.sess.launch(kern, [a_shard.data_ptr(), buf.data_ptr(),
                                    c_shard.data_ptr() + 4 * c0], wait=False)
        done = torch.cuda.Event()
        done.record(cur)
        self.done_events[which] = done
        return len(self.slabs)


def all_gather_rows(shard, full, rank, world, extent):
    """Optional last step of a row-sharded op: every rank ends up with all rows.

    shard [rows of this rank, ...] -> full [extent, ...] on every rank.  Rows are laid
    out by the block partition rule, so rank r's block lands at its own offset.  Even
    partitions travel as one all-gather straight into `full`; ragged ones as one
    broadcast per rank into that rank's row block (NCCL all-gather wants equal
    counts).  The reference leaves this to its distributed runtime's gather of the
    local parts (`ndarray`/`dist` lowering to `_idtr_*` calls, not in the reference
    tree); here it is NCCL over NVLink, or gloo on CPU tensors in the tests."""
    import torch.distributed as dist
    sizes = [rt.imexShardSize(r, world, extent) for r in range(world)]
    if world == 1:
        full.copy_(shard)
        return full
    if len(set(sizes)) == 1:
        dist.all_gather_into_tensor(full, shard.contiguous())
        return full
    for r in range(world):
        off = rt.imexShardOffset(r, world, extent)
        block = full[off:off + sizes[r]]
        if r == rank:
            block.copy_(shard)
        if sizes[r]:
            dist.broadcast(block, src=r)
    return full
