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

Three ways to replicate B (`overlap=`):

    "ce"     (default) no NCCL kernel at all: B is replicated by the copy engines over
             NVLink (PeerReplicator: buffers shared over CUDA IPC, a pull of this rank's
             slice from the source, a stream-ordered barrier, pulls of the other slices
             from their holders), beside the GEMM of the previous call; every call is ONE
             GEMM launch on all SMs.  B is handed over once with register_b().
             Measured on 8 GPUs: 0.81 ms per step against 0.88 ms for "calls".
    "calls"  NCCL broadcast across calls: B travels as ONE slab into one of two replica
             buffers and the replication for call i+1 runs beside the GEMM of call i (the
             host enqueues ahead).  NCCL's broadcast runs 32 CTAs and finishes only when
             all of them have had an SM, so the GEMM is cut into two launches over column
             ranges of the same replica: the first leaves 32 SMs free and lasts about as
             long as the replication, the second uses the whole machine.  For processes
             that cannot share memory over CUDA IPC.
    "slabs"  NCCL broadcast inside one call, as described above: several GEMM launches
             per call; for a lone call.
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


def _wave_cost(tiles, clusters):
    """Waves of the persistent GEMM that `tiles` tiles cost on `clusters` CTA pairs: whole
    waves, plus a tail that the k-split shortens when it fills at most half of the pairs."""
    full, rem = divmod(tiles, clusters)
    if rem == 0:
        return float(full)
    parts = min(8, clusters // rem)
    return full + (1.0 / parts + 0.1 if parts >= 2 else 1.0)


def plan_two_parts(rows, n_cols, k, sm_count=148, comm_sms=32, comm_ms=0.5, tflops=1400.0):
    """Column split (w1, w2) for `overlap="calls"`: the first launch leaves `comm_sms` SMs
    to the NCCL kernel and covers the columns that keep it busy for about `comm_ms`
    (the replication takes 0.2-0.4 ms for 128 MiB on 2-8 GPUs); the second launch has
    the whole machine.  Among the widths within a few blocks of that target the one
    with the cheapest tails wins.  w2 may be 0 (short GEMM: one launch with margin)."""
    col_blocks = -(-n_cols // PAIR_TILE)
    row_blocks = max(1, -(-rows // PAIR_TILE))
    est_ms = 2.0 * rows * n_cols * k / (tflops * 1e9)
    frac = min(1.0, comm_ms * (sm_count - comm_sms) / sm_count / max(est_ms, 1e-9))
    if frac >= 0.85 or col_blocks < 4:
        return n_cols, 0
    target = max(1, round(frac * col_blocks))
    c1 = (sm_count - comm_sms) // 2
    c2 = sm_count // 2
    best = None
    for cb1 in range(target, min(col_blocks - 1, target + 3) + 1):
        cost = _wave_cost(row_blocks * cb1, c1) * c2 / c1 + _wave_cost(row_blocks * (col_blocks - cb1), c2)
        if best is None or cost < best[0] - 1e-9:
            best = (cost, cb1)
    w1 = min(best[1] * PAIR_TILE, n_cols)
    return w1, n_cols - w1


def plan_peer_slices(rows, world, src=0):
    """Row slices of B for the copy-engine replication: B's `rows` rows are cut into one
    block per rank other than `src` (the partition rule of shard_rows over world-1 parts).
    Returns {rank: (row0, nrows)} for the non-source ranks, in rank order.  Rank r pulls its
    own slice from `src` first, then every other slice from the rank that holds it."""
    holders = [r for r in range(world) if r != src]
    out = {}
    for i, r in enumerate(holders):
        out[r] = (rt.imexShardOffset(i, len(holders), rows), rt.imexShardSize(i, len(holders), rows))
    return out


class _PeerBuffers:
    """Device buffers of this rank shared with the other processes of the node over CUDA IPC,
    the peers' buffers mapped here, and the flag arrays of imexPeerBarrier.  Collective."""

    def __init__(self, session, rank, world, sizes, group=None):
        import ctypes as C

        import torch.distributed as dist
        self.C, self.dist, self.group = C, dist, group
        self.sess, self.rank, self.world = session, rank, world
        self.epoch = 0
        self.local = {}    # name -> local device pointer
        self.peer = {}     # (name, rank) -> address of that rank's buffer in this process
        for name, size in list(sizes.items()) + [("flags", 256)]:
            self.local[name] = session.alloc(size)
        zeros = (C.c_char * 256)()
        rt.gpuMemCopy(session.stream, self.local["flags"], C.addressof(zeros), 256)
        mine = {}
        for name, ptr in self.local.items():
            buf = (C.c_char * 64)()
            rt.library().imexIpcExport(ptr, C.addressof(buf))
            mine[name] = bytes(buf)
        everyone = [None] * world
        dist.all_gather_object(everyone, mine, group=group)
        for r, handles in enumerate(everyone):
            for name, h in handles.items():
                if r == rank:
                    self.peer[(name, r)] = self.local[name]
                else:
                    hb = (C.c_char * 64).from_buffer_copy(h)
                    self.peer[(name, r)] = rt.library().imexIpcOpen(C.addressof(hb))
        self.flag_ptrs = (C.c_void_p * world)(*[self.peer[("flags", r)] for r in range(world)])
        dist.barrier(group=group)  # nobody starts copying before everyone has mapped everything

    def barrier(self, stream=None):
        """Stream-ordered barrier over the ranks (every rank calls it the same number of times)."""
        self.epoch += 1
        rt.library().imexPeerBarrier(stream or self.sess.stream, self.flag_ptrs, self.world, self.rank, self.epoch)
        rt.library().imexNoteLaunches(1)

    def pull(self, dst, src, nbytes, stream=None):
        rt.library().imexMemCopyAsync(stream or self.sess.stream, dst, src, nbytes)

    def close(self):
        for (name, r), ptr in self.peer.items():
            if r != self.rank:
                rt.library().imexIpcClose(ptr)
        self.peer.clear()


class PeerReplicator(_PeerBuffers):
    """B[k, n] of rank `src` copied into every rank's own HBM by the copy engines.

    Buffers come from gpuMemAlloc and are shared between the processes with CUDA IPC
    (imexIpcExport / imexIpcOpen); all copies are imexMemCopyAsync on `comm_session`'s stream
    (DMA over NVLink, no SM); the ranks meet once per replication in imexPeerBarrier.
    Per call, on a rank r other than src:   pull slice r from src   ->   barrier   ->
    pull slice j from rank j for every other j.  src only takes part in the barrier.
    Two replica buffers alternate so that the replication for the next call can run while
    the GEMM of this one still reads the other buffer.  Collective: every rank constructs,
    registers and replicates in the same order."""

    def __init__(self, comm_session, rank, world, k, n, elt_bytes, src=0, group=None):
        self.src, self.k, self.n, self.esz = src, k, n, elt_bytes
        self.nbytes = k * n * elt_bytes
        self.slices = plan_peer_slices(k, world, src)
        sizes = {"source": self.nbytes} if rank == src else {"replica0": self.nbytes, "replica1": self.nbytes}
        super().__init__(comm_session, rank, world, sizes, group)

    def register_source(self, b_full_ptr):
        """src: copies B (device pointer) into the shared source buffer.  Other ranks: no-op.
        Call again whenever B changes; the next replicate() carries the new contents."""
        if self.rank == self.src:
            rt.gpuMemCopy(self.sess.stream, self.local["source"], b_full_ptr, self.nbytes)

    def local_b(self, which):
        """Device pointer of the full B on this rank after replicate(which)."""
        return self.local["source"] if self.rank == self.src else self.local["replica%d" % which]

    def replicate(self, which):
        """Enqueues one replication into replica buffer `which` on the comm stream."""
        row_bytes = self.n * self.esz
        name = "replica%d" % which
        if self.rank != self.src:
            r0, nr = self.slices[self.rank]
            self.pull(self.local[name] + r0 * row_bytes, self.peer[("source", self.src)] + r0 * row_bytes,
                      nr * row_bytes)
        self.barrier()
        if self.rank != self.src:
            # start with the next rank up so that no holder serves everybody at once
            for j in sorted((r for r in self.slices if r != self.rank), key=lambda r: (r - self.rank) % self.world):
                r0, nr = self.slices[j]
                self.pull(self.local[name] + r0 * row_bytes, self.peer[(name, j)] + r0 * row_bytes, nr * row_bytes)


class PeerAllGather(_PeerBuffers):
    """An array of `rows` rows of `row_bytes` each, of which every rank fills its own block of
    rows (the partition rule of shard_rows) and fetches the others' blocks over NVLink with
    the copy engines.  Used by the host-buffer pipeline: the ranks of a node upload 1/world
    of B each instead of all of B each."""

    def __init__(self, session, rank, world, rows, row_bytes, group=None):
        self.rows, self.row_bytes = rows, row_bytes
        self.blocks = [shard_rows(r, world, rows) for r in range(world)]
        super().__init__(session, rank, world, {"array": rows * row_bytes}, group)

    @property
    def array(self):
        return self.local["array"]

    def own_block(self):
        """(byte offset, bytes) of the rows this rank has to fill before exchange()."""
        r0, nr = self.blocks[self.rank]
        return r0 * self.row_bytes, nr * self.row_bytes

    def exchange(self, stream=None):
        """Enqueues: barrier (every block is filled), pulls of the other ranks' blocks, barrier
        (nobody still reads a block that its owner may refill)."""
        self.barrier(stream)
        for j in sorted((r for r in range(self.world) if r != self.rank), key=lambda r: (r - self.rank) % self.world):
            r0, nr = self.blocks[j]
            if nr:
                self.pull(self.array + r0 * self.row_bytes, self.peer[("array", j)] + r0 * self.row_bytes,
                          nr * self.row_bytes, stream)
        self.barrier(stream)


class RowShardedGemm:
    """C[rows of this rank, :] = epilogue(A[rows of this rank, :] . B), B replicated
    from rank `src` inside every call."""

    def __init__(self, session, rank, world, m_total, n, k, in_dtype=B.BF16, epilogue=B.EPI_NONE,
                 src=0, sm_margin=None, slabs=None, device=None, overlap="ce", comm_ms=0.5):
        """overlap="ce": one launch on all SMs (sm_margin 0).  overlap="slabs": sm_margin (default
        8) SMs stay free during every slab GEMM.  overlap="calls": the first of two launches
        leaves sm_margin (default 32: NCCL runs 32 CTAs here) SMs free, the second none (see
        plan_two_parts)."""
        import torch
        self.torch = torch
        self.sess, self.rank, self.world, self.src = session, rank, world, src
        self.m_total, self.n, self.k = m_total, n, k
        self.row0, self.rows = shard_rows(rank, world, m_total)
        if overlap not in ("slabs", "calls", "ce"):
            raise ValueError("overlap must be 'slabs', 'calls' or 'ce'")
        self.overlap = overlap
        if sm_margin is None:
            sm_margin = 8 if overlap == "slabs" else 0 if overlap == "ce" else 32
        self.margin = sm_margin if world > 1 else 0
        if slabs is None:
            slabs = plan_slabs(self.rows, n, world, sm_margin=sm_margin) if overlap == "slabs" else [(0, n)]
        self.slabs = slabs
        self.device = device
        self.comm_stream = torch.cuda.Stream(device=device) if world > 1 else None
        elt = torch.bfloat16 if in_dtype == B.BF16 else torch.float16
        # two sets of slab buffers: the broadcast of call i+1 may run while the GEMMs of
        # call i still read theirs, so back-to-back calls hide the replication entirely
        self.slab_sets = None
        self.calls = 0
        self.done_events = [None, None]
        self.peer = None
        if world > 1 and overlap == "ce":
            # copy-engine replication: library-owned buffers shared over CUDA IPC, no NCCL kernel
            from .session import Session
            dev_index = device.index if hasattr(device, "index") and device.index is not None else 0
            self.comm_sess = Session(device=dev_index, adopt_stream=self.comm_stream.cuda_stream)
            self.peer = PeerReplicator(self.comm_sess, rank, world, k, n, B.DTYPE_BYTES[in_dtype], src=src)
        elif world > 1:
            self.slab_sets = [[torch.empty((k, w), dtype=elt, device=device) for _, w in self.slabs]
                              for _ in range(2)]
            self.slab_bufs = self.slab_sets[0]
        # launches: (slab index, first column inside the slab, first column of C, kernel)
        self.launches, self.launch_descs = [], []
        self.trace = None         # set to a list to collect four timing events per call (see __call__)
        self.slab_bufs = self.slab_sets[0] if self.slab_sets else None
        if world > 1 and overlap == "ce":
            desc = B.gemm("row_sharded_gemm_whole", self.rows, n, k, in_dtype, epilogue, sm_margin=self.margin)
            self.launch_descs.append(desc)
            self.launches.append((0, 0, 0, session.kernel(desc)))
        elif world > 1 and overlap == "calls" and len(self.slabs) == 1:
            w1, w2 = plan_two_parts(self.rows, n, k, comm_sms=self.margin, comm_ms=comm_ms)
            for j, (c0, w, margin) in enumerate([(0, w1, self.margin), (w1, w2, 0)]):
                if w:
                    desc = B.gemm(f"row_sharded_gemm_part{j}", self.rows, w, k, in_dtype, epilogue,
                                  ldb=n if w != n else 0, ldc=n if w != n else 0, sm_margin=margin)
                    self.launch_descs.append(desc)
                    self.launches.append((0, c0, c0, session.kernel(desc)))
        else:
            for j, (c0, w) in enumerate(self.slabs):
                ldb = w if world > 1 else 0
                desc = B.gemm(f"row_sharded_gemm_slab{j}", self.rows, w, k, in_dtype, epilogue,
                              ldb=ldb, ldc=n if w != n else 0, sm_margin=self.margin)
                self.launch_descs.append(desc)
                self.launches.append((j, 0, c0, session.kernel(desc)))
        self.kernels = [l[3] for l in self.launches]
        self.elt_bytes = 2

    def launch_gemms(self, a_shard, c_shard, bufs=None, works=None, on_first_wait=None):
        """Enqueue the GEMM launches of one call on the current stream; with `works`
        every launch first waits for the replication of its slab."""
        bufs = bufs if bufs is not None else self.slab_bufs
        waited = set()
        for slab, b_col, c_col, kern in self.launches:
            if works is not None and slab not in waited:
                works[slab].wait()  # the current stream waits for this slab only
                waited.add(slab)
                if on_first_wait is not None and len(waited) == 1:
                    on_first_wait()
            self.sess.launch(kern, [a_shard.data_ptr(), bufs[slab].data_ptr() + self.elt_bytes * b_col,
                                    c_shard.data_ptr() + 4 * c_col], wait=False)
        return len(self.launches)

    class _Ptr:
        """A device address with the data_ptr() of a tensor."""

        def __init__(self, ptr):
            self.ptr = int(ptr)

        def data_ptr(self):
            return self.ptr

    def register_b(self, b_full):
        """overlap="ce": hands B (valid on `src`) to the copy-engine replication.  Collective;
        needed once, and again whenever B's contents change."""
        if self.peer is not None:
            self.torch.cuda.current_stream().synchronize()
            self.peer.register_source(b_full.data_ptr())
            self.registered = b_full.data_ptr()

    def check(self):
        """Waits for the replication stream and raises (through the library's error convention)
        if a cross-rank barrier gave up waiting for a peer."""
        if self.peer is not None:
            self.comm_sess.wait()

    def close(self):
        """Collective: unmaps the peers' buffers, then frees this rank's."""
        if self.peer is not None:
            self.torch.cuda.synchronize()
            self.peer.dist.barrier()
            self.peer.close()
            self.peer.dist.barrier()
            self.comm_sess.close()
            self.peer = None

    def _call_ce(self, a_shard, c_shard):
        """One call with the replication on the copy engines: replica buffer `which` is filled
        on the comm stream (beside the GEMM of the previous call, which reads the other
        buffer), then ONE GEMM launch on all SMs."""
        torch = self.torch
        cur = torch.cuda.current_stream()
        which = self.calls & 1
        self.calls += 1
        if self.done_events[which] is not None:  # the GEMM that last read this replica buffer
            self.comm_stream.wait_event(self.done_events[which])
        self.peer.replicate(which)
        ready = torch.cuda.Event()
        ready.record(self.comm_stream)
        cur.wait_event(ready)
        self.slab_bufs = [RowShardedGemm._Ptr(self.peer.local_b(which))]
        n_launch = self.launch_gemms(a_shard, c_shard, self.slab_bufs)
        done = torch.cuda.Event()
        done.record(cur)
        self.done_events[which] = done
        return n_launch

    def __call__(self, a_shard, b_full, c_shard, b_ready=None):
        """a_shard [rows,k], c_shard [rows,n] on this rank; b_full [k,n] valid on `src`
        (a scratch tensor of that shape elsewhere).  Enqueues on the current stream.

        b_ready: None  -> the broadcast waits for everything queued so far on the
                          current stream (b_full may be produced there); safe default;
                 True  -> b_full is already complete in memory (resident weights): the
                          broadcast starts at once and overlaps earlier GEMMs;
                 event -> the broadcast waits for that CUDA event only.
        overlap="ce" replicates the B handed over with register_b() and ignores b_full / b_ready."""
        torch = self.torch
        if self.world == 1:
            return self.launch_gemms(a_shard, c_shard, bufs=[b_full])
        if self.overlap == "ce":
            if getattr(self, "registered", None) is None:
                raise RuntimeError("overlap='ce': call register_b(b_full) on every rank first")
            return self._call_ce(a_shard, c_shard)
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
        ev = None
        if self.trace is not None:  # (broadcast may start, broadcast done, GEMMs may start, GEMMs done)
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            ev[0].record(self.comm_stream)
        if self.rank == self.src and len(self.slabs) == 1 and b_full.is_contiguous():
            # one full-width slab: the source sends B from where it lies and multiplies
            # with it in place (no packing copy competing with the GEMM for SMs)
            if b_ready is not None and b_ready is not True:
                cur.wait_event(b_ready)
            bufs = self.slab_bufs = [b_full]
            with torch.cuda.stream(self.comm_stream):
                import torch.distributed as dist
                works = [dist.broadcast(b_full, src=self.src, async_op=True)]
        else:
            works = replicate_slabs(b_full, bufs, self.slabs, self.src, self.rank == self.src,
                                    self.comm_stream)
        if ev is not None:
            with torch.cuda.stream(self.comm_stream):
                works[-1].wait()
            ev[1].record(self.comm_stream)
        n_launch = self.launch_gemms(a_shard, c_shard, bufs, works,
                                     on_first_wait=(lambda: ev[2].record(cur)) if ev is not None else None)
        if ev is not None:
            ev[3].record(cur)
            self.trace.append(ev)
        done = torch.cuda.Event()
        done.record(cur)
        self.done_events[which] = done
        return n_launch


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
