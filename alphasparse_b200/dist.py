"""Row-block sharding of one matrix over the GPUs of a node, x replicated.

Rank p owns the contiguous rows [bounds[p], bounds[p+1]) (nnz-balanced, asp_partition_rows_by_nnz),
builds its own format on that block with global column indices and runs the single-GPU path. A
single SpMV needs no communication. In repeated-SpMV mode (x <- A x) every rank's new slice has to
reach every other rank before the next iteration. The slices differ in length (nnz-balanced blocks of
a skewed matrix differ several-fold in rows), so they are exchanged unpadded: each rank sends its
slice straight into the peers' next-x buffers at the slice's own offset (NCCL grouped send/recv,
i.e. `all_to_all` on tensor lists), and the kernels write their slice of the next x in place, so
there is no staging copy either. To hide the exchange a rank's block is cut into row chunks, each
with its own plan group: chunk c travels on a second stream while chunk c+1 is computed. Kernels
only ever read local memory; NCCL moves remote data into it first.

The reference is single-GPU (code_builder.cc:1483-1489); this module has no counterpart there.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist


class ShardedSpmv:
    """`local_spmv(x, y_rows)` computes this rank's slice: x is the full replicated vector (torch
    tensor, length n_cols), y_rows a tensor view of exactly the rows to produce. On a GPU it is
    `PlanGroup.spmv` on the tensors' pointers; the CPU tests pass a host function.

    `chunks`, if given, replaces `local_spmv` by a list of `(fn, lo, hi)`: fn(x, y_rows) produces the
    local rows [lo, hi) (relative to bounds[rank]); the ranges must tile the rank's block. They are
    computed and exchanged in list order, and only the last exchange is not hidden behind a kernel,
    so the chunk with the fewest rows belongs last. The ranks may cut their blocks into different
    numbers of chunks; the pairwise exchanges ("a2a", "allgather", the gloo loop) pair the c-th chunks
    of all ranks and then exchange each block as one piece instead.

    exchange="publish": a chunk may carry a 4th entry `pub(x_ptr, y_ptr, y_multicast_ptr)` that computes
    AND publishes its rows from one kernel (PlanGroup.spmv_publish); then nothing is exchanged
    afterwards, and one bounded-wait barrier kernel per SpMV (asp_rank_barrier) orders the ranks.
    Vectors must come from new_vector(), which returns them zero-filled: rows that no kernel ever
    writes (rows without non-zeros that a format dropped) stay zero in every replica.
    """

    def __init__(self, local_spmv, bounds, rank: int, world: int, dtype, device, group=None, chunks=None, exchange: str = "allgather",
                 n_total: int | None = None):
        self.bounds = [int(b) for b in bounds]
        self.rank, self.world, self.group = rank, world, group
        self.rows = [self.bounds[p + 1] - self.bounds[p] for p in range(world)]
        # length of the vectors; rows [bounds[-1], n_total) belong to nobody: no non-zeros, zero in every vector
        self.n = int(n_total) if n_total is not None else self.bounds[-1]
        assert self.n >= self.bounds[-1]
        self.device = torch.device(device)
        my_rows = self.rows[rank]
        self.chunks = [tuple(c) for c in chunks] if chunks is not None else [(local_spmv, 0, my_rows)]
        self._pub = [c[3] if len(c) > 3 else None for c in self.chunks]
        self.chunks = [c[:3] for c in self.chunks]
        tiled = sorted((lo, hi) for _, lo, hi in self.chunks)
        assert tiled[0][0] == 0 and tiled[-1][1] == my_rows and all(tiled[i][1] == tiled[i + 1][0] for i in range(len(tiled) - 1))
        self.y_local = torch.zeros(max(1, my_rows), dtype=dtype, device=device)
        # every rank's chunks in global rows, in the order they are computed and exchanged:
        # span[p][c] = (first row, end row) of the c-th chunk of rank p
        C = len(self.chunks)
        mine = torch.tensor([[self.bounds[rank] + lo, self.bounds[rank] + hi] for _, lo, hi in self.chunks], dtype=torch.int64).reshape(-1)
        if world > 1:
            counts = [torch.zeros(1, dtype=torch.int64, device=device) for _ in range(world)]
            dist.all_gather(counts, torch.tensor([C], dtype=torch.int64, device=device), group=group)
            counts = [int(c.item()) for c in counts]
            self._equal_chunks = all(c == C for c in counts)
            cmax = max(counts)
            padded = torch.zeros(2 * cmax, dtype=torch.int64)
            padded[: 2 * C] = mine
            allc = [torch.zeros(2 * cmax, dtype=torch.int64, device=device) for _ in range(world)]
            dist.all_gather(allc, padded.to(device), group=group)
            self.span = [[(int(t[2 * c]), int(t[2 * c + 1])) for c in range(counts[p])] for p, t in enumerate(u.cpu() for u in allc)]
        else:
            self.span = [[(int(mine[2 * c]), int(mine[2 * c + 1])) for c in range(C)]]
            self._equal_chunks = True
        self.on_gpu = self.device.type == "cuda"
        # (default priority: a high-priority exchange stream was measured and lost at 8 GPUs,
        # 0.85 -> 0.95 ms per SpMV at scale 26)
        self._comm = torch.cuda.Stream(device=self.device) if (self.on_gpu and world > 1) else None
        self._ev = [torch.cuda.Event() for _ in range(C)] if self._comm is not None else None
        self._done = torch.cuda.Event() if self._comm is not None else None
        self._empty = torch.empty(0, dtype=dtype, device=device)
        # NCCL: "allgather" = all_gather on unequal views (one broadcast per owner, grouped into one
        # launch; the owner's slice leaves its GPU once), "a2a" = grouped send/recv pairs (the slice
        # leaves the owner once per peer). gloo has neither for unequal sizes: broadcasts in a loop.
        #   "multicast" = the owner stores its slice once through an NVLink multicast address and
        # NVSwitch replicates it into every rank's buffer (asp_multicast_store); x and x_next must
        # then come from new_vector(), which maps them symmetrically on all ranks. A one-element
        # all-reduce after the last chunk orders the stores of all ranks before the next SpMV.
        nccl = world > 1 and dist.get_backend(group) == "nccl"
        self._mode = exchange if nccl else "bcast_loop"
        self._fallback_mode = "allgather" if nccl else "bcast_loop"
        if self._mode not in ("allgather", "a2a", "bcast_loop", "multicast", "publish"):
            raise ValueError(f"unknown exchange mode {exchange}")
        if self._mode == "publish" and any(p is None for p, (_, lo, hi) in zip(self._pub, self.chunks) if hi > lo):
            self._mode = "multicast"  # a chunk without a publishing kernel: separate store pass
        # the ranks must agree on the mode (one rank's chunks may lack a publishing kernel)
        if nccl:
            code = {"publish": 3, "multicast": 2}.get(self._mode, 1)
            t = torch.tensor([code], dtype=torch.int32, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
            if int(t.item()) != code:
                self._mode = {3: "publish", 2: "multicast"}.get(int(t.item()), exchange if exchange in ("allgather", "a2a") else "allgather")
        if self._mode in ("allgather", "a2a", "bcast_loop") and not self._equal_chunks:
            self._whole_blocks()
        self._epoch = 0
        self._flags = self._flags_mc = self._status = None
        self._dtype = dtype
        self._mc = {}  # data_ptr of a symmetric vector -> its multicast address
        self._symm_keep = []
        self._flag = torch.zeros(1, dtype=torch.float32, device=device) if self._mode in ("multicast", "publish") else None

    def _all_agree(self, ok: bool) -> bool:
        """Collective: True only when `ok` holds on every rank. Every rank calls it at the same points
        of new_vector(), whatever happened locally, so a rank with a local failure never leaves the
        others waiting in a rendezvous or a collective it has skipped."""
        t = torch.tensor([1 if ok else 0], dtype=torch.int32, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.group)
        return int(t.item()) == 1

    def _symm_alloc(self):
        """Local part of a symmetric allocation (may raise on this rank only)."""
        import torch.distributed._symmetric_memory as symm

        gname = (self.group or dist.group.WORLD).group_name
        try:
            symm.enable_symm_mem_for_group(gname)
        except Exception:
            pass
        return symm, gname, symm.empty(self.n, dtype=self._dtype, device=self.device)

    def _whole_blocks(self) -> None:
        """The pairwise exchanges pair the c-th chunks of all ranks: when the ranks cut their blocks into different
        numbers of chunks, every rank's block is exchanged as ONE piece after its last chunk (no overlap then)."""
        self._whole_block_exchange = True
        self.span = [[(self.bounds[p], self.bounds[p + 1])] for p in range(self.world)]

    def _fall_back(self, why: str) -> None:
        # (called on every rank with the collectively agreed outcome, so all ranks take the same path)
        if not self._equal_chunks:
            self._whole_blocks()
        self._mode = self._fallback_mode
        self.fallback_reason = why[:200]

    def new_vector(self) -> torch.Tensor:
        """A length-n vector usable as x / x_next. In multicast mode it is symmetric memory mapped
        on every rank and bound to a multicast object; when any rank cannot provide that, ALL ranks
        fall back to the plain exchange together (then an ordinary tensor is returned)."""
        if self._mode in ("multicast", "publish"):
            t = hdl = None
            err = ""
            try:
                symm, gname, t = self._symm_alloc()
            except Exception as e:  # local: import, out of memory, ...
                err = repr(e)
            if not self._all_agree(t is not None):
                self._fall_back(err or "symmetric allocation failed on another rank")
            else:
                mc = 0
                try:
                    hdl = symm.rendezvous(t, gname)
                    mc = int(hdl.multicast_ptr)
                except Exception as e:
                    err = repr(e)
                if not self._all_agree(mc != 0):
                    self._fall_back(err or "no multicast address for symmetric memory on some rank")
                else:
                    t.zero_()
                    self._mc[t.data_ptr()] = mc
                    self._symm_keep.append((t, hdl))
                    if self._flags is None:
                        self._make_flags(symm, gname)
                    torch.cuda.synchronize(self.device)
                    dist.barrier(group=self.group)  # nobody publishes into a vector that a peer is still clearing
                    return t
        return torch.zeros(self.n, dtype=self._dtype, device=self.device)

    def _make_flags(self, symm, gname) -> None:
        """Symmetric flag words of the barrier kernel (one slot per rank); on any failure the ranks keep
        the NCCL all-reduce as their barrier (agreed collectively)."""
        f = hdl = None
        try:
            f = symm.empty(64, dtype=torch.int32, device=self.device)
            f.zero_()
        except Exception:
            f = None
        if not self._all_agree(f is not None):
            return
        mc = 0
        try:
            hdl = symm.rendezvous(f, gname)
            mc = int(hdl.multicast_ptr)
        except Exception:
            mc = 0
        if not self._all_agree(mc != 0):
            return
        self._flags, self._flags_mc = f, mc
        self._status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._symm_keep.append((f, hdl))

    def use_native_loop(self, ctx, groups, max_polls: int = 0) -> bool:
        """Moves step_into() / iterate() behind the C ABI (asp_dist_create / asp_dist_spmv_iter): the same
        chunk kernels, store passes and barrier kernel, enqueued by one native call per iteration loop.
        `groups[c]` is the PlanGroup of the c-th chunk (None for a chunk without non-zeros). Only for the
        multicast exchange with the flag barrier (or a single rank); call it after the vectors were made
        and before the first step. Returns whether ALL ranks switched (agreed collectively)."""
        from . import capi

        self._native = None
        ok = self.world == 1 or (self._mode == "multicast" and self._flags is not None)
        loop = None
        if ok:
            try:
                base = self.bounds[self.rank]
                ch = [(g, base + lo, base + hi) for g, (_, lo, hi) in zip(groups, self.chunks)]
                loop = capi.DistLoop(ctx, ch, self.n, self.rank, self.world, self._dtype == torch.float64,
                                     self._flags.data_ptr() if self._flags is not None else 0, self._flags_mc or 0, max_polls)
            except Exception as e:
                self.native_error = repr(e)[:200]
                ok = False
        if self.world > 1 and not self._all_agree(ok):
            ok = False
        if ok:
            self._native = loop
        elif loop is not None:
            loop.close()
        return ok

    def _barrier(self) -> None:
        """All ranks' published rows are in every replica past this point (on the current stream)."""
        if self._flags is not None:
            from . import capi

            self._epoch += 1
            capi.rank_barrier(self._flags.data_ptr(), self._flags_mc, self.rank, self.world, self._epoch, self._status.data_ptr(),
                              torch.cuda.current_stream(self.device).cuda_stream)
        else:
            dist.all_reduce(self._flag, group=self.group)

    def check_barrier_status(self) -> None:
        """Raises if a barrier kernel gave up waiting for a rank (the wait is bounded by design)."""
        if getattr(self, "_native", None) is not None:
            self._native.status()  # raises AspError (status 7: a bounded wait expired)
        if self._status is not None and int(self._status.item()) != 0:
            raise RuntimeError(f"rank barrier timed out waiting for rank {int(self._status.item()) - 1}")

    # -- one SpMV of this rank's block, no communication -------------------------------------
    def spmv_slice(self, x: torch.Tensor) -> torch.Tensor:
        """y[bounds[rank]:bounds[rank+1]] for the replicated x."""
        for fn, lo, hi in self.chunks:
            if hi > lo:
                fn(x, self.y_local[lo:hi])
        return self.y_local[: self.rows[self.rank]]

    # -- exchange of chunk c: my rows span[rank][c] go to every peer, theirs come here -------
    def _exchange(self, c: int, x_next: torch.Tensor) -> None:
        me = self.rank
        src = x_next[self.span[me][c][0] : self.span[me][c][1]]
        if self._mode == "a2a":
            outs = [self._empty if p == me else x_next[self.span[p][c][0] : self.span[p][c][1]] for p in range(self.world)]
            ins = [self._empty if p == me else src for p in range(self.world)]
            dist.all_to_all(outs, ins, group=self.group)
        elif self._mode == "multicast":
            from . import capi

            mc = self._mc.get(x_next.data_ptr())
            if mc is None:
                raise ValueError("multicast exchange needs vectors from new_vector()")
            if src.numel():
                off = self.span[me][c][0] * src.element_size()
                capi.multicast_store(src.data_ptr(), mc + off, src.numel() * src.element_size(), torch.cuda.current_stream(self.device).cuda_stream, 0)
            if c == len(self.chunks) - 1:
                self._barrier()  # every rank's stores are done past this point
        elif self._mode == "allgather":
            outs = [x_next[self.span[p][c][0] : self.span[p][c][1]] for p in range(self.world)]
            dist.all_gather(outs, src, group=self.group)
        else:
            for p in range(self.world):
                seg = x_next[self.span[p][c][0] : self.span[p][c][1]]
                if seg.numel():
                    dist.broadcast(seg, src=p if self.group is None else dist.get_global_rank(self.group, p), group=self.group)

    def step_into(self, x: torch.Tensor, x_next: torch.Tensor) -> None:
        """x_next <- A x on every rank (replicated result)."""
        # (Running the chunks' kernels concurrently on prioritised streams was measured and lost:
        # the chunks then finish together and no exchange is hidden.)
        base = self.bounds[self.rank]
        if getattr(self, "_native", None) is not None:
            self._native.spmv(x.data_ptr(), x_next.data_ptr(), self._mc.get(x_next.data_ptr(), 0))
            return
        if self._mode == "publish":
            mc = self._mc.get(x_next.data_ptr())
            if mc is None:
                raise ValueError("the publishing exchange needs vectors from new_vector()")
            es = x_next.element_size()
            for (fn, lo, hi), pub in zip(self.chunks, self._pub):
                if hi > lo:
                    pub(x.data_ptr(), x_next.data_ptr() + (base + lo) * es, mc + (base + lo) * es)
            self._barrier()
            return
        cur = torch.cuda.current_stream(self.device) if self._comm is not None else None
        if getattr(self, "_whole_block_exchange", False):
            for fn, lo, hi in self.chunks:
                if hi > lo:
                    fn(x, x_next[base + lo : base + hi])
            self._exchange(0, x_next)
            return
        for c, (fn, lo, hi) in enumerate(self.chunks):
            if hi > lo:
                fn(x, x_next[base + lo : base + hi])
            if self.world == 1:
                continue
            if self._comm is not None:
                self._ev[c].record(cur)
                self._comm.wait_event(self._ev[c])
                with torch.cuda.stream(self._comm):
                    self._exchange(c, x_next)
            else:
                self._exchange(c, x_next)
        if self._comm is not None:
            self._done.record(self._comm)
            cur.wait_event(self._done)

    def iterate(self, x0: torch.Tensor, iters: int, scratch: torch.Tensor | None = None, scratch2: torch.Tensor | None = None) -> torch.Tensor:
        """x <- A x, `iters` times (square matrices); returns the final replicated x. With two scratch
        vectors x0 is only read (the results alternate between the two); with one, x0 itself is the
        second buffer and is overwritten from the second iteration on. The publishing exchange needs
        two, both from new_vector(): it relies on rows that are never written staying zero."""
        if scratch2 is not None and getattr(self, "_native", None) is not None:
            outs = (scratch, scratch2)
            last = self._native.iterate(x0.data_ptr(), [t.data_ptr() for t in outs], [self._mc.get(t.data_ptr(), 0) for t in outs], iters)
            return x0 if last < 0 else outs[last]
        if scratch2 is not None:
            a, outs = x0, (scratch, scratch2)
            for i in range(iters):
                self.step_into(a, outs[i & 1])
                a = outs[i & 1]
            return a
        if self._mode == "publish":
            raise ValueError("the publishing exchange needs two scratch vectors from new_vector()")
        a = x0
        b = scratch if scratch is not None else torch.empty_like(x0)
        for _ in range(iters):
            self.step_into(a, b)
            a, b = b, a
        return a


def all_ranks_ok(ok: bool, what: str, device="cpu", group=None) -> None:
    """Host-side agreement before the ranks enter a collective phase: every rank reports whether its
    own set-up (generation, lowering, upload) succeeded, and ALL ranks raise if any of them failed, so
    that a rank with an error never leaves the others waiting inside a collective. Call it with the
    local outcome on every rank (also on the failing one)."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        if not ok:
            raise RuntimeError(f"{what} failed on this rank")
        return
    t = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
    if int(t.item()) == 0:
        raise RuntimeError(f"{what} failed on " + ("this rank" if not ok else "another rank") + "; all ranks stop before the exchange")


def balanced_bounds_from_degrees(deg: np.ndarray, parts: int) -> np.ndarray:
    """Row bounds with about sum(deg) / parts non-zeros per part, from per-row counts."""
    from .graph import partition_rows_by_nnz

    indptr = np.zeros(deg.shape[0] + 1, dtype=np.int64)
    np.cumsum(deg, out=indptr[1:])
    return partition_rows_by_nnz(indptr, parts)
