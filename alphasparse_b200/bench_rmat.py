"""The sharded graph workload of bench.py: R-MAT adjacency, nnz-balanced row blocks over the ranks,
x replicated, `iters` repeated SpMVs whose results reach every rank before the next one (strong
scaling: the matrix is the same at every N). Returns the fields bench.py prints.

Nothing here checks results: bench.py hands in `check_fn` (the CPU oracle lives with the tests) and
this module only calls it with the first SpMV's output.
"""
from __future__ import annotations

import time

import numpy as np
import torch

from . import capi, matrices_gpu, tuner
from .dist import ShardedSpmv, all_ranks_ok, balanced_bounds_from_degrees
from .graph import partition_rows_by_nnz

# One CSR5-like kernel over the block. The coarse row sort with a bin wider than any row is a stable
# partition: rows keep their order, rows without non-zeros go last, where the CSR5-like lowering
# drops them (it would otherwise store one explicit zero per empty row, and R-MAT blocks are up to
# half empty rows). y is still written in row order, so a row chunk of the block is a contiguous
# slice of the next x.
DEFAULT_GRAPH = {"dense": "dense sort 1073741824 | dense compress",
                 "subs": [{"graph": "S9_K9_s32", "nodes": ["tlb_nnz 32"], "template": "K9", "threads": 128, "row_reduce": 1}]}


def graph_with_tlb_size(s: int, sort: bool = True) -> dict:
    """The one-kernel graph with `s` non-zeros per thread. Without the one-bin sort every row, empty or not, is
    written (an empty row costs one stored zero), in row order and unpermuted: what the publishing kernels
    need to send a warp's rows as one contiguous run of 16-byte multicast stores."""
    return {"dense": DEFAULT_GRAPH["dense"] if sort else "dense compress",
            "subs": [{"graph": f"S9_K9_s{s}", "nodes": [f"tlb_nnz {s}"], "template": "K9", "threads": 128, "row_reduce": 1}]}


def run(args, rank: int, world: int, local_rank: int, dist, log, check_fn=None):
    dev = torch.device("cuda", local_rank)
    scale, ef, seed, iters = args.scale, 16, 4, args.iters
    n = 1 << scale
    t0 = time.perf_counter()
    # pass 1: per-row edge counts (every rank takes a share of the chunks), summed over ranks
    total = n * ef
    n_gen = (total + matrices_gpu.CHUNK - 1) // matrices_gpu.CHUNK
    relabel = getattr(args, "relabel", "indegree") == "indegree"
    deg, cdeg = matrices_gpu.rmat_degrees(scale, ef, seed, dev, chunk_ids=range(rank, n_gen, world), columns=relabel)
    if dist:
        dist.all_reduce(deg)
        if relabel:
            dist.all_reduce(cdeg)
    labels = inverse = None
    if relabel:
        # Vertices renumbered by how often their column is read (the same numbering on every rank and at every N:
        # it depends on the column counts only). The loop runs on P A P^T: x0 is permuted once on the way in, the
        # result once on the way out. With the hot entries of x contiguous, an L2 smaller than x (268 MB at scale
        # 26) keeps exactly the lines the gathers read; measured on row blocks of scale 26: 10-12 % less kernel time.
        # Vertices whose row is empty come last: that suffix of every vector stays zero (the vectors are created
        # zero-filled and nobody writes it), so it is neither computed nor exchanged.
        labels, inverse = matrices_gpu.hotness_labels(cdeg, deg)
        deg = deg[inverse]  # degrees of the relabelled rows
    del cdeg
    # "nnz": equal non-zeros per rank; "bytes": equal algorithmic bytes, i.e. a row weighs as much
    # as one non-zero (4 B of y + 4 B of row structure against 4 B value + 4 B index); a number w:
    # a row weighs w non-zeros
    import math

    row_weight = {"nnz": 0.0, "bytes": 1.0, "auto": 3.0 + 1.5 * math.log2(max(world, 2) / 2.0)}.get(args.balance)
    if row_weight is None:
        row_weight = float(args.balance)
    # (weights are scaled by 8 so that fractional row weights survive the integer prefix sums; rows
    # without non-zeros cost nothing: the format drops them)
    w8 = int(round(row_weight * 8))
    bounds = balanced_bounds_from_degrees((deg * 8 + (deg > 0) * w8).cpu().numpy(), world)
    n_active = int((deg > 0).sum().item()) if relabel else n  # relabelled: rows [n_active, n) have no non-zeros
    bounds[-1] = n_active
    del deg
    r0, r1 = int(bounds[rank]), int(bounds[rank + 1])
    # pass 2: this rank's row block (global columns), duplicates merged
    indptr, cols, vals = matrices_gpu.rmat_block(scale, ef, seed, r0, r1, dev, labels, inverse)
    nnz_local = int(indptr[-1].item())
    m = matrices_gpu.to_host_csr(indptr, cols, vals, n)
    del indptr, cols, vals
    torch.cuda.empty_cache()
    gen_s = time.perf_counter() - t0
    if log:
        log(f"rows [{r0}, {r1}) nnz {nnz_local} generated in {gen_s:.1f} s")

    exchange = args.exchange if world > 1 else "none"
    if args.chunks > 0:
        n_chunks = args.chunks
    elif exchange in ("publish", "none"):
        n_chunks = 1
    elif exchange == "multicast":
        # The store pass of a chunk costs in proportion to its rows, and only a rank's LAST pass is exposed: a rank
        # cuts its block into one chunk per 1/(2 world) of all rows it owns (nnz-balanced blocks of a skewed matrix
        # differ a hundred-fold in rows, so the hub ranks get one chunk and the rank with the sparse tail up to 8).
        n_chunks = int(min(8, max(1, -(-(r1 - r0) * 2 * world // n_active))))
    else:
        n_chunks = 2  # the pairwise exchanges pair the c-th chunks of all ranks
    ctx = capi.Context(local_rank)
    t0 = time.perf_counter()
    cuts = partition_rows_by_nnz(m.indptr, n_chunks)
    if args.graph:
        import json
        import os

        if os.path.exists(args.graph):
            cfg = json.load(open(args.graph))["config"]
            desc = cfg.get("graph", cfg.get("graph_rank0"))
        else:
            desc = json.loads(args.graph)
    elif args.full_search or args.search:
        # search on the chunk in the middle of the block, reuse its graph for the others
        mid = n_chunks // 2
        mc = m.row_slice(int(cuts[mid]), int(cuts[mid + 1]))
        fmt_, group_, _, desc = tuner.search(ctx, mc, quick=not args.full_search, log=log, warmup=1, reps=5)
        group_.close()
        del fmt_, group_, mc
    else:
        sort = args.sort != "no"  # (auto = yes: unpermuted rows were measured slower with every exchange form)
        desc = graph_with_tlb_size(args.tlb or 32, sort)
    fmts, groups, chunks, chunk_groups = [], [], [], []
    build_error = None
    # most rows first: with a separate store pass the exchange of the last chunk is the only one no kernel hides
    order = sorted(range(n_chunks), key=lambda c: -(int(cuts[c + 1]) - int(cuts[c])))
    for c in order:
        lo, hi = int(cuts[c]), int(cuts[c + 1])
        if hi == lo or m.indptr[hi] == m.indptr[lo]:
            # nothing to compute: the rows (if any) are zero
            def fz(xt, yt):
                yt.zero_()

            chunks.append((fz, lo, hi, (lambda xp, yp, mp: None)))
            chunk_groups.append(None)
            continue
        mc = m.row_slice(lo, hi) if n_chunks > 1 else m
        try:
            f, g = tuner.build(ctx, mc, desc)
            if args.stage or args.cap_log2 or args.generic_csr5:
                for i in range(g.n):
                    g.set_tuning(i, 0, (1 if args.stage else 0) | (2 if args.generic_csr5 else 0) | (args.cap_log2 << 4))
        except Exception as e:  # reported to every rank below, before anybody enters a collective
            build_error = e
            break
        fmts.append(f)
        groups.append(g)

        def fn(xt, yt, g=g):
            g.spmv(xt.data_ptr(), yt.data_ptr(), True)  # empty rows are never stored by a kernel: clear y

        def pub(xp, yp, mp, g=g):
            g.spmv_publish(xp, yp, mp)

        chunks.append((fn, lo, hi, pub))
        chunk_groups.append(g)
        del mc
    all_ranks_ok(build_error is None, f"lowering / upload of the row block ({build_error})", dev)
    search_s = time.perf_counter() - t0
    stream = torch.cuda.ExternalStream(ctx.stream)
    x0 = matrices_gpu.rmat_x(scale, seed, dev)  # the caller's x, in the matrix's own vertex numbering
    x0p = x0[inverse] if relabel else x0       # the same vector as the loop sees it
    x_in = torch.empty_like(x0) if relabel else None
    x_out = torch.empty_like(x0) if relabel else None

    with torch.cuda.stream(stream):
        sh = ShardedSpmv(None, bounds, rank, world, torch.float32, dev, chunks=chunks, exchange=args.exchange, n_total=n)
        xa = sh.new_vector()
        xb = sh.new_vector()
        native = getattr(args, "loop", "native") == "native" and build_error is None and sh.use_native_loop(ctx, chunk_groups, max_polls=20_000_000)  # (five times the default wait: a bench run shares its host with 7 other ranks)

        def iterate(x_caller, count):
            """x <- A x `count` times for a vector in the caller's numbering; returns the result in the same numbering."""
            if not relabel:
                return sh.iterate(x_caller, count, xa, xb)
            torch.index_select(x_caller, 0, inverse, out=x_in)
            xf = sh.iterate(x_in, count, xa, xb)
            torch.index_select(xf, 0, labels, out=x_out)
            return x_out
        # parity of the first SpMV of this rank's slice (the caller's checker; bounded sizes only)
        parity = None
        y1 = sh.spmv_slice(x0p).clone()
        torch.cuda.synchronize()
        if check_fn is not None:
            parity = check_fn(m, x0p.cpu().numpy(), y1.cpu().numpy())
        del y1
        if getattr(args, "profile_launches", 0):
            for _ in range(args.profile_launches):
                sh.spmv_slice(x0p)
            torch.cuda.synchronize()
            return {"profile_only": True, "nnz": nnz_local, "rows": n, "graph": desc, "format_bytes": int(sum(g.format_bytes() for g in groups))}
        W, K = max(args.warmup, 3), max(args.steps, 1)
        # the ranks enter the loop together: the barrier kernels wait for a late rank only for about a second, and the
        # parity check above takes a different time on every rank
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        for _ in range(W):
            iterate(x0, 2)
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        c0 = torch.cuda.Event(enable_timing=True)
        c1 = torch.cuda.Event(enable_timing=True)
        step_ev = [torch.cuda.Event(enable_timing=True) for _ in range(K + 1)]
        torch.cuda.synchronize()
        t_host0 = time.perf_counter()
        e0.record(stream)
        step_ev[0].record(stream)
        for k in range(K):
            iterate(x0, iters)  # x0 is only read: every step starts from the same vector
            step_ev[k + 1].record(stream)
        e1.record(stream)
        e1.synchronize()
        timed_wall_s = time.perf_counter() - t_host0
        ms_total = e0.elapsed_time(e1)
        per_step = [step_ev[k].elapsed_time(step_ev[k + 1]) for k in range(K)]
        sh.check_barrier_status()
        # compute-only time of the same number of local SpMVs (no exchange), for the breakdown
        c0.record(stream)
        for _ in range(iters):
            sh.spmv_slice(x0p)
        c1.record(stream)
        c1.synchronize()
        ms_compute = c0.elapsed_time(c1) / iters
        if log:
            log(f"rows {r1 - r0} nnz {nnz_local} chunks {n_chunks} compute-only {ms_compute:.4f} ms per SpMV; timed {ms_total / K / iters:.4f} ms per SpMV")
    nnz_total = torch.tensor([nnz_local], dtype=torch.int64, device=dev)
    t = torch.tensor([ms_total, ms_compute, float(np.median(per_step))], device=dev)
    if dist:
        dist.all_reduce(nnz_total)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t[0].item()) / K  # one step = `iters` repeated SpMVs
    nnz_all = int(nnz_total.item())
    launches = int(sum(g.launches() for g in groups))
    if sh._mode == "publish":
        launches = 3 * launches + 1  # clear end rows, compute + publish, send end rows; one barrier kernel per SpMV
    elif sh._mode == "multicast":
        launches = 2 * launches + (1 if sh._flags is not None else 0)
    out = {
        "ms_per_step": ms_step, "ms_per_spmv": ms_step / iters, "ms_compute_per_spmv_max": float(t[1].item()), "ms_per_step_median": float(t[2].item()),
        "gflops": 2.0 * nnz_all * iters / (ms_step * 1e-3) * 1e-9, "nnz": nnz_all, "rows": n, "iters": iters, "graph": desc,
        "search_s": search_s, "gen_s": gen_s, "parity": parity, "rows_local": r1 - r0, "nnz_local": nnz_local, "timed_wall_s": timed_wall_s,
        "format_bytes": int(sum(g.format_bytes() for g in groups)), "launches_per_spmv": launches, "chunks": n_chunks, "exchange_used": sh._mode if world > 1 else "none", "loop": "native (asp_dist_spmv_iter)" if native else "python",
        "fallback_reason": getattr(sh, "fallback_reason", None), "barrier": "flag kernel" if sh._flags is not None else ("nccl all_reduce" if world > 1 else "none"),
        "end_rows_local": int(sum(g.end_rows() for g in groups)), "staged": bool(args.stage),
        "m_local": m, "group": groups, "ctx": ctx, "x0": x0, "sharded": sh, "fmt": fmts, "bufs": (xa, xb, x_in, x_out), "iterate": iterate,
        "relabel": "vertices renumbered by column count (P A P^T), x permuted in and out inside every step" if relabel else "none",
        "labels": (labels, inverse),
    }
    return out
