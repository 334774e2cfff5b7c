"""The sharded graph workload of bench.py: R-MAT adjacency, nnz-balanced row blocks over the ranks,
x replicated, `iters` repeated SpMVs with an all-gather of y into the next x (strong scaling: the
matrix is the same at every N). Returns the fields bench.py prints."""
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
# half empty rows). y is still written in nearly row order, so a row chunk of the block is a
# contiguous slice of the next x.
DEFAULT_GRAPH = {"dense": "dense sort 1073741824 | dense compress",
                 "subs": [{"graph": "S9_K9_s32", "nodes": ["tlb_nnz 32"], "template": "K9", "threads": 128, "row_reduce": 1}]}


def run(args, rank: int, world: int, local_rank: int, dist, log):
    dev = torch.device("cuda", local_rank)
    scale, ef, seed, iters = args.scale, 16, 4, args.iters
    n = 1 << scale
    t0 = time.perf_counter()
    # pass 1: per-row edge counts (every rank takes a share of the chunks), summed over ranks
    total = n * ef
    n_chunks = (total + matrices_gpu.CHUNK - 1) // matrices_gpu.CHUNK
    deg = matrices_gpu.rmat_row_degrees(scale, ef, seed, dev, chunk_ids=range(rank, n_chunks, world))
    if dist:
        dist.all_reduce(deg)
    # "nnz": equal non-zeros per rank; "bytes": equal algorithmic bytes, i.e. a row weighs as much
    # as one non-zero (4 B of y + 4 B of row structure against 4 B value + 4 B index)
    row_weight = {"nnz": 0.0, "bytes": 1.0}.get(args.balance)
    if row_weight is None:
        row_weight = float(args.balance)  # a row weighs this many non-zeros
    # (weights are scaled by 8 so that fractional row weights survive the integer prefix sums)
    bounds = balanced_bounds_from_degrees((deg * 8 + int(round(row_weight * 8))).cpu().numpy(), world)
    del deg
    r0, r1 = int(bounds[rank]), int(bounds[rank + 1])
    # pass 2: this rank's row block (global columns), duplicates merged
    indptr, cols, vals = matrices_gpu.rmat_block(scale, ef, seed, r0, r1, dev)
    nnz_local = int(indptr[-1].item())
    m = matrices_gpu.to_host_csr(indptr, cols, vals, n)
    del indptr, cols, vals
    torch.cuda.empty_cache()
    gen_s = time.perf_counter() - t0
    if log:
        log(f"rows [{r0}, {r1}) nnz {nnz_local} generated in {gen_s:.1f} s")

    n_chunks = max(1, args.chunks if args.chunks > 0 else (2 if world > 1 else 1))
    ctx = capi.Context(local_rank)
    t0 = time.perf_counter()
    # row chunks of this rank's block (nnz-balanced), one plan group each: chunk c is exchanged
    # while chunk c+1 is computed
    if args.chunk_shape == "geometric" and n_chunks > 1:
        # chunk c (in row order) holds 2^c shares of the block's non-zeros: the chunk that is
        # computed and published last is the smallest, so the exposed exchange is short
        tot = float(m.indptr[-1])
        fr = [(2.0 ** (c + 1) - 1.0) / (2.0 ** n_chunks - 1.0) for c in range(n_chunks - 1)]
        cuts = np.array([0] + [int(np.searchsorted(m.indptr, f * tot, side="left")) for f in fr] + [m.n_rows], dtype=np.int64)
        cuts = np.maximum.accumulate(cuts)
    else:
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
        desc = DEFAULT_GRAPH
    fmts, groups, chunks = [], [], []
    build_error = None
    # most rows first: the exchange of the last chunk is the only one no kernel hides
    order = sorted(range(n_chunks), key=lambda c: -(int(cuts[c + 1]) - int(cuts[c])))
    if args.chunk_shape == "geometric":
        order = list(range(n_chunks - 1, -1, -1))  # the big tail chunk first, the small head chunk last
    for c in order:
        lo, hi = int(cuts[c]), int(cuts[c + 1])
        if hi == lo or m.indptr[hi] == m.indptr[lo]:
            # nothing to compute: the rows (if any) stay zero; still a chunk so that every rank has as many
            def fz(xt, yt):
                yt.zero_()

            chunks.append((fz, lo, hi))
            continue
        mc = m.row_slice(lo, hi) if n_chunks > 1 else m
        try:
            f, g = tuner.build(ctx, mc, desc)
        except Exception as e:  # reported to every rank below, before anybody enters a collective
            build_error = e
            break
        fmts.append(f)
        groups.append(g)

        def fn(xt, yt, g=g):
            g.spmv(xt.data_ptr(), yt.data_ptr(), True)  # empty rows are never stored by a kernel: clear y

        chunks.append((fn, lo, hi))
        del mc
    all_ranks_ok(build_error is None, f"lowering / upload of the row block ({build_error})", dev)
    search_s = time.perf_counter() - t0
    stream = torch.cuda.ExternalStream(ctx.stream)
    x0 = matrices_gpu.rmat_x(scale, seed, dev)

    with torch.cuda.stream(stream):
        sh = ShardedSpmv(None, bounds, rank, world, torch.float32, dev, chunks=chunks, exchange=args.exchange)
        xa = sh.new_vector()
        xb = sh.new_vector()
        xa.copy_(x0)
        # parity of the first SpMV of this rank's slice against the CPU oracle (bounded sizes only)
        parity = None
        y1 = sh.spmv_slice(x0).clone()
        torch.cuda.synchronize()
        if True:
            import os
            import sys

            sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "tests"))
            import refdump

            # the CPU oracle checks whole blocks up to 3e8 non-zeros, else three row windows of the
            # block (head, middle, tail) of about 2e7 non-zeros each
            xh, yh = x0.cpu().numpy(), y1.cpu().numpy()
            if m.nnz <= 300_000_000:
                windows = [(0, m.n_rows)]
            else:
                windows = []
                for frac in (0.0, 0.5, 1.0):
                    target = int(frac * (m.nnz - 20_000_000))
                    a = int(np.searchsorted(m.indptr, target, side="left"))
                    b = int(np.searchsorted(m.indptr, target + 20_000_000, side="right")) - 1
                    windows.append((min(a, m.n_rows - 1), max(min(b, m.n_rows), min(a, m.n_rows - 1) + 1)))
            parity = 0.0
            for a, b in windows:
                sub = m.row_slice(a, b) if (a, b) != (0, m.n_rows) else m
                y_ref, scl = refdump.csr_ref(sub, xh)
                parity = max(parity, refdump.rel_err(yh[a:b], y_ref, scl))
        W, K = max(args.warmup, 3), max(args.steps, 1)
        for _ in range(W):
            sh.step_into(xa, xb)
        torch.cuda.synchronize()
        if dist:
            dist.barrier()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        c0 = torch.cuda.Event(enable_timing=True)
        c1 = torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(K):
            xa.copy_(x0)
            sh.iterate(xa, iters, xb)
        e1.record(stream)
        e1.synchronize()
        ms_total = e0.elapsed_time(e1)
        # compute-only time of the same number of local SpMVs (no exchange), for the breakdown
        c0.record(stream)
        for _ in range(iters):
            sh.spmv_slice(x0)
        c1.record(stream)
        c1.synchronize()
        ms_compute = c0.elapsed_time(c1) / iters
    nnz_total = torch.tensor([nnz_local], dtype=torch.int64, device=dev)
    t = torch.tensor([ms_total, ms_compute], device=dev)
    if dist:
        dist.all_reduce(nnz_total)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t[0].item()) / K  # one step = `iters` repeated SpMVs
    nnz_all = int(nnz_total.item())
    out = {
        "ms_per_step": ms_step, "ms_per_spmv": ms_step / iters, "ms_compute_per_spmv_max": float(t[1].item()),
        "gflops": 2.0 * nnz_all * iters / (ms_step * 1e-3) * 1e-9, "nnz": nnz_all, "rows": n, "iters": iters, "graph": desc,
        "search_s": search_s, "gen_s": gen_s, "parity": parity, "rows_local": r1 - r0, "nnz_local": nnz_local,
        "format_bytes": int(sum(g.format_bytes() for g in groups)), "launches_per_spmv": int(sum(g.launches() for g in groups)), "chunks": n_chunks, "exchange_used": sh._mode,
        "m_local": m, "group": groups, "ctx": ctx, "x0": x0, "sharded": sh, "fmt": fmts,
    }
    return out
