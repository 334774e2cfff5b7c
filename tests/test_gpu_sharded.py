"""GPU suite, sharded repeated SpMV: row chunks with their own plan groups on one GPU, the GPU
R-MAT generator, and (where the box has two GPUs) every exchange form against the single-rank result."""
import os
import socket

import numpy as np
import pytest
import torch

import refdump
from alphasparse_b200 import bench_rmat, capi, matrices as M, matrices_gpu, tuner
from alphasparse_b200.dist import ShardedSpmv
from alphasparse_b200.graph import partition_rows_by_nnz

pytestmark = pytest.mark.gpu


def _chunks(ctx, blk, n_chunks, keep):
    cuts = partition_rows_by_nnz(blk.indptr, n_chunks)
    out = []
    for c in sorted(range(n_chunks), key=lambda c: -(int(cuts[c + 1]) - int(cuts[c]))):
        lo, hi = int(cuts[c]), int(cuts[c + 1])
        f, g = tuner.build(ctx, blk.row_slice(lo, hi), bench_rmat.DEFAULT_GRAPH if (c & 1) == 0 else bench_rmat.graph_with_tlb_size(16, sort=False))
        keep.append((f, g))

        def fn(xt, yt, g=g):
            g.spmv(xt.data_ptr(), yt.data_ptr(), True)

        def pub(xp, yp, mp, g=g):
            g.spmv_publish(xp, yp, mp)

        out.append((fn, lo, hi, pub))
    return out


def _reference_iterations(m, x, iters):
    ref = x.astype(np.float64)
    for _ in range(iters):
        ref, _ = refdump.csr_ref(m, ref.astype(np.float32))
    return ref


@pytest.mark.parametrize("loop", ["python", "native"])
def test_row_chunks_on_one_gpu_match_the_oracle(asp_ctx, loop):
    m, x = M.rmat(13, 16, seed=4)
    m.values *= 0.02
    keep = []
    chunks = _chunks(asp_ctx, m, 3, keep)
    stream = torch.cuda.ExternalStream(asp_ctx.stream)
    with torch.cuda.stream(stream):
        sh = ShardedSpmv(None, [0, m.n_rows], 0, 1, torch.float32, "cuda", chunks=chunks)
        if loop == "native":  # the same loop behind the C ABI (asp_dist_spmv_iter)
            assert sh.use_native_loop(asp_ctx, [g for _, g in keep])
        x0 = torch.from_numpy(x).cuda()
        y = sh.spmv_slice(x0).clone()
        xf = sh.iterate(x0, 3, sh.new_vector(), sh.new_vector())
        torch.cuda.synchronize()
    y_ref, scale = refdump.csr_ref(m, x)
    refdump.assert_y(y.cpu().numpy(), y_ref, scale, np.float32, "chunked slice")
    ref = _reference_iterations(m, x, 3)
    got = xf.cpu().numpy().astype(np.float64)
    assert np.max(np.abs(got - ref)) <= 1e-4 * max(1e-30, np.max(np.abs(ref)))
    for f, g in keep:
        g.close()
        f.close()


def test_gpu_rmat_blocks_do_not_depend_on_the_partition():
    dev = torch.device("cuda", 0)
    scale, ef, seed = 12, 8, 4
    n = 1 << scale
    ip, cols, vals = matrices_gpu.rmat_block(scale, ef, seed, 0, n, dev)
    whole = matrices_gpu.to_host_csr(ip, cols, vals, n)
    deg = matrices_gpu.rmat_row_degrees(scale, ef, seed, dev).cpu().numpy()
    assert deg.sum() == n * ef and np.all(deg >= whole.row_lengths())  # duplicates only ever merge
    cut = 700
    parts = [matrices_gpu.to_host_csr(*matrices_gpu.rmat_block(scale, ef, seed, a, b, dev), n) for a, b in ((0, cut), (cut, n))]
    assert parts[0].nnz + parts[1].nnz == whole.nnz
    assert np.array_equal(np.concatenate([parts[0].indices, parts[1].indices]), whole.indices)
    assert np.array_equal(np.concatenate([parts[0].values, parts[1].values]), whole.values)
    assert np.all(whole.values > 0) and np.all(whole.values <= 1)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _two_rank_matrix():
    # more than 65536 columns, so that the column indices are 32 bits wide (what the publishing kernels take)
    m, x = M.rmat(17, 8, seed=4)
    m.values *= 0.03
    return m, x


def _worker(rank, world, port, mode, out_dir):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    m, x = _two_rank_matrix()
    bounds = partition_rows_by_nnz(m.indptr, world)
    blk = m.row_slice(int(bounds[rank]), int(bounds[rank + 1]))
    ctx = capi.Context(rank)
    keep = []
    # the multicast forms pair nothing across ranks: every rank cuts its block as it likes
    native = mode == "native"
    mode = "multicast" if native else mode
    n_chunks = 2 if mode in ("allgather", "a2a") else (1 if rank == 0 else 3)
    chunks = _chunks(ctx, blk, n_chunks, keep)
    stream = torch.cuda.ExternalStream(ctx.stream)
    timed_out = None
    with torch.cuda.stream(stream):
        sh = ShardedSpmv(None, bounds, rank, world, torch.float32, torch.device("cuda", rank), chunks=chunks, exchange=mode)
        a, b = sh.new_vector(), sh.new_vector()
        went_native = native and sh.use_native_loop(ctx, [g for _, g in keep], max_polls=20000)
        x0 = torch.from_numpy(x).cuda()
        xf = sh.iterate(x0, 3, a, b)  # x0 is only read; the results alternate between a and b
        torch.cuda.synchronize()
        sh.check_barrier_status()
        if went_native:
            # one more SpMV on rank 0 alone: its barrier runs out (bounded wait) and asp_dist_status names rank 1
            xf = xf.clone()
            dist.barrier()
            if rank == 0:
                sh.step_into(x0, a)
                try:
                    sh.check_barrier_status()
                    timed_out = "no"
                except capi.AspError as e:
                    timed_out = str(e)
            dist.barrier()
        if mode == "publish" and sh._flags is not None:
            # a barrier that one rank never joins runs out (bounded wait) and reports which rank was missing
            dist.barrier()
            if rank == 0:
                sh._epoch += 1
                capi.rank_barrier(sh._flags.data_ptr(), sh._flags_mc, rank, world, sh._epoch, sh._status.data_ptr(), stream.cuda_stream, max_polls=20000)
                torch.cuda.synchronize()
                try:
                    sh.check_barrier_status()
                    timed_out = "no"
                except RuntimeError as e:
                    timed_out = str(e)
            dist.barrier()
    np.save(os.path.join(out_dir, f"final_{rank}.npy"), xf.cpu().numpy())
    with open(os.path.join(out_dir, f"mode_{rank}.txt"), "w") as fh:
        fh.write(f"{sh._mode};{'flags' if sh._flags is not None else 'nccl'};{timed_out};{'native' if native and went_native else 'python'}")
    del sh, a, b, xf
    for f, g in keep:
        g.close()
        f.close()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("mode", ["allgather", "a2a", "multicast", "publish", "native"])
def test_two_ranks_agree_with_one(mode, tmp_path):
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(2, _free_port(), mode, str(tmp_path)), nprocs=2, join=True)
    m, x = _two_rank_matrix()
    ref = _reference_iterations(m, x, 3)
    f0, f1 = np.load(tmp_path / "final_0.npy"), np.load(tmp_path / "final_1.npy")
    assert np.array_equal(f0.view(np.uint32), f1.view(np.uint32)), "the ranks' replicas of x differ"
    assert np.max(np.abs(f0.astype(np.float64) - ref)) <= 1e-4 * np.max(np.abs(ref))
    used = [open(tmp_path / f"mode_{r}.txt").read().split(";") for r in range(2)]
    assert used[0][0] == used[1][0], used
    if mode == "publish" and used[0][0] == "publish" and used[0][1] == "flags":
        assert "rank 1" in used[0][2], used  # rank 0 waited for rank 1 in vain, and said so
    if mode == "native" and used[0][3] == "native":
        assert used[1][3] == "native" and "status 7" in used[0][2] and "rank 1" in used[0][2], used


def _bench_args(**kw):
    import argparse

    d = dict(scale=13, iters=3, balance="6", chunks=0, exchange="multicast", graph=None, full_search=False, search=False, sort="auto", tlb=0, stage=False,
             cap_log2=0, generic_csr5=False, warmup=3, steps=1, loop="native", relabel="indegree", profile_launches=0)
    d.update(kw)
    return argparse.Namespace(**d)


def _close(r):
    torch.cuda.synchronize()
    for g in r["group"]:
        g.close()
    for f in r["fmt"]:
        f.close()


def test_graph_workload_with_and_without_relabelling_gives_the_same_vector():
    """The whole workload function on one GPU at a small scale: the loop on P A P^T (vertices renumbered by column
    count, x permuted in and out) returns what the loop on A returns, and both first SpMVs match the oracle."""
    check = lambda m, x, y: refdump.rel_err(y, *refdump.csr_ref(m, x))
    finals = {}
    for relabel in ("indegree", "none"):
        r = bench_rmat.run(_bench_args(relabel=relabel), 0, 1, 0, None, None, check_fn=check)
        assert r["parity"] <= refdump.TOL[np.dtype(np.float32)], (relabel, r["parity"])
        assert r["loop"].startswith("native")
        stream = torch.cuda.ExternalStream(r["ctx"].stream)
        with torch.cuda.stream(stream):
            finals[relabel] = r["iterate"](r["x0"], 3).clone()
        torch.cuda.synchronize()
        if relabel == "none":
            m, x = r["m_local"], r["x0"].cpu().numpy()
            ref = _reference_iterations(m, x, 3)
        _close(r)
    a, b = finals["indegree"].cpu().numpy().astype(np.float64), finals["none"].cpu().numpy().astype(np.float64)
    assert np.max(np.abs(a - ref)) <= 1e-4 * np.max(np.abs(ref))
    assert np.max(np.abs(b - ref)) <= 1e-4 * np.max(np.abs(ref))


def test_twenty_iterations_of_a_rescaled_graph_match_the_oracle(asp_ctx):
    """x <- A x twenty times on an R-MAT block whose values are scaled so that x neither overflows nor dies out
    (the bench's own values make x overflow after ~40 SpMVs, so its parity is checked on the first one): the native
    loop's last vector against twenty CPU SpMVs, each rounded to fp32 as the GPU rounds it."""
    m, x = M.rmat(13, 16, seed=4)
    m.values *= 1.0 / 8.0
    keep = []
    chunks = _chunks(asp_ctx, m, 3, keep)
    stream = torch.cuda.ExternalStream(asp_ctx.stream)
    with torch.cuda.stream(stream):
        sh = ShardedSpmv(None, [0, m.n_rows], 0, 1, torch.float32, "cuda", chunks=chunks)
        assert sh.use_native_loop(asp_ctx, [g for _, g in keep])
        x0 = torch.from_numpy(x).cuda()
        xf = sh.iterate(x0, 20, sh.new_vector(), sh.new_vector())
        torch.cuda.synchronize()
    ref = _reference_iterations(m, x, 20)
    got = xf.cpu().numpy().astype(np.float64)
    assert np.isfinite(ref).all() and np.max(np.abs(ref)) > 1e-20
    assert np.max(np.abs(got - ref)) <= 2e-4 * np.max(np.abs(ref))
    for f, g in keep:
        g.close()
        f.close()


def test_native_loop_clears_a_chunk_without_non_zeros(asp_ctx):
    """asp_dist_* straight through the binding: two chunks with plan groups and one without any non-zeros (no plan
    group: its rows are cleared every SpMV, also when the buffer held something else before)."""
    n = 3000
    lens = np.concatenate([np.random.default_rng(5).integers(1, 9, size=2000), np.zeros(400, dtype=np.int64), np.full(600, 3)])
    m, x = M.from_row_lengths(lens, n, seed=9)
    m.values *= 0.1
    parts = [(0, 2000), (2000, 2400), (2400, 3000)]
    built = [tuner.build(asp_ctx, m.row_slice(lo, hi), bench_rmat.graph_with_tlb_size(8, sort=False)) if m.indptr[hi] > m.indptr[lo] else (None, None) for lo, hi in parts]
    assert built[1] == (None, None)
    loop = capi.DistLoop(asp_ctx, [(g, lo, hi) for (f, g), (lo, hi) in zip(built, parts)], n)
    stream = torch.cuda.ExternalStream(asp_ctx.stream)
    with torch.cuda.stream(stream):
        x0 = torch.from_numpy(x).cuda()
        a, b = torch.full((n,), 7.0, device="cuda"), torch.full((n,), -3.0, device="cuda")  # dirty buffers
        last = loop.iterate(x0.data_ptr(), [a.data_ptr(), b.data_ptr()], None, 3)
        loop.status()
        torch.cuda.synchronize()
    assert last == 0
    ref = _reference_iterations(m, x, 3)
    got = a.cpu().numpy().astype(np.float64)
    assert np.all(got[2000:2400] == 0)
    assert np.max(np.abs(got - ref)) <= 1e-4 * np.max(np.abs(ref))
    # the same vector as x and y is refused
    with pytest.raises(capi.AspError):
        loop.spmv(a.data_ptr(), a.data_ptr())
    loop.close()
    for f, g in built:
        if g is not None:
            g.close()
            f.close()
