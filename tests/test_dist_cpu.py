"""CPU suite, part 5: the multi-GPU plumbing with gloo ranks on the host.

The product's local SpMV needs a GPU; here each rank's slice is computed by the CPU oracle (test
infrastructure) so that partitioning, the uneven all-gather and the repeated-SpMV loop are checked
against the single-rank result."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import refdump
from alphasparse_b200 import matrices as M
from alphasparse_b200.dist import ShardedSpmv, all_ranks_ok, balanced_bounds_from_degrees
from alphasparse_b200.graph import partition_rows_by_nnz


def test_partition_balances_nnz_and_covers_all_rows():
    m, _ = M.power_law(50000, 2.1, 3000, seed=2)
    for parts in (1, 2, 3, 4, 8):
        b = partition_rows_by_nnz(m.indptr, parts)
        assert b[0] == 0 and b[-1] == m.n_rows and np.all(np.diff(b) >= 0)
        per = np.diff(m.indptr[b])
        assert per.sum() == m.nnz
        assert per.max() - per.min() <= 2 * m.row_lengths().max()  # each cut is off by at most one row
    deg = m.row_lengths()
    assert np.array_equal(balanced_bounds_from_degrees(deg, 4), partition_rows_by_nnz(m.indptr, 4))


def test_partition_with_more_parts_than_rows_with_nonzeros():
    m, _ = M.rmat(6, 2, seed=1)
    b = partition_rows_by_nnz(m.indptr, 8)
    assert b[0] == 0 and b[-1] == m.n_rows and np.all(np.diff(b) >= 0)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, iters, out_dir, n_chunks=1):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    m, x = M.rmat(10, 8, seed=4)  # has empty rows; values in (0, 1]
    m.values *= 0.05  # keep x <- A x from overflowing in a few iterations
    bounds = partition_rows_by_nnz(m.indptr, world)
    blk = m.row_slice(int(bounds[rank]), int(bounds[rank + 1]))

    def make(sub):
        def fn(xt, yt):
            assert yt.shape[0] == sub.n_rows
            yt.copy_(torch.from_numpy(refdump.csr_native(sub, xt.numpy())))

        return fn

    if n_chunks == 1:
        sh = ShardedSpmv(make(blk), bounds, rank, world, torch.float32, "cpu")
    else:
        cuts = partition_rows_by_nnz(blk.indptr, n_chunks)
        order = sorted(range(n_chunks), key=lambda c: -(int(cuts[c + 1]) - int(cuts[c])))  # most rows first
        chunks = [(make(blk.row_slice(int(cuts[c]), int(cuts[c + 1]))), int(cuts[c]), int(cuts[c + 1])) for c in order]
        sh = ShardedSpmv(None, bounds, rank, world, torch.float32, "cpu", chunks=chunks)
    xt = torch.from_numpy(x.copy())
    y_slice = sh.spmv_slice(xt).clone()
    xf = sh.iterate(xt, iters)
    np.save(os.path.join(out_dir, f"slice_{rank}.npy"), y_slice.numpy())
    np.save(os.path.join(out_dir, f"final_{rank}.npy"), xf.numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,n_chunks", [(2, 1), (3, 1), (2, 3)])
def test_sharded_repeated_spmv_matches_single_rank(world, n_chunks, tmp_path):
    iters = 4
    mp.spawn(_worker, args=(world, _free_port(), iters, str(tmp_path), n_chunks), nprocs=world, join=True)
    m, x = M.rmat(10, 8, seed=4)
    m.values *= 0.05
    ref = x.copy()
    first = refdump.csr_native(m, ref)
    for _ in range(iters):
        ref = refdump.csr_native(m, ref)
    bounds = partition_rows_by_nnz(m.indptr, world)
    for r in range(world):
        sl = np.load(tmp_path / f"slice_{r}.npy")
        assert np.array_equal(sl, first[bounds[r] : bounds[r + 1]])
        assert np.array_equal(np.load(tmp_path / f"final_{r}.npy"), ref)


def _failing_worker(rank, world, port, out_dir):
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    ok = True
    try:
        if rank == 1:
            raise ValueError("injected: this rank cannot build its block")  # the failure is made on the host
    except ValueError:
        ok = False
    outcome = "entered the exchange"
    try:
        all_ranks_ok(ok, "set-up")
        # only reached when every rank is fine: the collective phase
        t = torch.ones(4)
        dist.all_reduce(t)
    except RuntimeError as e:
        outcome = "stopped: " + str(e)
    with open(os.path.join(out_dir, f"outcome_{rank}.txt"), "w") as fh:
        fh.write(outcome)
    dist.destroy_process_group()


def test_a_failing_rank_stops_all_ranks_before_the_collective(tmp_path):
    world = 3
    mp.spawn(_failing_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    outcomes = [open(tmp_path / f"outcome_{r}.txt").read() for r in range(world)]
    assert all(o.startswith("stopped:") for o in outcomes), outcomes
    assert "this rank" in outcomes[1] and "another rank" in outcomes[0] and "another rank" in outcomes[2]


def test_all_ranks_ok_without_a_process_group():
    all_ranks_ok(True, "nothing")
    with pytest.raises(RuntimeError):
        all_ranks_ok(False, "single process")


def _symm_failure_worker(rank, world, port, out_dir):
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    bounds = [0, 5, 12]
    sh = ShardedSpmv(lambda xt, yt: yt.copy_(xt[bounds[rank] : bounds[rank + 1]] * 2.0), bounds, rank, world, torch.float32, "cpu")
    # put the object in the state an NCCL run starts in, with the local allocation replaced by one that
    # fails on rank 1 only (out of memory, a missing module: anything that happens on one host)
    sh._mode = "multicast"

    def alloc():
        if rank == 1:
            raise MemoryError("injected: symmetric allocation failed on this rank")
        raise AssertionError("rank 0 must not go on to the rendezvous alone")

    if rank == 1:
        sh._symm_alloc = alloc
    else:
        # rank 0's allocation would succeed; it must still drop to the fallback because rank 1 could not
        sh._symm_alloc = lambda: (None, None, torch.empty(12))
    v = sh.new_vector()
    xt = torch.arange(12, dtype=torch.float32)
    want = (xt * 4).tolist()  # (iterate reuses x0 as one of its two buffers)
    out = sh.iterate(xt, 2)
    with open(os.path.join(out_dir, f"mode_{rank}.txt"), "w") as fh:
        fh.write(f"{sh._mode};{getattr(sh, 'fallback_reason', '')};{out.tolist() == want};{v.shape[0]}")
    dist.destroy_process_group()


def _unequal_chunks_worker(rank, world, port, out_dir):
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    bounds = [0, 5, 12]
    base = bounds[rank]

    def piece(lo, hi):
        return (lambda xt, yt: yt.copy_(xt[base + lo : base + hi] * 3.0), lo, hi)

    # rank 0 computes its block in one piece, rank 1 in three: a pairwise exchange cannot pair them
    chunks = [piece(0, 5)] if rank == 0 else [piece(2, 7), piece(0, 2), piece(7, 7)]
    sh = ShardedSpmv(None, bounds, rank, world, torch.float32, "cpu", chunks=chunks)
    xt = torch.arange(12, dtype=torch.float32)
    out = sh.iterate(xt.clone(), 2, sh.new_vector(), sh.new_vector())
    with open(os.path.join(out_dir, f"whole_{rank}.txt"), "w") as fh:
        fh.write(f"{out.tolist() == (xt * 9).tolist()};{getattr(sh, '_whole_block_exchange', False)}")
    dist.destroy_process_group()


def _suffix_worker(rank, world, port, out_dir):
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    bounds = [0, 5, 9]  # rows 9..11 belong to nobody: they have no non-zeros and stay zero in every vector
    sh = ShardedSpmv(lambda xt, yt: yt.copy_(xt[bounds[rank] : bounds[rank + 1]] * 2.0 + xt[11]), bounds, rank, world, torch.float32, "cpu", n_total=12)
    a, b = sh.new_vector(), sh.new_vector()
    xt = torch.arange(12, dtype=torch.float32)
    out = sh.iterate(xt, 2, a, b)
    # first SpMV: y[i] = 2 x[i] + x[11] for i < 9, 0 beyond; second: the suffix of its input is zero
    want = [(2.0 * (2.0 * i + 11.0)) for i in range(9)] + [0.0, 0.0, 0.0]
    with open(os.path.join(out_dir, f"suffix_{rank}.txt"), "w") as fh:
        fh.write(f"{out.tolist() == want};{a.shape[0]};{xt.tolist() == list(range(12))}")
    dist.destroy_process_group()


def test_rows_beyond_the_last_block_stay_zero(tmp_path):
    world = 2
    mp.spawn(_suffix_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert [open(tmp_path / f"suffix_{r}.txt").read() for r in range(world)] == ["True;12;True"] * 2


def test_ranks_with_different_chunk_counts_exchange_whole_blocks(tmp_path):
    world = 2
    mp.spawn(_unequal_chunks_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert [open(tmp_path / f"whole_{r}.txt").read() for r in range(world)] == ["True;True"] * 2


def test_a_local_allocation_failure_makes_every_rank_fall_back_together(tmp_path):
    world = 2
    mp.spawn(_symm_failure_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    modes = [open(tmp_path / f"mode_{r}.txt").read().split(";") for r in range(world)]
    assert modes[0][0] == modes[1][0] == "bcast_loop", modes
    assert "injected" in modes[1][1] and "another rank" in modes[0][1], modes
    assert modes[0][2] == modes[1][2] == "True" and modes[0][3] == "12"
