"""CPU suite: renumbering the vertices of the graph workload by column count gives P A P^T, the same edges and
values under new numbers (the generator runs on the CPU here; its streams differ from the GPU's, the logic does not)."""
import numpy as np
import pytest
import scipy.sparse as sp
import torch

import plan_interp
import refdump
from alphasparse_b200 import matrices as M, matrices_gpu
from alphasparse_b200.graph import Matrix
from native_manifest import NativeManifest


def _csr(ip, cols, vals, n):
    return sp.csr_matrix((vals.numpy(), cols.numpy(), ip.numpy()), shape=(ip.shape[0] - 1, n))


def test_hotness_labels_sort_by_count_and_keep_ties_in_order():
    cnt = torch.tensor([3, 9, 3, 0, 9, 1])
    labels, inverse = matrices_gpu.hotness_labels(cnt)
    assert inverse.tolist() == [1, 4, 0, 2, 5, 3]
    assert labels.tolist() == [2, 0, 3, 5, 1, 4]
    assert torch.equal(labels[inverse], torch.arange(6))
    # vertices whose row is empty go last, in the same order among themselves
    labels, inverse = matrices_gpu.hotness_labels(cnt, torch.tensor([1, 0, 2, 5, 0, 0]))
    assert inverse.tolist() == [0, 2, 3, 1, 4, 5]
    assert torch.equal(labels[inverse], torch.arange(6))


def test_relabelled_blocks_are_the_permuted_matrix():
    scale, ef, seed = 9, 8, 4
    n = 1 << scale
    dev = torch.device("cpu")
    deg, cdeg = matrices_gpu.rmat_degrees(scale, ef, seed, dev)
    assert int(deg.sum()) == int(cdeg.sum()) == n * ef
    assert torch.equal(deg, matrices_gpu.rmat_row_degrees(scale, ef, seed, dev))
    labels, inverse = matrices_gpu.hotness_labels(cdeg, deg)
    n_active = int((deg > 0).sum())
    a = _csr(*matrices_gpu.rmat_block(scale, ef, seed, 0, n, dev), n)
    # the relabelled matrix, generated in two row blocks
    cut = 100
    parts = [_csr(*matrices_gpu.rmat_block(scale, ef, seed, r0, r1, dev, labels, inverse), n) for r0, r1 in ((0, cut), (cut, n))]
    b = sp.vstack(parts).tocsr()
    assert b.nnz == a.nnz
    assert n_active < n and b[n_active:].nnz == 0 and np.all(np.diff(b.indptr)[:n_active] > 0)  # the empty rows are the suffix
    # b[labels[i], labels[j]] == a[i, j]
    lab = labels.numpy()
    back = b[lab][:, lab]
    assert (back != a).nnz == 0
    # the hottest column of the original matrix is column 0 of the relabelled one, and column counts never increase
    col_counts = np.asarray((b != 0).sum(axis=0)).ravel()
    assert col_counts[0] >= col_counts[:n_active].max() - 2  # (counts before duplicates merge decide the order)
    # x permuted the same way gives the permuted product
    x = matrices_gpu.rmat_x(scale, seed, dev).numpy().astype(np.float64)
    y = a.astype(np.float64) @ x
    yp = b.astype(np.float64) @ x[inverse.numpy()]
    assert np.allclose(yp[lab], y, rtol=1e-12, atol=0)


@pytest.mark.parametrize("empty_last", [True, False])
def test_host_operator_renumbers_a_matrix_and_the_lowered_format_gives_the_permuted_product(empty_last):
    """asp_matrix_relabel_by_column_count on a host matrix: the result, lowered by the ordinary operators and walked
    the way the kernels walk it, is P A P^T: y'[labels[v]] = (A x)[v] for x'[labels[v]] = x[v]."""
    m, x = M.rmat(10, 8, seed=4)
    hm = Matrix.from_csr(m)
    m2, labels, n_active = hm.relabel_by_column_count(empty_last)
    lens = m.row_lengths()
    assert n_active == int((lens > 0).sum()) and m2.nnz == m.nnz and m2.shape == (m.n_rows, m.n_cols)
    assert sorted(labels.tolist()) == list(range(m.n_rows))
    counts = np.bincount(m.indices, minlength=m.n_cols)
    inverse = np.argsort(labels)
    if empty_last:
        assert np.all(lens[inverse[:n_active]] > 0) and np.all(lens[inverse[n_active:]] == 0)
        assert np.all(np.diff(counts[inverse[:n_active]]) <= 0) and np.all(np.diff(counts[inverse[n_active:]]) <= 0)
    else:
        assert np.all(np.diff(counts[inverse]) <= 0)  # most frequent column first
    fmt = m2.execute("dense compress\nsub all tlb_nnz 8\nsub all template K9")
    xp = np.zeros_like(x, dtype=np.float64)
    xp[labels] = x
    yp = plan_interp.interpret(NativeManifest(fmt, m.n_rows), xp)
    y_ref, scale = refdump.csr_ref(m, x)
    assert refdump.rel_err(yp[labels], y_ref, scale) <= 1e-12
    fmt.close()
    m2.close()
    # a matrix that already went through a dense-view node is refused
    cm = hm.dense("dense sort 1\ndense compress")
    with pytest.raises(Exception):
        cm.relabel_by_column_count()
    cm.close()
    hm.close()


def test_host_operator_on_random_matrices_with_empty_rows_and_unused_columns():
    """Drawn matrices (fp64, rows without non-zeros, columns nobody reads, one long row): labels are a permutation,
    P A P^T has the same multiset of values per relabelled row, and the product commutes with the permutation."""
    rng = np.random.default_rng(11)
    for trial in range(6):
        n = int(rng.integers(40, 400))
        lens = rng.integers(0, 7, size=n)
        lens[rng.integers(0, n)] = n // 2  # one long row
        lens[rng.integers(0, n, size=n // 5)] = 0
        if lens.sum() == 0:
            lens[0] = 3
        m, x = M.from_row_lengths(lens, n, seed=100 + trial, dtype=np.float64)
        hm = Matrix.from_csr(m)
        m2, labels, n_active = hm.relabel_by_column_count(True)
        assert sorted(labels.tolist()) == list(range(n)) and n_active == int((lens > 0).sum())
        fmt = m2.execute("dense compress\nsub all tlb_nnz 4\nsub all template K9")
        xp = np.zeros(n)
        xp[labels] = x
        yp = plan_interp.interpret(NativeManifest(fmt, n), xp)
        y_ref, scale = refdump.csr_ref(m, x)
        assert refdump.rel_err(yp[labels], y_ref, scale) <= 1e-12
        assert np.all(yp[n_active:] == 0)
        fmt.close()
        m2.close()
        hm.close()
