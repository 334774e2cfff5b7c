"""The diagonal-value operator (`diag_value` + template D1): DIA storage for matrices on a few diagonals.

Not an operator of the reference (its formats carry one column index per non-zero, also where the index is a closed
form of the row), so there is no reference array to compare with: the CPU tests read the stored arrays back with the
layout the header documents and compare the matrix they describe with the original; the GPU tests compare the kernel
with the CPU oracle, at the full size of the benchmark's Laplacian too.
"""
import numpy as np
import pytest

import refdump
from alphasparse_b200 import capi, matrices as M
from alphasparse_b200.graph import Format, Matrix

SPEC = "dense compress\nsub all diag_value\nsub all template D1"


def banded(n, offsets, seed, dtype=np.float64, holes=0.0):
    rng = np.random.default_rng(seed)
    rows, cols = [], []
    for r in range(n):
        for o in offsets:
            c = r + o
            if 0 <= c < n and rng.random() >= holes:
                rows.append(r)
                cols.append(c)
    rows, cols = np.array(rows), np.array(cols)
    order = np.lexsort((cols, rows))
    rows, cols = rows[order], cols[order]
    indptr = np.zeros(n + 1, dtype=np.int64)
    np.add.at(indptr, rows + 1, 1)
    return M.CsrMatrix(n, n, np.cumsum(indptr), cols.astype(np.uint32), rng.standard_normal(rows.shape[0]).astype(dtype)), rng.uniform(-1, 1, n).astype(dtype)


def dense_from_arrays(fmt, n_rows, n_cols):
    d = fmt.plan_descs()[0]
    a = fmt.arrays(0)
    off, val = a["col_index_arr"][0].astype(np.int64) - n_cols, a["val_arr"][0]
    D = int(d.tlb_size)
    NR = val.shape[0] // D
    A = np.zeros((n_rows, n_cols))
    for k in range(D):
        for r in range(n_rows):
            c = r + int(off[k])
            if 0 <= c < n_cols:
                A[r, c] = val[k * NR + r]
            else:
                assert val[k * NR + r] == 0
    return A


@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("holes", [0.0, 0.2])
def test_stored_diagonals_describe_the_matrix(dtype, holes):
    m, _ = banded(203, (-17, -1, 0, 1, 17, 40), seed=3, dtype=dtype, holes=holes)
    fmt = Matrix.from_csr(m).execute(SPEC)
    d = fmt.plan_descs()[0]
    assert d.template_type == capi.TEMPLATE["D1"] and d.tlb_size == 6 and d.effective_num == 203
    A = dense_from_arrays(fmt, 203, 203)
    ref = np.zeros_like(A)
    for r in range(203):
        ref[r, m.indices[m.indptr[r] : m.indptr[r + 1]]] = m.values[m.indptr[r] : m.indptr[r + 1]]
    assert np.array_equal(A, ref)
    capi.validate_descs(fmt.plan_descs())
    fmt.close()


def test_laplacian_stores_five_diagonals_and_no_index_per_entry():
    m, _ = M.laplacian_2d(64, 1)
    fmt = Matrix.from_csr(m).execute(SPEC)
    a = fmt.arrays(0)
    assert a["col_index_arr"][3] == 5 and sorted((a["col_index_arr"][0].astype(np.int64) - m.n_cols).tolist()) == [-64, -1, 0, 1, 64]
    assert fmt.padding_rate(0) < 1.03
    fmt.close()


def test_rejections_and_file_round_trip(tmp_path):
    m, _ = M.uniform_random(500, 6, seed=2)
    with pytest.raises(capi.AspError) as e:
        Matrix.from_csr(m).execute(SPEC)
    assert "diagonals" in str(e.value)
    lap, _ = M.laplacian_2d(40, 1)
    for bad, needle in (("dense compress\nsub all diag_value\nsub all template K3", "go together"), ("dense sort 1\ndense compress\nsub all diag_value\nsub all template D1", "sorted")):
        with pytest.raises(capi.AspError) as e:
            Matrix.from_csr(lap).execute(bad)
        assert needle in str(e.value)
    fmt = Matrix.from_csr(lap).execute(SPEC)
    p = str(tmp_path / "d.asp")
    fmt.save(p)
    back = Format.load(p)
    for name in ("val_arr", "col_index_arr"):
        assert np.array_equal(fmt.arrays(0)[name][0], back.arrays(0)[name][0])
    capi.validate_descs(back.plan_descs())
    back.close()
    fmt.close()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("n,offsets,holes", [(20001, (-300, -1, 0, 1, 300), 0.0), (9999, (-2000, -7, -1, 0, 2, 5, 1999, 5000), 0.3), (1003, (0,), 0.0)])
def test_kernel_matches_oracle(asp_ctx, n, offsets, holes, dtype):
    m, x = banded(n, offsets, seed=n % 97, dtype=dtype, holes=holes)
    fmt = Matrix.from_csr(m).execute(SPEC)
    g = fmt.upload(asp_ctx)
    y_ref, scale = refdump.csr_ref(m, x)
    for threads in (256, 64):
        g.set_launch(0, 1, threads, 1)
        refdump.assert_y(g.spmv_host(x), y_ref, scale, dtype, f"diagonals {offsets} threads {threads}")
    g.close()
    fmt.close()


@pytest.mark.gpu
def test_benchmark_laplacian_at_full_size(asp_ctx):
    m, x = M.laplacian_2d(2048, 1)
    fmt = Matrix.from_csr(m).execute(SPEC)
    g = fmt.upload(asp_ctx)
    y_ref, scale = refdump.csr_ref(m, x)
    refdump.assert_y(g.spmv_host(x), y_ref, scale, np.float64, "config 2 on five diagonals")
    g.close()
    fmt.close()
