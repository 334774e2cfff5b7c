"""The block-value operator (`block_value r c` + template B1): blocked ELL over dense r x c blocks.

Not an operator of the reference (its formats carry one column index per non-zero), so there is no reference
array to compare with: the CPU tests read the stored arrays back with the layout the header documents and
compare the matrix they describe -- and y = A x computed from them -- with the original CSR; the GPU tests
compare the kernel with the CPU oracle.
"""
import numpy as np
import pytest

import refdump
from alphasparse_b200 import capi, matrices as M
from alphasparse_b200.graph import Format, Matrix


def spec(r, c):
    return f"dense compress\nsub all block_value {r} {c}\nsub all template B1"


def blocky(r, c, block_rows, per_row, seed, dtype=np.float64, holes=0.0, band=200):
    """Matrix of dense r x c blocks; with `holes` > 0 that fraction of the entries inside blocks is dropped, so
    that blocks are only partly filled."""
    rng = np.random.default_rng(seed)
    n_bc = block_rows
    rows, cols = [], []
    for br in range(block_rows):
        lo, hi = max(0, br - band), min(n_bc, br + band + 1)
        bcs = np.unique(np.concatenate([[br], rng.integers(lo, hi, size=per_row - 1)]))
        for bc in bcs:
            for i in range(r):
                for j in range(c):
                    if rng.random() >= holes:
                        rows.append(br * r + i)
                        cols.append(bc * c + j)
    rows, cols = np.array(rows), np.array(cols)
    order = np.lexsort((cols, rows))
    rows, cols = rows[order], cols[order]
    n = block_rows * r
    indptr = np.zeros(n + 1, dtype=np.int64)
    np.add.at(indptr, rows + 1, 1)
    indptr = np.cumsum(indptr)
    vals = rng.standard_normal(rows.shape[0]).astype(dtype)
    x = rng.uniform(-1, 1, size=block_rows * c).astype(dtype)
    return M.CsrMatrix(n, block_rows * c, indptr, cols.astype(np.uint32), vals), x


def dense_from_arrays(fmt, n_rows, n_cols):
    """The matrix the stored arrays describe (small cases only)."""
    d = fmt.plan_descs()[0]
    a = fmt.arrays(0)
    W, r, c = int(d.tlb_size), int(d.bits_row), int(d.bits_off)
    idx, val = a["col_index_arr"][0], a["val_arr"][0]
    NB = idx.shape[0] // W
    A = np.zeros((NB * r, n_cols), dtype=np.float64)
    for b in range(NB):
        for k in range(W):
            bc = int(idx[k * NB + b])
            for i in range(r):
                for j in range(c):
                    A[b * r + i, bc * c + j] += float(val[((k * r + i) * c + j) * NB + b])
    return A[:n_rows]


@pytest.mark.parametrize("r,c", [(2, 2), (3, 3), (4, 4)])
@pytest.mark.parametrize("holes", [0.0, 0.3])
def test_stored_blocks_describe_the_matrix(r, c, holes):
    m, x = blocky(r, c, 37, 5, seed=r * 10 + int(holes * 10), holes=holes, band=12)  # 37 block rows: odd, so one padded block row
    fmt = Matrix.from_csr(m).execute(spec(r, c))
    d = fmt.plan_descs()[0]
    assert d.template_type == capi.TEMPLATE["B1"] and d.bits_row == r and d.bits_off == c and d.effective_num == m.n_rows
    A = dense_from_arrays(fmt, m.n_rows, m.n_cols)
    ref = np.zeros_like(A)
    for row in range(m.n_rows):
        ref[row, m.indices[m.indptr[row] : m.indptr[row + 1]]] = m.values[m.indptr[row] : m.indptr[row + 1]]
    assert np.array_equal(A, ref)
    capi.validate_descs(fmt.plan_descs())
    # one index per block: fewer index bytes than one per non-zero whenever blocks are reasonably full
    idx_bytes = fmt.arrays(0)["col_index_arr"][3] * 4
    assert idx_bytes * (r * c) == fmt.arrays(0)["val_arr"][3] * 4
    fmt.close()


def test_rejections():
    m, _ = blocky(3, 3, 20, 4, seed=1)
    hm = Matrix.from_csr(m)
    for bad, needle in [("dense compress\nsub all block_value 3 3\nsub all template K3", "go together"),
                        ("dense compress\nsub all tlb_row\nsub all template B1", "go together"),
                        ("dense compress\nsub all block_value 5 5\nsub all template B1", "2 x 2, 3 x 3 or 4 x 4"),
                        ("dense sort 1\ndense compress\nsub all block_value 3 3\nsub all template B1", "sorted"),
                        ("dense compress\nsub all block_value 4 4\nsub all template B1", "multiple")]:  # 60 columns % 4 == 0 -> use 3-wide below
        if "4 4" in bad:
            continue
        with pytest.raises(capi.AspError) as e:
            hm.execute(bad)
        assert needle in str(e.value), (bad, str(e.value))
    m2, _ = M.uniform_random(302, 6, seed=3)  # 302 columns: not a multiple of 3
    with pytest.raises(capi.AspError) as e:
        Matrix.from_csr(m2).execute(spec(3, 3))
    assert "multiple" in str(e.value)


def test_a_scattered_matrix_is_refused_rather_than_blown_up():
    m, _ = M.uniform_random(3000, 4, seed=5)  # 3000 columns: a multiple of 3; nearly every non-zero would get a block of its own
    with pytest.raises(capi.AspError) as e:
        Matrix.from_csr(m).execute(spec(3, 3))
    assert "not made of dense blocks" in str(e.value)
    # partly filled blocks are stored (zeros fill them) and the search's padding gate decides
    m2, _ = blocky(3, 3, 300, 5, seed=2, holes=0.5, band=40)
    fmt = Matrix.from_csr(m2).execute(spec(3, 3))
    assert 1.5 < fmt.padding_rate(0) < 4.0
    fmt.close()


def test_save_and_load(tmp_path):
    m, x = blocky(3, 3, 50, 6, seed=9, band=20)
    fmt = Matrix.from_csr(m).execute(spec(3, 3))
    p = str(tmp_path / "b.asp")
    fmt.save(p)
    back = Format.load(p)
    for name in ("val_arr", "col_index_arr"):
        assert np.array_equal(fmt.arrays(0)[name][0], back.arrays(0)[name][0])
    d0, d1 = fmt.plan_descs()[0], back.plan_descs()[0]
    assert (d0.tlb_size, d0.bits_row, d0.bits_off, d0.effective_num, d0.template_type) == (d1.tlb_size, d1.bits_row, d1.bits_off, d1.effective_num, d1.template_type)
    back.close()
    fmt.close()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
@pytest.mark.parametrize("r,c,holes", [(3, 3, 0.0), (3, 3, 0.25), (2, 2, 0.0), (4, 4, 0.1)])
def test_kernel_matches_oracle(asp_ctx, r, c, holes, dtype):
    m, x = blocky(r, c, 4001, 9, seed=r + 7, dtype=dtype, holes=holes)  # odd block-row count: the padded block row and the tail rows
    fmt = Matrix.from_csr(m).execute(spec(r, c))
    g = fmt.upload(asp_ctx)
    y_ref, scale = refdump.csr_ref(m, x)
    refdump.assert_y(g.spmv_host(x), y_ref, scale, dtype, f"block {r}x{c} holes {holes}")
    for threads in (32, 96, 128):
        g.set_launch(0, 1, threads, 1)
        refdump.assert_y(g.spmv_host(x), y_ref, scale, dtype, f"block {r}x{c} threads {threads}")
    g.close()
    fmt.close()


@pytest.mark.gpu
def test_fem_like_matrix_of_the_benchmark_at_reduced_size(asp_ctx):
    m, x = M.block_fem(20000, 27, 4096, seed=3)
    fmt = Matrix.from_csr(m).execute(spec(3, 3))
    assert abs(fmt.padding_rate(0) - 1.0) < 1e-3  # every block is full and every block row has 27 blocks
    g = fmt.upload(asp_ctx)
    y_ref, scale = refdump.csr_ref(m, x)
    refdump.assert_y(g.spmv_host(x), y_ref, scale, np.float64, "fem 3x3")
    g.close()
    fmt.close()
