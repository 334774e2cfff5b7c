"""CPU suite: the `.mtx.coo` input path of configuration 1 (uniform random 4096 x 4096, fp32, seed 0).
The native reader must give the same matrix, and therefore byte-identical format arrays, as the
in-memory CSR entry point; the Python reader must round-trip the writer."""
import numpy as np

import specs
from alphasparse_b200 import matrices as M
from alphasparse_b200.graph import Matrix


def _arrays(fmt):
    out = []
    for sub in range(fmt.n_subs):
        for name, (arr, comp, dt, ln) in sorted(fmt.arrays(sub).items()):
            out.append((sub, name, arr, comp, dt, ln))
    return out


def test_config1_from_coo_file_equals_from_csr(tmp_path):
    m, x = M.uniform_random(4096, 16, seed=0)
    path = str(tmp_path / "c1.mtx.coo")
    M.write_mtx_coo(path, m)
    back = M.read_mtx_coo(path)
    assert back.n_rows == m.n_rows and back.n_cols == m.n_cols
    assert np.array_equal(back.indptr, m.indptr) and np.array_equal(back.indices, m.indices)
    assert np.allclose(back.values, m.values, rtol=1e-6)  # the text format keeps 7-9 significant digits
    a, b = Matrix.from_coo_file(path, np.float32), Matrix.from_csr(back)
    assert (tuple(a.shape), a.nnz) == (tuple(b.shape), b.nnz) == ((m.n_rows, m.n_cols), m.nnz)
    for name in ("S5_K3", "S9_K9"):
        fa, fb = a.execute(specs.full_spec(name)), b.execute(specs.full_spec(name))
        la, lb = _arrays(fa), _arrays(fb)
        assert len(la) == len(lb) > 0
        for (sa, na, xa, ca, da, na_len), (sb, nb, xb, cb, db, nb_len) in zip(la, lb):
            assert (sa, na, ca, da, na_len) == (sb, nb, cb, db, nb_len), (name, sa, na)
            assert (xa is None) == (xb is None) and (xa is None or np.array_equal(xa, xb)), (name, sa, na)
        fa.close()
        fb.close()
    a.close()
    b.close()


def test_sell_tlb_size_array_is_wide_enough_for_its_largest_entry():
    # reference defect (direct_atom_op_warp_compress.cc:239): typed by the LAST entry, so a strip of
    # 372 elements per row is stored as 116 in a u8 array when the last strip is narrow
    m, _ = M.rmat(11, 8, seed=4)
    lens = m.row_lengths()
    assert lens.max() > 255 and lens[-128:].max() < 256
    fmt = Matrix.from_csr(m).execute("dense compress\nsub all row_padding 128 1\nsub all blb_row_evenly 128\nsub all tlb_row\nsub all template K2")
    arr = fmt.arrays(0)["thread_block_size_in_block"][0]
    assert arr.dtype == np.uint16 and int(arr.max()) == int(lens.max())
    fmt.close()


def test_laplacian_row_block_equals_the_slice_of_the_whole_grid():
    # what each rank of the weak-scaling run builds: its rows only, global columns, the full x
    whole, x = M.laplacian_2d(48, 1, grid_y=48 * 3)
    for r in range(3):
        blk, xb = M.laplacian_2d(48, 1, grid_y=48 * 3, rows=(r * 48 * 48, (r + 1) * 48 * 48))
        ref = whole.row_slice(r * 48 * 48, (r + 1) * 48 * 48)
        assert (blk.n_rows, blk.n_cols) == (ref.n_rows, ref.n_cols) and np.array_equal(x, xb)
        assert np.array_equal(blk.indptr, ref.indptr) and np.array_equal(blk.indices, ref.indices) and np.array_equal(blk.values, ref.values)
