"""CPU suite: a lowered format saved to its binary file and loaded back answers every query like the
original (arrays byte for byte, closed forms, scalars, launch parameters, shared row permutation),
and the interpreter computes the same y from it. Corrupt files are rejected, not trusted."""
import numpy as np
import pytest

import plan_interp
import refdump
import specs
from alphasparse_b200 import capi, matrices as M
from alphasparse_b200.graph import Format, Matrix
from native_manifest import NativeManifest

DESC_FIELDS = ("template_type", "val_dtype", "n_rows", "n_cols", "first_row", "first_col", "true_nnz", "n_arrays", "effective_num", "tlb_size",
               "bits_word", "bits_flag", "bits_row", "bits_off", "is_atom_add", "sort_kind", "tblock_num", "thread_num_in_block", "thread_num_of_row_reduce")
INFO_FIELDS = ("min_row", "max_row", "min_col", "max_col", "begin_coo", "end_coo", "n_blb", "n_wlb", "n_tlb", "template_type", "n_arrays")


def same(a: Format, b: Format):
    assert a.n_subs == b.n_subs
    pa, pb = a.global_perm(), b.global_perm()
    assert (pa is None) == (pb is None) and (pa is None or (pa.dtype == pb.dtype and np.array_equal(pa, pb)))
    for i, (da, db) in enumerate(zip(a.plan_descs(), b.plan_descs())):
        for k in DESC_FIELDS:
            assert getattr(da, k) == getattr(db, k), (i, k)
        ia, ib = a.sub_info(i), b.sub_info(i)
        for k in INFO_FIELDS:
            assert getattr(ia, k) == getattr(ib, k), (i, k)
        assert a.padding_rate(i) == b.padding_rate(i)
        xa, xb = a.arrays(i), b.arrays(i)
        assert list(xa) == list(xb)
        for name in xa:
            (ra, ca, ta, la), (rb, cb, tb, lb) = xa[name], xb[name]
            assert (ca, ta, la) == (cb, tb, lb), (i, name)
            assert (ra is None) == (rb is None) and (ra is None or (ra.dtype == rb.dtype and np.array_equal(ra.view(np.uint8), rb.view(np.uint8)))), (i, name)


@pytest.mark.parametrize("dense,spec", [("dense compress", "S5_K3"), ("dense compress", "S9_K10"), ("dense sort 1\ndense compress", "S2_K6"),
                                        ("dense sort 1\ndense rowdiv_exp 32 4096 4\ndense compress", "S9_K9"), ("dense sort 1\ndense compress", "S1_K2")])
def test_round_trip(tmp_path, dense, spec):
    m, x = M.rmat(10, 6, seed=4) if "sort" in dense else M.uniform_random(700, 9, seed=5)
    fmt = Matrix.from_csr(m).execute(specs.full_spec(spec, dense))
    path = str(tmp_path / "fmt.asp")
    fmt.save(path)
    back = Format.load(path)
    same(fmt, back)
    y = plan_interp.interpret(NativeManifest(back, m.n_rows), x.astype(np.float64))
    y_ref, scale = refdump.csr_ref(m, x)
    assert refdump.rel_err(y, y_ref, scale) <= 1e-6
    # the permutation is stored once and shared by every sub-matrix that refers to it
    if back.global_perm() is not None and back.n_subs > 1:
        ptrs = {a.host_ptr for d in back.plan_descs() for a in (d.arrays[k] for k in range(d.n_arrays)) if a.role == capi.ROLE["row_index_before_sort"]}
        assert len(ptrs) == 1
    back.close()
    fmt.close()


def test_bad_files_are_rejected(tmp_path):
    m, _ = M.uniform_random(300, 6, seed=1)
    fmt = Matrix.from_csr(m).execute(specs.full_spec("S5_K3"))
    good = tmp_path / "good.asp"
    fmt.save(str(good))
    data = good.read_bytes()
    (tmp_path / "magic.asp").write_bytes(b"NOTASPF\0" + data[8:])
    (tmp_path / "short.asp").write_bytes(data[: len(data) // 2])
    for name in ("magic.asp", "short.asp", "missing.asp"):
        with pytest.raises(capi.AspError):
            Format.load(str(tmp_path / name))
    with pytest.raises(capi.AspError):
        fmt.save(str(tmp_path / "no_such_dir" / "x.asp"))
