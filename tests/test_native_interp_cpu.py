"""CPU suite: y computed from the NATIVE format arrays by the template interpreter equals the CSR
oracle, for every strategy on seeded and on randomly drawn matrices (rows without non-zeros, a few
long rows, sorted and unsorted). This checks the native operators and lowerings beyond the inputs the
reference itself can process, without a GPU."""
import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

import plan_interp
import refdump
import specs
from alphasparse_b200 import capi, matrices as M
from alphasparse_b200.graph import Matrix
from native_manifest import NativeManifest


def check(m, x, spec, what):
    fmt = Matrix.from_csr(m).execute(spec)
    y = plan_interp.interpret(NativeManifest(fmt, m.n_rows), x)
    y_ref, scale = refdump.csr_ref(m, x)
    err = refdump.rel_err(y, y_ref, scale)
    assert err <= 1e-12, f"{what}: {err}"
    fmt.close()


@pytest.mark.parametrize("spec", sorted(specs.COMPRESSED_SPECS))
def test_every_strategy_native_uniform(spec):
    m, x = M.uniform_random(600, 9, seed=5, dtype=np.float64)
    check(m, x, specs.full_spec(spec), spec)


@pytest.mark.parametrize("dense", ["dense compress", "dense sort 1\ndense compress", "dense sort 1073741824\ndense compress"])
@pytest.mark.parametrize("spec", ["S9_K9", "S9_K10", "S8_K7", "S3_K6", "S7_K8"])
def test_rows_without_nonzeros_sorted_and_unsorted(dense, spec):
    m, x = M.rmat(9, 6, seed=4)
    check(m, x.astype(np.float32), specs.full_spec(spec, dense), f"{dense!r} {spec}")


def test_wide_sell_strips_keep_their_size():
    m, x = M.rmat(11, 8, seed=4)
    for dense in ("dense compress", "dense sort 1\ndense compress"):
        check(m, x, dense + "\nsub all row_padding 128 1\nsub all blb_row_evenly 128\nsub all tlb_row\nsub all template K2", f"wide SELL {dense!r}")


@settings(max_examples=80, deadline=None)
@given(seed=st.integers(0, 1_000_000), n=st.integers(20, 400), kind=st.integers(0, 3), holes=st.booleans(),
       spec=st.sampled_from(sorted(specs.COMPRESSED_SPECS)),
       dense=st.sampled_from(["dense compress", "dense sort 1\ndense compress", "dense sort 1\ndense rowdiv_exp 8 4096 4\ndense compress"]))
def test_random_matrices_every_strategy(seed, n, kind, holes, spec, dense):
    """Short rows, power-law rows, medium rows, a few very long rows; optionally a quarter of the rows
    empty; unsorted, sorted, sorted and divided into strips. The lowering either refuses the graph
    with a status or yields arrays whose interpretation equals the CSR product."""
    rng = np.random.default_rng(seed)
    if kind == 0:
        lengths = rng.integers(0, 12, size=n)
    elif kind == 1:
        lengths = np.minimum(rng.zipf(1.7, size=n), n // 2)
    elif kind == 2:
        lengths = rng.integers(30, min(n, 200) + 31, size=n).clip(max=n)
    else:
        lengths = np.minimum(rng.zipf(2.0, size=n), n // 3)
        lengths[rng.integers(0, n, size=3)] = rng.integers(n // 2, n, size=3)
    if holes:
        lengths[rng.random(n) < 0.25] = 0
    if lengths.sum() == 0:
        lengths[0] = 1
    m, x = M.from_row_lengths(lengths.astype(np.int64), n, seed=seed % 1000, dtype=np.float64)
    try:
        check(m, x, specs.full_spec(spec, dense), f"seed {seed} n {n} kind {kind} holes {holes} {spec} {dense!r}")
    except capi.AspError:
        pass  # a graph this matrix does not admit: reported, not fatal


def test_explicit_row_division_with_a_template_per_strip():
    # DENSE_ROW_DIV with explicit positions; strips without non-zeros are dropped as in the reference
    m, x = M.uniform_random(900, 7, seed=9, dtype=np.float64)
    hm = Matrix.from_csr(m)
    cm = hm.dense("dense rowdiv 100 450 451\ndense compress")
    assert cm.n_subs == 4
    assert [cm.sub_rows(i)[0] for i in range(4)] == [100, 350, 1, 449]
    spec = ("dense rowdiv 100 450 451\ndense compress\n" + "sub 0 tlb_nnz 4\nsub 0 template K9\n" + "sub 1 row_padding 32 1\nsub 1 tlb_row\nsub 1 template K3\n"
            + "sub 2 template EMPTY\n" + "sub 3 blb_row_nnz 512\nsub 3 tlb_col_fixed 2\nsub 3 template K6")
    fmt = hm.execute(spec)
    y = plan_interp.interpret(NativeManifest(fmt, m.n_rows), x)
    y_ref, scale = refdump.csr_ref(m, x)
    keep = np.ones(m.n_rows, bool)
    keep[450] = False  # the strip given the EMPTY template is not computed
    assert refdump.rel_err(y[keep], y_ref[keep], scale[keep]) <= 1e-12 and y[450] == 0
    for bad in ("dense rowdiv 0 10\ndense compress", "dense rowdiv 500 400\ndense compress", "dense rowdiv 900\ndense compress"):
        with pytest.raises(Exception):
            hm.dense(bad)


@pytest.mark.parametrize("templ", ["K9", "K10"])
@pytest.mark.parametrize("s", [1, 2, 3, 4, 5, 6, 7, 8, 16, 32])
def test_csr5_like_small_exhaustive(templ, s):
    """Small cases for the two CSR5-like templates at every TLB size 1..8 (and 16, 32): rows of 1 .. 70 threads' worth of
    non-zeros, rows that end exactly on a thread or warp boundary, rows without non-zeros between them, a matrix that
    is one long row. Where the reference's emitted kernels store a thread's partial instead of the row total
    (unaligned_warp_reduce_same_TLB_size_op.cc:1152-1250), the arrays walked the way the native kernels walk them must
    give the CSR result."""
    n_cols = 70 * 32 + 7
    shapes = [
        [1, s, s + 1, 0, 2 * s, 32 * s, 32 * s + 1, 0, 0, 3, 70 * s, 1, 31 * s, s - 1 if s > 1 else 1],
        [70 * s],
        [0, 0, 5, 0, 33 * s, 0],
        list(range(1, 40)),
        [64 * s] * 3 + [1] * 50,
    ]
    for k, lens in enumerate(shapes):
        m, x = M.from_row_lengths(np.array(lens, dtype=np.int64), n_cols, seed=50 + k, dtype=np.float64)
        for dense in ("dense compress", "dense sort 1\ndense compress"):
            check(m, x, f"{dense}\nsub all tlb_nnz {s}\nsub all template {templ}", f"{templ} s={s} shape {k} {dense!r}")
