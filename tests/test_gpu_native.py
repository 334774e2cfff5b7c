"""GPU suite, native path end to end: seeded matrix -> native Operator Graph -> C-ABI upload ->
CUDA kernel -> y against the CPU oracle. Sizes are chosen so the oracle finishes in well under a
second; the full-size configurations are checked the same way inside bench.py."""
import numpy as np
import pytest

import refdump
import specs
from alphasparse_b200 import capi, matrices as M, tuner
from alphasparse_b200.graph import Matrix

pytestmark = pytest.mark.gpu


def run(ctx, m, x, spec, what):
    fmt = Matrix.from_csr(m).execute(spec)
    g = fmt.upload(ctx)
    y = g.spmv_host(x)
    y_ref, scale = refdump.csr_ref(m, x)
    refdump.assert_y(y, y_ref, scale, m.values.dtype, what)
    g.close()
    fmt.close()


@pytest.fixture(scope="module")
def mats():
    rng = np.random.default_rng(3)
    lengths = np.concatenate([rng.integers(600, 5000, size=24), rng.integers(130, 500, size=300), rng.integers(33, 127, size=2000),
                              np.minimum(rng.zipf(2.1, size=30000), 31)])
    rng.shuffle(lengths)
    return {
        "uniform_f32": M.uniform_random(20000, 16, seed=0),
        "laplace_f64": M.laplacian_2d(160, seed=1),
        "fem_f64": M.block_fem(4096, 27, 256, seed=3),
        "mixed_f32": M.from_row_lengths(lengths, 40000, seed=2),
        "rmat_f32": M.rmat(13, 16, seed=4),
    }


@pytest.mark.parametrize("mat", ["uniform_f32", "laplace_f64"])
@pytest.mark.parametrize("spec", sorted(specs.COMPRESSED_SPECS))
def test_every_strategy_on_short_row_matrices(asp_ctx, mats, mat, spec):
    m, x = mats[mat]
    run(asp_ctx, m, x, specs.full_spec(spec), f"{mat} {spec}")


@pytest.mark.parametrize("spec", ["S5_K3", "S1_K2", "S4_K4", "S6_K8", "S7_K8", "S8_K7", "S2_K6", "S9_K9", "S9_K10"])
def test_block_fem_fp64(asp_ctx, mats, spec):
    m, x = mats["fem_f64"]
    run(asp_ctx, m, x, specs.full_spec(spec), f"fem {spec}")


@pytest.mark.parametrize("dense", ["dense sort 1\ndense compress", "dense compress"])
@pytest.mark.parametrize("spec", ["S8_K7", "S4_K4", "S7_K8", "S3_K6", "S2_K6", "X_K1", "X_K5"])
def test_power_law_rows_sorted_and_unsorted(asp_ctx, mats, dense, spec):
    m, x = mats["mixed_f32"]
    run(asp_ctx, m, x, specs.full_spec(spec, dense), f"mixed {dense!r} {spec}")


@pytest.mark.parametrize("dense", ["dense sort 1\ndense rowdiv_exp 32 4096 4\ndense compress", "dense sort 1\ndense rowdiv_exp 128 4096 8\ndense compress"])
@pytest.mark.parametrize("pick", [0, -1])
def test_sorted_row_division_with_a_template_per_strip(asp_ctx, mats, dense, pick):
    """Dense-view strategy 3 of the tuner: every strip gets the first / last whitelist strategy its
    row statistics allow."""
    m, x = mats["mixed_f32"]
    hm = Matrix.from_csr(m)
    cm = hm.dense(dense)
    assert cm.n_subs >= 3
    lines = []
    for i in range(cm.n_subs):
        rows, nnz, mn, mx = cm.sub_rows(i)
        cands = tuner.compressed_candidates(mn, mx, nnz / rows, True, quick=True)
        assert cands, (i, mn, mx)
        lines.append(cands[pick].lines(i))
    fmt = cm.execute("\n".join(lines))
    g = fmt.upload(asp_ctx)
    y = g.spmv_host(x)
    y_ref, scale = refdump.csr_ref(m, x)
    refdump.assert_y(y, y_ref, scale, m.values.dtype, f"{dense!r} pick {pick}: {lines}")
    g.close()
    fmt.close()


@pytest.mark.parametrize("spec", ["S8_K7", "S9_K9", "S9_K10", "S3_K6", "S7_K8"])
def test_rows_without_nonzeros(asp_ctx, mats, spec):
    """R-MAT adjacency has empty rows (the reference's front door rejects them, main.cc:604-621);
    their y must be exactly 0."""
    m, x = mats["rmat_f32"]
    assert (m.row_lengths() == 0).any()
    run(asp_ctx, m, x, specs.full_spec(spec), f"rmat {spec}")
    run(asp_ctx, m, x, specs.full_spec(spec, "dense sort 1\ndense compress") if spec not in ("S9_K9", "S9_K10") else specs.full_spec(spec), f"rmat sorted {spec}")


@pytest.mark.parametrize("mat", ["uniform_f32", "mixed_f32", "fem_f64"])
def test_tuner_search_returns_a_correct_plan(asp_ctx, mats, mat):
    m, x = mats[mat]
    fmt, group, trials, desc = tuner.search(asp_ctx, m, quick=True, warmup=1, reps=3)
    assert len(trials) > 0 and desc["subs"]
    y = group.spmv_host(x)
    y_ref, scale = refdump.csr_ref(m, x)
    refdump.assert_y(y, y_ref, scale, m.values.dtype, f"tuner {mat}: {desc}")
    group.close()
    fmt.close()


@pytest.mark.parametrize("dense", ["dense compress", "dense sort 1\ndense compress"])
def test_sell_strips_wider_than_255_elements(asp_ctx, mats, dense):
    # the reference types thread_block_size_in_block by its last entry and truncates wider strips
    # (372 -> 116); the native lowering keeps the value
    m, x = M.rmat(11, 8, seed=4)
    assert m.row_lengths().max() > 255
    run(asp_ctx, m, x, dense + "\nsub all row_padding 128 1\nsub all blb_row_evenly 128\nsub all tlb_row\nsub all template K2", f"wide SELL {dense!r}")


def test_format_loaded_from_its_file_runs_like_the_original(asp_ctx, mats, tmp_path):
    from alphasparse_b200.graph import Format

    m, x = mats["mixed_f32"]
    fmt = Matrix.from_csr(m).execute(specs.full_spec("S8_K7", "dense sort 1\ndense compress"))
    path = str(tmp_path / "mixed.asp")
    fmt.save(path)
    back = Format.load(path)
    g0, g1 = fmt.upload(asp_ctx), back.upload(asp_ctx)
    y0, y1 = g0.spmv_host(x), g1.spmv_host(x)
    y_ref, scale = refdump.csr_ref(m, x)
    refdump.assert_y(y1, y_ref, scale, m.values.dtype, "loaded format")
    assert np.array_equal(y0, y1) or refdump.rel_err(y1, y0.astype(np.float64), scale) <= 1e-6  # atomics may reorder sums
    for o in (g0, g1, fmt, back):
        o.close()


@pytest.mark.parametrize("templ", ["K9", "K10"])
@pytest.mark.parametrize("s", [4, 8, 16, 32, 5])
@pytest.mark.parametrize("mat", ["rmat_f32", "mixed_f32", "laplace_f64", "fem_f64"])
def test_csr5_like_kernels_for_every_tlb_size_direct_and_staged(asp_ctx, mats, mat, s, templ):
    """The CSR5-like family is specialised on the TLB size (4, 8, 16, 32; any other size takes the generic
    kernel). Both write-out forms -- one store per row, and the warp's rows through shared memory as one
    contiguous run -- must give the oracle's y; rows spanning many warps (mixed_f32 has rows of up to
    5000 non-zeros) and rows without non-zeros (rmat_f32) included."""
    m, x = mats[mat]
    fmt = Matrix.from_csr(m).execute(f"dense compress\nsub all tlb_nnz {s}\nsub all template {templ}")
    g = fmt.upload(asp_ctx)
    y_ref, scale = refdump.csr_ref(m, x)
    for path in (0, 1):
        for threads in (64, 256):
            tuner.set_launch(fmt, g, 0, threads, 1 + path)  # third launch parameter: 1 = row by row, 2 = staged write-out
            assert g.get_launch(0)[2] == 1 + path
            refdump.assert_y(g.spmv_host(x), y_ref, scale, m.values.dtype, f"{mat} {templ} s={s} path={path} threads={threads}")
    g.close()
    fmt.close()


def test_search_times_coinciding_launch_requests_once(asp_ctx):
    """The launch sweep of the reference asks for CTA widths that the kernels fold into the same effective launch
    (CSR5-like: 64..256 threads walk the same warps with more or fewer CTAs only up to the CTAs that have work).
    The GPU timer measures every effective launch once and says how many requests it folded."""
    m, x = M.uniform_random(4096, 16, seed=0)
    lines = []
    fmt, group, trials, desc = tuner.search(asp_ctx, m, quick=0, warmup=1, reps=3, log=lines.append)
    tail = [l for l in lines if l.startswith("timer:")]
    assert len(tail) == 1, lines[-3:]
    measured, reused = [int(t) for t in tail[0].replace(",", "").split() if t.isdigit()]
    assert measured > 0 and measured + reused >= len(trials), (tail, len(trials))
    print(tail[0])
    y = group.spmv_host(x)
    y_ref, scale = refdump.csr_ref(m, x)
    refdump.assert_y(y, y_ref, scale, m.values.dtype, f"search {desc}")
    group.close()
    fmt.close()


@pytest.mark.parametrize("case", ["laplacian_D1", "laplacian_K3", "fem_B1", "uniform_K9"])
def test_pipelined_host_spmv_matches_the_oracle(asp_ctx, case):
    """asp_spmv_host_pipelined: row chunks with their own plan groups, x uploaded as a growing prefix, y leaving chunk by
    chunk. Banded matrices (every chunk starts before all of x has arrived) and a matrix with random columns (col_hi =
    all columns for every chunk: no overlap, same result)."""
    import torch

    if case.startswith("laplacian"):
        m, x = M.laplacian_2d(256, seed=1)
        sub = {"D1": {"graph": "S0_D1", "nodes": ["diag_value"], "template": "D1", "threads": 128, "row_reduce": 1},
               "K3": {"graph": "S5_K3", "nodes": ["row_padding 32 1", "tlb_row"], "template": "K3", "threads": 256, "row_reduce": 1}}[case[-2:]]
        align = 32
    elif case == "fem_B1":
        m, x = M.block_fem(3000, 9, half_band=64, seed=3)
        sub = {"graph": "S0_B1_3x3", "nodes": ["block_value 3 3"], "template": "B1", "threads": 128, "row_reduce": 1}
        align = 6
    else:
        m, x = M.uniform_random(20000, 12, seed=7)
        sub = {"graph": "S9_K9_s8", "nodes": ["tlb_nnz 8"], "template": "K9", "threads": 128, "row_reduce": 1}
        align = 1
    desc = {"dense": "dense compress", "subs": [sub]}
    chunks = tuner.build_row_chunks(asp_ctx, m, desc, 7, align)
    assert chunks[0][2] == 0 and chunks[-1][3] == m.n_rows and len(chunks) >= 6
    if case != "uniform_K9":
        assert chunks[0][4] < m.n_cols // 2  # banded: the first chunk needs less than half of x
    hx = torch.from_numpy(np.ascontiguousarray(x)).pin_memory()
    hy = torch.empty(m.n_rows, dtype=hx.dtype).pin_memory()
    y_ref, scale = refdump.csr_ref(m, x)
    for rep in range(2):  # the second call reuses the context's streams, events and staging buffers
        hy.fill_(-1.0)
        capi.spmv_host_pipelined(asp_ctx, [(g, lo, hi, ch) for _, g, lo, hi, ch in chunks], hx.data_ptr(), hy.data_ptr())
        refdump.assert_y(hy.numpy(), y_ref, scale, m.values.dtype, f"{case} pipelined, call {rep}")
    # chunks that do not tile the rows are refused before anything is copied
    bad = [(g, lo, hi, ch) for _, g, lo, hi, ch in chunks][1:]
    with pytest.raises(capi.AspError):
        capi.spmv_host_pipelined(asp_ctx, bad, hx.data_ptr(), hy.data_ptr())
    for f, g, *_ in chunks:
        g.close()
        f.close()


@pytest.mark.parametrize("templ", ["K9", "K10"])
@pytest.mark.parametrize("s", [1, 2, 3, 4, 5, 6, 7, 8, 16, 32])
def test_csr5_like_small_exhaustive_on_the_gpu(asp_ctx, templ, s):
    """The small shapes of the CPU suite's exhaustive test through the kernels (specialised for TLB size 4 / 8 / 16 / 32,
    generic otherwise; column indices fit 16 bits here, so sizes 4 .. 32 also run the generic kernel's narrow-column
    path), and a wide copy of each shape (more than 65536 columns) that takes the specialised kernels."""
    shapes = [
        [1, s, s + 1, 0, 2 * s, 32 * s, 32 * s + 1, 0, 0, 3, 70 * s, 1, 31 * s, s - 1 if s > 1 else 1],
        [70 * s],
        [0, 0, 5, 0, 33 * s, 0],
        list(range(1, 40)),
        [64 * s] * 3 + [1] * 50,
    ]
    for n_cols in (70 * 32 + 7, 70000):
        for k, lens in enumerate(shapes):
            m, x = M.from_row_lengths(np.array(lens, dtype=np.int64), n_cols, seed=50 + k, dtype=np.float32)
            for dense in ("dense compress", "dense sort 1\ndense compress"):
                run(asp_ctx, m, x, f"{dense}\nsub all tlb_nnz {s}\nsub all template {templ}", f"{templ} s={s} shape {k} cols {n_cols} {dense!r}")


def test_renumbered_matrix_runs_like_the_original(asp_ctx):
    """asp_matrix_relabel_by_column_count, then the ordinary lowering and kernels: y'[labels[v]] is the original y[v],
    and the rows without non-zeros are the suffix of y' (R-MAT: half of the rows are empty, the hub columns get the
    low numbers)."""
    m, x = M.rmat(17, 8, seed=4)
    hm = Matrix.from_csr(m)
    m2, labels, n_active = hm.relabel_by_column_count(True)
    fmt = m2.execute("dense sort 1073741824\ndense compress\nsub all tlb_nnz 32\nsub all template K9")
    g = fmt.upload(asp_ctx)
    xp = np.zeros_like(x)
    xp[labels] = x
    yp = g.spmv_host(xp)
    y_ref, scale = refdump.csr_ref(m, x)
    refdump.assert_y(yp[labels], y_ref, scale, m.values.dtype, "renumbered R-MAT")
    assert n_active == int((m.row_lengths() > 0).sum()) and np.all(yp[n_active:] == 0)
    for o in (g, fmt, m2, hm):
        o.close()
