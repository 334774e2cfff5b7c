"""BASELINE configuration 1 itself -- uniform_random(4096, 16, seed 0), fp32 -- through the reference's host pipeline
and through the native path, for every whitelist strategy its row statistics admit (1, 5, 9 with both CSR5-like
templates, 2, 3): the native format arrays equal the reference's bit for bit (CPU), and the kernels' y from the native
arrays matches the oracle (GPU). Configuration 1 exists precisely because the reference can ingest it whole."""
import numpy as np
import pytest

import refdump
from alphasparse_b200 import matrices as M
from alphasparse_b200.graph import Matrix
from test_format_parity import compare_with_manifest

# node parameters inside the grids the reference's tuner sweeps on this matrix (rows of 4..32 non-zeros)
SPECS = {
    "S1_K2_m64": "dense compress\nsub all row_padding 64 1\nsub all blb_row_evenly 64\nsub all tlb_row\nsub all template K2",
    "S1_K2_m192": "dense compress\nsub all row_padding 192 1\nsub all blb_row_evenly 192\nsub all tlb_row\nsub all template K2",
    "S5_K3": "dense compress\nsub all row_padding 32 1\nsub all tlb_row\nsub all template K3",
    "S9_K9_s2": "dense compress\nsub all tlb_nnz 2\nsub all template K9",
    "S9_K9_s14": "dense compress\nsub all tlb_nnz 14\nsub all template K9",
    "S9_K10_s8": "dense compress\nsub all tlb_nnz 8\nsub all template K10",
    "S2_K6_m32_c4": "dense compress\nsub all row_padding 32 4\nsub all blb_row_evenly 32\nsub all tlb_col_fixed 4\nsub all template K6",
    "S2_K6_m64_c13": "dense compress\nsub all row_padding 64 4\nsub all blb_row_evenly 64\nsub all tlb_col_fixed 13\nsub all template K6",
    "S3_K6_b512_c3": "dense compress\nsub all blb_row_nnz 512\nsub all tlb_col_fixed 3\nsub all template K6",
    "S3_K6_b128_c1": "dense compress\nsub all blb_row_nnz 128\nsub all tlb_col_fixed 1\nsub all template K6",
}


@pytest.fixture(scope="module")
def c1():
    return M.uniform_random(4096, 16, 0)


@pytest.mark.skipif(not refdump.have_ref_dump(), reason="reference format oracle not built")
@pytest.mark.parametrize("name", sorted(SPECS))
def test_native_arrays_equal_the_references(c1, name):
    m, _ = c1
    assert int(m.row_lengths().min()) == 4  # the padding rows of strategy 2 take the shortest row's length
    man = refdump.run_ref_dump(m, SPECS[name])
    fmt = Matrix.from_csr(m).execute(SPECS[name])
    compare_with_manifest(fmt, man, f"config 1 {name}")
    fmt.close()


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(SPECS))
def test_kernels_on_config_1(asp_ctx, c1, name):
    m, x = c1
    fmt = Matrix.from_csr(m).execute(SPECS[name])
    g = fmt.upload(asp_ctx)
    y_ref, scale = refdump.csr_ref(m, x)
    refdump.assert_y(g.spmv_host(x), y_ref, scale, np.float32, f"config 1 {name}")
    g.close()
    fmt.close()


@pytest.mark.gpu
def test_config_2_at_full_size(asp_ctx):
    """The 2048 x 2048 Laplacian (4,194,304 rows, fp64) with the graph the search picks, against the oracle."""
    m, x = M.laplacian_2d(2048, 1)
    fmt = Matrix.from_csr(m).execute("dense compress\nsub all row_padding 32 1\nsub all tlb_row\nsub all template K3")
    g = fmt.upload(asp_ctx)
    y_ref, scale = refdump.csr_ref(m, x)
    refdump.assert_y(g.spmv_host(x), y_ref, scale, np.float64, "config 2, full size")
    g.close()
    fmt.close()


@pytest.mark.gpu
@pytest.mark.parametrize("reduce", [1, 2])
def test_rescaled_graph_matrix_iterated_twenty_times(asp_ctx, reduce):
    """The repeated SpMV of configuration 5 on a matrix whose values are scaled so that x stays finite: after 20
    iterations of x <- A x on the GPU the vector still matches 20 iterations of the oracle."""
    import torch

    from alphasparse_b200 import tuner

    m, x = M.rmat(14, 16, seed=4)
    m.values *= 1.0 / 16.0
    fmt = Matrix.from_csr(m).execute("dense sort 1073741824\ndense compress\nsub all tlb_nnz 32\nsub all template K9")
    g = fmt.upload(asp_ctx)
    tuner.set_launch(fmt, g, 0, 128, reduce)
    a = torch.from_numpy(x.copy()).cuda()
    b = torch.zeros_like(a)
    for _ in range(20):
        g.spmv(a.data_ptr(), b.data_ptr(), True)
        a, b = b, a
    asp_ctx.synchronize()
    ref = x.astype(np.float64)
    for _ in range(20):
        ref, _ = refdump.csr_ref(m, ref.astype(np.float32))
    got = a.cpu().numpy().astype(np.float64)
    assert np.isfinite(got).all() and np.max(np.abs(ref)) > 0
    assert np.max(np.abs(got - ref)) <= 2e-4 * np.max(np.abs(ref))
    g.close()
    fmt.close()
