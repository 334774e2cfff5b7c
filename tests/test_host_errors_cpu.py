"""CPU suite: error behaviour of the host entry points. Every failure is a status plus a message
(asp_host_last_error); nothing aborts, unlike the reference's asserts on the same inputs."""
import numpy as np
import pytest

from alphasparse_b200 import capi, matrices as M
from alphasparse_b200.graph import Matrix


@pytest.fixture(scope="module")
def hm():
    m, _ = M.uniform_random(300, 6, seed=1)
    return Matrix.from_csr(m)


@pytest.mark.parametrize("spec,needle", [
    ("dense compress\nsub all frobnicate 3\nsub all template K3", "frobnicate"),
    ("dense compress\nsub all template K99", "K99"),
    ("dense compress\nsub all tlb_row\nsub all template K9", "nnz division"),
    ("dense compress\nsub 7 tlb_nnz 4\nsub 7 template K9", "sub"),
    ("dense sort 0\ndense compress\nsub all tlb_nnz 4\nsub all template K9", "sort"),
])
def test_bad_graph_specs_are_reported_not_fatal(hm, spec, needle):
    with pytest.raises(capi.AspError) as e:
        hm.execute(spec)
    assert needle.lower() in str(e.value).lower()


def test_unsorted_columns_and_bad_shapes_are_rejected():
    indptr = np.array([0, 2, 3], dtype=np.int64)
    bad = M.CsrMatrix(2, 4, indptr, np.array([3, 1, 0], dtype=np.uint32), np.ones(3, dtype=np.float32))
    with pytest.raises(capi.AspError) as e:
        Matrix.from_csr(bad)
    assert "sorted" in str(e.value)
    out_of_range = M.CsrMatrix(2, 2, indptr, np.array([0, 5, 1], dtype=np.uint32), np.ones(3, dtype=np.float32))
    with pytest.raises(capi.AspError):
        Matrix.from_csr(out_of_range)


def test_missing_coo_file_is_an_error(tmp_path):
    with pytest.raises(capi.AspError):
        Matrix.from_coo_file(str(tmp_path / "nope.mtx.coo"))
