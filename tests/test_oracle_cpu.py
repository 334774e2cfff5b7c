"""CPU suite, part 1: the oracles against each other and against the golden fixtures."""
import numpy as np
import pytest

import plan_interp
import refdump
from golden_util import golden_names, load_golden

NAMES = golden_names()


def test_golden_present():
    assert len(NAMES) >= 20


@pytest.mark.parametrize("name", NAMES)
def test_reference_arrays_reproduce_csr_spmv(name):
    """The reference's template arrays, walked the way its emitted kernels walk them, give the
    same y as the plain CSR loop over the original matrix."""
    m, x, _, man = load_golden(name)
    y_ref, scale = refdump.csr_ref(m, x)
    y = plan_interp.interpret(man, x)
    assert refdump.rel_err(y, y_ref, scale) <= 1e-13


@pytest.mark.parametrize("name", NAMES)
def test_closed_forms_match_their_arrays(name):
    """Every closed form the reference chose (linear, constant, branch, cycle-*) reproduces the
    array it replaces."""
    _, _, _, man = load_golden(name)
    for i in range(len(man.subs)):
        for nm, (arr, comp, _) in man.sub_arrays(i).items():
            if comp["kind"] != "none":
                assert plan_interp.closed_form_matches(arr, comp), (name, i, nm, comp)


def test_native_loop_matches_double_accumulation():
    m, x, _, _ = load_golden("uniform1024_f32_S5_K3")
    y_ref, scale = refdump.csr_ref(m, x)
    y = refdump.csr_native(m, x)
    refdump.assert_y(y, y_ref, scale, np.float32, "native f32 loop")
    m, x, _, _ = load_golden("laplace48_f64_S5_K3")
    y_ref, scale = refdump.csr_ref(m, x)
    refdump.assert_y(refdump.csr_native(m, x), y_ref, scale, np.float64, "native f64 loop")


def test_csr_ref_known_answer():
    """Hand-computed 3x3 case: y = A x."""
    from alphasparse_b200.matrices import CsrMatrix

    m = CsrMatrix(3, 3, np.array([0, 2, 2, 4], dtype=np.int64), np.array([0, 2, 1, 2], dtype=np.uint32),
                  np.array([2.0, -1.0, 0.5, 4.0]))
    x = np.array([1.0, 2.0, 3.0])
    y, sc = refdump.csr_ref(m, x)
    assert y.tolist() == [-1.0, 0.0, 13.0]
    assert sc.tolist() == [5.0, 0.0, 13.0]


@pytest.mark.skipif(not refdump.have_ref_dump(), reason="reference format oracle not built")
@pytest.mark.parametrize("name", ["uniform1024_f32_S2_K6", "laplace48_f64_S9_K9", "mixed4096_f32_sorted_split"])
def test_golden_regenerates_bit_identically(name):
    """The committed fixtures are what the reference host code produces today."""
    m, x, spec, man = load_golden(name)
    body = "\n".join(l for l in spec.splitlines() if not l.startswith("dtype"))
    again = refdump.run_ref_dump(m, body)
    assert again.meta == man.meta
    assert np.array_equal(again.blob, man.blob)
