"""CPU suite, part 3: the native format operators against the reference's own host code.

For every golden fixture the native Operator Graph is run on the same matrix with the same
spec; every template array (bytes, element type, length), every closed form, every scalar and
flag, the dense block table and the global row permutation must equal what the reference
produced. Value arrays are compared against reference dumps made with the two value defects of
the reference repaired (see oracle/ref_dump.cc: fix_values)."""
import numpy as np
import pytest

import refdump
from alphasparse_b200 import capi
from alphasparse_b200.graph import Matrix
from golden_util import golden_names, load_golden

NAMES = golden_names()
SKIP_ARRAYS = {"first_relative_reduce_row_of_thread_level_block", "tmp_result_reduce_offset_of_thread_level_block"}
IMPLEMENTED = {"K1", "K2", "K3", "K4", "K5", "K6", "K7", "K8", "K9", "K10"}


def compare_with_manifest(fmt, man, what):
    meta = man.meta
    assert fmt.n_subs == len(man.subs), what
    perm_ref = man.global_perm()
    perm = fmt.global_perm()
    if perm_ref is None:
        assert perm is None, what
    else:
        assert perm is not None and perm.dtype == perm_ref.dtype and np.array_equal(perm, perm_ref), f"{what}: sorted_row_index"
    descs = fmt.plan_descs()
    for i, s in enumerate(man.subs):
        info = fmt.sub_info(i)
        for k in ("min_row", "max_row", "min_col", "max_col"):
            assert getattr(info, k) == s[k], f"{what} sub {i}: {k}"
        assert info.begin_coo == s["begin_coo"] and info.end_coo == s["end_coo"], f"{what} sub {i}: coo range"
        assert (info.n_blb, info.n_wlb, info.n_tlb) == (s["n_blb"], s["n_wlb"], s["n_tlb"]), f"{what} sub {i}: block counts"
        d = descs[i]
        assert d.template_type == capi.TEMPLATE[s["template"]]
        assert d.first_row == s["first_row"] and d.first_col == s["first_col"]
        assert d.is_atom_add == s.get("is_atom_add", s.get("is_all_force_atom_add", 0)), f"{what} sub {i}: is_atom_add"
        assert d.sort_kind == (capi.SORT_GLOBAL if s["global_sort"] else capi.SORT_LOCAL if s["local_sort"] else capi.SORT_NONE)
        eff = s.get("effective_TLB_num", s.get("effective_WLB_num", s.get("effective_row_num")))
        if eff is not None:
            assert d.effective_num == eff, f"{what} sub {i}: effective count {d.effective_num} != {eff}"
        tl = s.get("thread_block_size_in_block", s.get("tlb_size"))
        if tl is not None:
            assert d.tlb_size == tl
        for k in ("bits_word", "bits_flag", "bits_row", "bits_off"):
            if k in s:
                assert getattr(d, k) == s[k], f"{what} sub {i}: {k}"
        assert d.tblock_num == s.get("tblock", d.tblock_num) and d.thread_num_in_block == s["threads"]
        mine = fmt.arrays(i)
        ref = {k: v for k, v in man.sub_arrays(i).items() if k not in SKIP_ARRAYS}
        assert set(mine) == set(ref), f"{what} sub {i}: arrays {sorted(mine)} vs {sorted(ref)}"
        for name, (rarr, rcomp, rdesc) in ref.items():
            arr, comp, dt, ln = mine[name]
            assert ln == rdesc["len"], f"{what} sub {i} {name}: length {ln} != {rdesc['len']}"
            assert arr.dtype == rarr.dtype, f"{what} sub {i} {name}: dtype {arr.dtype} != {rarr.dtype}"
            assert comp == rcomp, f"{what} sub {i} {name}: closed form {comp} != {rcomp}"
            assert np.array_equal(arr.view(np.uint8), rarr.view(np.uint8)), f"{what} sub {i} {name}: contents differ"


@pytest.mark.parametrize("name", NAMES)
def test_native_format_equals_reference(name):
    m, x, spec, man = load_golden(name)
    if any(s["template"] not in IMPLEMENTED for s in man.subs):
        pytest.skip("template lowering not implemented yet")
    fmt = Matrix.from_csr(m).execute(spec)
    compare_with_manifest(fmt, man, name)
