"""CPU suite: asp_search enumerates the search space of the reference's own tuner.

The reference's tuner is run here unmodified (oracle/_ref/ref_tune: its whitelist dispatcher
find_best_path_of_compressed_sub_matrix, whilte_list_path_impl.cc:3411, over the compressed view of the
whole matrix) with oracle/ref_shim_executor.cc in place of its executor.cc, in recording mode: every trial
it hands to part_execute_code_builder (executor.hpp:12-22) is logged as a fingerprint -- template, #BLB,
#WLB, #TLB, padded non-zeros, tblock_num, thread_num_in_block, thread_num_of_row_reduce -- and "runs" in a
constant time, so nothing steers the enumeration. asp_search in its exact mode (quick = 2), with a timer that
records the same fingerprint, must visit the same set of points: same node-parameter grids (param_enumerater
ranges), same derived launch sweeps, same padding gate, same formats.
"""
import os
import subprocess

import numpy as np
import pytest

import refdump
from alphasparse_b200 import capi, matrices as M, tuner
from alphasparse_b200.matrices import write_mtx_coo

REF_TUNE = os.path.join(refdump.REF_DIR, "ref_tune")
pytestmark = pytest.mark.skipif(not os.path.exists(REF_TUNE), reason="oracle/_ref/ref_tune not built (needs the reference tree)")

K10 = capi.TEMPLATE["K10"]


def reference_points(m, tmp_path, which="all"):
    """Fingerprints of every trial the reference's tuner makes; None when the reference aborts on this input."""
    mtx = str(tmp_path / "m.mtx.coo")
    rec = str(tmp_path / f"trials_{which}.txt")
    if not os.path.exists(mtx):
        write_mtx_coo(mtx, m)
    env = dict(os.environ, ASP_SHIM_NO_GPU="1", ASP_SHIM_RECORD=rec)
    r = subprocess.run([REF_TUNE, mtx, "double" if m.values.dtype == np.float64 else "float", str(which)], cwd=refdump.REF_DIR, env=env,
                       stdout=subprocess.DEVNULL, stderr=subprocess.PIPE, timeout=1200)
    if r.returncode != 0:
        assert b"Assertion" in r.stderr, r.stderr.decode()[-800:]  # one of the reference's own asserts, nothing else
        return None
    if not os.path.exists(rec):
        return set()
    pts = set()
    for line in open(rec):
        t, blb, wlb, tlb, padded, tb, th, rd = (int(v) for v in line.split(";")[:8])
        pts.add((t, blb, wlb, tlb, padded, 0 if t == K10 else tb, th, rd))  # the second CSR5-like template has no tblock_num
    return pts


def native_points(m, quick, strategies=None):
    pts = set()

    def timer(fmt, tb, th, rd):
        if fmt.n_subs == 1 and fmt.global_perm() is None:  # the compress-only dense view: what the reference run covers
            info = fmt.sub_info(0)
            padded = fmt.arrays(0)["val_arr"][3]
            t = info.template_type
            pts.add((t, info.n_blb, info.n_wlb, info.n_tlb, padded, 0 if t == K10 else tb[0], th[0], rd[0]))
        return 1.0

    try:
        tuner.search_with_timer(m, timer, quick=quick, strategies=strategies)
    except capi.AspError:
        pass  # no strategy of the requested ones applies to this matrix
    return pts


def rows_between(lo, hi, n_rows, n_cols, seed):
    rng = np.random.default_rng(seed)
    return M.from_row_lengths(rng.integers(lo, hi + 1, size=n_rows), n_cols, seed=seed)


CASES = {
    # BASELINE config 1: rows of ~5..35 non-zeros -> strategies 1, 5, 9, 2, 3
    "c1_uniform4096": lambda: M.uniform_random(4096, 16, 0),
    # rows of 40..120 -> adds strategies 4, 6, 7
    "rows_40_120": lambda: rows_between(40, 120, 3000, 6000, 7),
    # rows of 150..900 -> strategy 8 (long rows), 6, 7, 2, 3
    "rows_150_900": lambda: rows_between(150, 900, 700, 5000, 8),
}


# which whitelist strategies the dispatcher's gates admit (whilte_list_path_impl.cc:3453-3958) for each case
ADMITTED = {"c1_uniform4096": (1, 5, 9, 2, 3), "rows_40_120": (1, 5, 9, 4, 6, 7, 2, 3), "rows_150_900": (8, 6, 7, 2, 3, 9)}


@pytest.mark.parametrize("case", sorted(CASES))
def test_exact_mode_visits_the_reference_tuners_points(case, tmp_path):
    """Strategy by strategy (the reference's own drivers run them one at a time too, main.cc:368-443). Where the
    reference aborts on one of its asserts -- strategy 7 does on every matrix tried here, `row_block_size_of_this_block_vec
    .size() > 1` in sep_warp_level_row_csr, op_manager.cc:2029 -- there is nothing to compare with; the native loop
    runs those points (and the GPU tests check their results)."""
    m, _ = CASES[case]()
    compared, total = [], 0
    for k in ADMITTED[case]:
        ref = reference_points(m, tmp_path, k)
        if ref is None:
            continue
        got = native_points(m, quick=2, strategies=[k])
        missing, extra = sorted(ref - got), sorted(got - ref)
        assert not missing and not extra, f"{case} strategy {k}: {len(ref)} reference points, {len(got)} native; missing {missing[:6]} extra {extra[:6]}"
        compared.append(k)
        total += len(ref)
    assert len(compared) >= len(ADMITTED[case]) - 1 and total > 20, (compared, total)


def test_the_dispatcher_as_a_whole_on_baseline_config_1(tmp_path):
    m, _ = CASES["c1_uniform4096"]()
    ref = reference_points(m, tmp_path, "all")
    assert ref is not None and len(ref) == 170
    assert native_points(m, quick=2) == ref


def test_default_full_mode_is_the_reference_space_plus_named_extensions(tmp_path):
    m, _ = CASES["c1_uniform4096"]()
    ref = reference_points(m, tmp_path)
    got = native_points(m, quick=0)
    assert ref <= got, sorted(ref - got)[:8]
    k9, k10 = capi.TEMPLATE["K9"], capi.TEMPLATE["K10"]
    for p in got - ref:
        # extensions: TLB size 32 for the CSR5-like templates, and their staged write-out (third launch parameter 2)
        assert p[0] in (k9, k10) and (p[7] == 2 or p[4] // p[3] >= 30), p
