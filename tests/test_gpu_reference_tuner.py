"""GPU suite: the reference's own tuner, unmodified, timing the hand-written kernels.

oracle/_ref/ref_tune is the reference's host code (compiled from its sources where they lie) linked with
oracle/ref_shim_executor.cc in place of its executor.cc: the two functions through which the tuner reaches the GPU
(executor.hpp:12-22) lower every template struct to an asp_plan_desc and call asp_plan_group_create / asp_time.
Its whitelist strategies then run as they always did (find_best_path_of_white_list_strategy1 / 5 / 9 / 2 on
BASELINE config 1, find_best_param_of_<template> sweeping the launch parameters, default_auto_tuner.cc:449-2030),
and what they time is the sm_100a kernel family of each template. The fastest trial's y, computed through
asp_spmv_host from the reference-built arrays, must match the CPU oracle.
"""
import os
import subprocess

import numpy as np
import pytest

import refdump
from alphasparse_b200 import matrices as M
from alphasparse_b200.matrices import write_mtx_coo

REF_TUNE = os.path.join(refdump.REF_DIR, "ref_tune")
pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not os.path.exists(REF_TUNE), reason="oracle/_ref/ref_tune not built")]

# template_type of the reference (code_builder.hpp:15-29) each strategy ends in
EXPECT = {1: {1}, 5: {2}, 9: {8, 9}, 2: {4}}


@pytest.fixture(scope="module")
def c1(tmp_path_factory):
    d = tmp_path_factory.mktemp("c1")
    m, x = M.uniform_random(4096, 16, 0)  # BASELINE config 1
    write_mtx_coo(str(d / "c1.mtx.coo"), m)
    x.astype(np.float32).tofile(str(d / "x.bin"))
    return d, m, x


@pytest.mark.parametrize("strategy", [1, 5, 9, 2])
def test_reference_strategy_times_the_new_kernels_and_its_winner_is_correct(c1, strategy):
    d, m, x = c1
    rec, yf = str(d / f"rec_{strategy}.txt"), str(d / f"y_{strategy}.bin")
    env = dict(os.environ, ASP_SHIM_RECORD=rec, ASP_SHIM_X=str(d / "x.bin"), ASP_SHIM_Y=yf)
    env.pop("ASP_SHIM_NO_GPU", None)
    r = subprocess.run([REF_TUNE, str(d / "c1.mtx.coo"), "float", str(strategy)], cwd=refdump.REF_DIR, env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-1500:]
    last = r.stdout.strip().splitlines()[-1].split()  # "strategy k ms T gflops G template t"
    ms, gflops, templ = float(last[3]), float(last[5]), int(last[7])
    assert gflops > 0 and 0 < ms < 10 and templ in EXPECT[strategy], last
    trials = [l.split(";") for l in open(rec).read().splitlines()]
    assert len(trials) >= 4 and all(float(t[9]) > 0 for t in trials), "every trial the tuner made ran on the GPU"
    assert {int(t[0]) for t in trials} == EXPECT[strategy]
    y = np.fromfile(yf, dtype=np.float32)
    y_ref, scale = refdump.csr_ref(m, x)
    if strategy == 2:
        # The reference's row-grouped template leaves the values and columns of its LAST row strip un-interleaved
        # (shared_memory_op_warp_compress.cc:472 stops one BLB early; the strip is uninitialised heap memory), so the
        # arrays it hands over do not describe the last strip's rows (at most 64 of them here). Everything before is A.
        keep = slice(0, m.n_rows - 64)
        assert refdump.rel_err(y[keep], y_ref[keep], scale[keep]) <= refdump.TOL[np.dtype(np.float32)]
        return
    refdump.assert_y(y, y_ref, scale, np.float32, f"winner of reference strategy {strategy}")
