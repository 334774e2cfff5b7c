"""GPU suite: every template's CUDA kernel, through the C ABI, against the CPU y-oracle on the
golden fixtures (the reference's own arrays), plus launch-parameter sweeps and error paths."""
import ctypes as C

import numpy as np
import pytest

import refdump
from alphasparse_b200 import capi, matrices as M
from alphasparse_b200.graph import Matrix
from golden_util import golden_names, load_golden

pytestmark = pytest.mark.gpu
NAMES = golden_names()


def run_golden(ctx, name, launch=None):
    m, x, _, man = load_golden(name)
    descs, keep = refdump.plan_descs(man, launch)
    g = capi.PlanGroup(ctx, descs, keep)
    y = g.spmv_host(x)
    g.close()
    y_ref, scale = refdump.csr_ref(m, x)
    return y, y_ref, scale, m


@pytest.mark.parametrize("name", NAMES)
def test_template_matches_oracle(asp_ctx, name):
    y, y_ref, scale, m = run_golden(asp_ctx, name)
    refdump.assert_y(y, y_ref, scale, m.values.dtype, name)


LAUNCHES = {
    "K2": [(7, 32), (1000, 64), (3, 256)],
    "K3": [(1, 32), (5, 64), (400, 256), (2, 1024)],
    "K4": [(1, 32), (33, 96), (999, 512)],
    "K6": [(1, 32, 1), (9, 128, 4), (77, 704, 16), (500, 64, 32), (5, 96, 2)],
    "K7": [(1, 32), (13, 320), (2000, 1024)],
    "K8": [(3, 64, 1), (50, 288, 2), (640, 128, 32)],
    "K9": [(1, 64), (9, 256)],
    "K10": [(1, 32), (1, 512)],
    "K1": [(2, 64), (70, 512)],
    "K5": [(2, 64, 1), (70, 512, 8)],
}


@pytest.mark.parametrize("name", [n for n in NAMES if n.startswith("uniform1024")])
def test_launch_parameters_do_not_change_y(asp_ctx, name):
    """Any tblock_num / thread_num_in_block / thread_num_of_row_reduce the tuner may try gives
    the same y (grid-stride loops cover what the grid does not)."""
    m, x, _, man = load_golden(name)
    y_ref, scale = refdump.csr_ref(m, x)
    descs, keep = refdump.plan_descs(man)
    g = capi.PlanGroup(asp_ctx, descs, keep)
    t = man.subs[0]["template"]
    for lp in LAUNCHES[t]:
        tb, th = lp[0], lp[1]
        g.set_launch(0, tb, th, lp[2] if len(lp) > 2 else 1)
        y = g.spmv_host(x)
        refdump.assert_y(y, y_ref, scale, np.float32, f"{name} launch {lp}")
    g.close()


def test_device_pointer_entry_and_timing(asp_ctx):
    import torch

    m, x, _, man = load_golden("laplace48_f64_S5_K3")
    descs, keep = refdump.plan_descs(man)
    g = capi.PlanGroup(asp_ctx, descs, keep)
    dx = torch.from_numpy(x).cuda()
    dy = torch.full((m.n_rows,), 7.0, dtype=torch.float64, device="cuda")
    torch.cuda.synchronize()
    g.spmv(dx.data_ptr(), dy.data_ptr(), zero_y=True)
    asp_ctx.synchronize()
    y_ref, scale = refdump.csr_ref(m, x)
    refdump.assert_y(dy.cpu().numpy(), y_ref, scale, np.float64, "device-pointer spmv")
    ms, gf = g.time(warmup=2, reps=5)
    assert ms > 0 and gf > 0
    with pytest.raises(capi.AspError) as ei:
        g.time(warmup=1, reps=2, gflops_up_bound=1e-9)
    assert ei.value.status == 6
    g.close()


def test_atomic_plans_accumulate_when_y_is_not_cleared(asp_ctx):
    """The reference never clears y between repeats; with zero_y=0 an atomic plan adds to y."""
    import torch

    m, x, _, man = load_golden("uniform1024_f32_S8_K7")
    descs, keep = refdump.plan_descs(man)
    descs[0].is_atom_add = 1
    g = capi.PlanGroup(asp_ctx, descs, keep)
    dx = torch.from_numpy(x).cuda()
    dy = torch.zeros(m.n_rows, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    g.spmv(dx.data_ptr(), dy.data_ptr(), zero_y=False)
    g.spmv(dx.data_ptr(), dy.data_ptr(), zero_y=False)
    asp_ctx.synchronize()
    y_ref, scale = refdump.csr_ref(m, x)
    refdump.assert_y(dy.cpu().numpy() / 2, y_ref, scale, np.float32, "two accumulating passes")
    g.close()


def test_error_paths(asp_ctx):
    m, x, _, man = load_golden("uniform1024_f32_S5_K3")
    descs, keep = refdump.plan_descs(man)
    # wrong TLB size: #TLB * size != padded nnz
    descs[0].tlb_size += 1
    with pytest.raises(capi.AspError) as ei:
        capi.PlanGroup(asp_ctx, descs, keep)
    assert ei.value.status == 5
    descs, keep = refdump.plan_descs(man)
    descs[0].val_dtype = capi.F64  # val_arr is f32
    with pytest.raises(capi.AspError) as ei:
        capi.PlanGroup(asp_ctx, descs, keep)
    assert ei.value.status == 1
    descs, keep = refdump.plan_descs(man)
    descs[0].n_arrays = 1  # row map only: val / col missing
    with pytest.raises(capi.AspError):
        capi.PlanGroup(asp_ctx, descs, keep)
    descs, keep = refdump.plan_descs(man)
    g = capi.PlanGroup(asp_ctx, descs, keep)
    with pytest.raises(capi.AspError):
        g.set_launch(0, 10, 2048, 1)
    # the context is still usable after every rejected call
    y = g.spmv_host(x)
    y_ref, scale = refdump.csr_ref(m, x)
    refdump.assert_y(y, y_ref, scale, np.float32, "after errors")
    g.close()


def test_empty_template_is_skipped(asp_ctx):
    m, x, _, man = load_golden("mixed4096_f32_split")
    descs, keep = refdump.plan_descs(man)
    y_ref, scale = refdump.csr_ref(m, x)
    full = capi.PlanGroup(asp_ctx, descs, keep)
    y_full = full.spmv_host(x)
    refdump.assert_y(y_full, y_ref, scale, np.float32, "all strips")
    full.close()
    # mute strip 0 the way the tuner does with EMPTY_TEMPLATE: its rows stay zero
    descs, keep = refdump.plan_descs(man)
    descs[0].template_type = capi.TEMPLATE["EMPTY"]
    part = capi.PlanGroup(asp_ctx, descs, keep)
    y = part.spmv_host(x)
    s0 = man.subs[0]
    assert np.all(y[s0["min_row"] : s0["max_row"] + 1] == 0)
    assert np.array_equal(y[s0["max_row"] + 1 :], y_full[s0["max_row"] + 1 :])
    part.close()


def test_fp64_group_whose_first_strip_is_empty(asp_ctx):
    """The host-buffer entry points size x and y from the group, not from plans[0]: an fp64 matrix
    whose strip 0 carries the EMPTY template (what the search builds for every strip but the one it
    is timing) must still move 8-byte elements."""
    m, x = M.rmat(10, 6, seed=4)
    m64 = M.CsrMatrix(m.n_rows, m.n_cols, m.indptr, m.indices, m.values.astype(np.float64))
    x64 = x.astype(np.float64)
    hm = Matrix.from_csr(m64)
    cm = hm.dense("dense sort 1\ndense rowdiv_exp 32 4096 4\ndense compress")
    assert cm.n_subs >= 2
    lines = ["sub 0 template EMPTY"]
    for i in range(1, cm.n_subs):
        lines += [f"sub {i} row_padding 32 1", f"sub {i} tlb_row", f"sub {i} template K3"]
    fmt = cm.execute("\n".join(lines))
    g = fmt.upload(capi.Context(0))  # a fresh context: its staging buffers start empty
    y_ref, scale = refdump.csr_ref(m64, x64)
    info0 = fmt.sub_info(0)
    perm = fmt.global_perm()
    rows0 = perm[info0.min_row : info0.max_row + 1].astype(np.int64)  # original rows of strip 0
    keep_rows = np.ones(m.n_rows, dtype=bool)
    keep_rows[rows0] = False
    for fn in (g.spmv_host, g.spmv_host_static, g.spmv_host):
        y = fn(x64)
        assert y.dtype == np.float64 and np.all(y[rows0] == 0)
        assert refdump.rel_err(y[keep_rows], y_ref[keep_rows], scale[keep_rows]) <= refdump.TOL[np.dtype(np.float64)]
    g.close()
    fmt.close()


def test_group_of_empty_templates_yields_zeros(asp_ctx):
    """A group in which every strip is EMPTY is the zero matrix: y must come back cleared, not as
    whatever the staging buffer held from the previous call."""
    m, x, _, man = load_golden("uniform1024_f32_S5_K3")
    descs, keep = refdump.plan_descs(man)
    live = capi.PlanGroup(asp_ctx, descs, keep)
    assert np.abs(live.spmv_host(x)).max() > 0 and np.abs(live.spmv_host_static(x)).max() > 0  # leaves non-zero results behind
    descs2, keep2 = refdump.plan_descs(man)
    descs2[0].template_type = capi.TEMPLATE["EMPTY"]
    dead = capi.PlanGroup(asp_ctx, descs2, keep2)
    assert np.all(dead.spmv_host(x) == 0)
    assert np.all(dead.spmv_host_static(x) == 0)
    import torch

    dx = torch.from_numpy(x).cuda()
    dy = torch.full((m.n_rows,), 7.0, dtype=torch.float32, device="cuda")
    dead.spmv(dx.data_ptr(), dy.data_ptr(), "auto")
    asp_ctx.synchronize()
    assert float(dy.abs().max()) == 0.0
    live.close()
    dead.close()


def test_reported_launch_is_the_launch_used(asp_ctx):
    """asp_plan_get_launch: requests the kernels fold into an equivalent launch are reported as such."""
    _, _, _, man = load_golden("uniform1024_f32_S5_K3")
    descs, keep = refdump.plan_descs(man)
    g = capi.PlanGroup(asp_ctx, descs, keep)
    g.set_launch(0, 4, 1024, 1)
    tb, th, _ = g.get_launch(0)
    assert th == 512 and tb >= 1  # the ELL-like kernel is compiled for at most 512 threads per CTA
    g.set_launch(0, 1000000, 128, 1)
    tb, th, _ = g.get_launch(0)
    assert th == 128 and tb * th * 4 < 1024 * 4 + 128 * 4  # never more CTAs than work (4 TLBs per thread)
    g.close()


def test_a_bad_column_never_reaches_a_kernel(asp_ctx):
    m, x, _, man = load_golden("uniform1024_f32_S9_K9")
    descs, keep = refdump.plan_descs(man)
    descs[0].n_cols = 512  # x shorter than the columns the arrays name
    with pytest.raises(capi.AspError) as e:
        capi.PlanGroup(asp_ctx, descs, keep)
    assert e.value.status == 5 and "column outside x" in str(e.value)
