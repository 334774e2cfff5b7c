"""GPU test of asp_spmv_host_static, the host-buffer SpMV that allocates nothing.

Some callers cannot let this library call cudaMalloc: a solver that has given all device memory
to its own pool, or a loop that cannot afford the device-wide synchronisation an allocation
implies. For them x and y are staged in a fixed device array instead of in buffers grown on
demand. The result must equal asp_spmv_host's, call after call: the array is shared and keeps
the previous call's contents, so the second call (with another x) would show stale data if the
entry point did not clear and overwrite what it must.

Collected last on purpose, so that a run stopping at the first failure has run everything else.
"""
import numpy as np
import pytest

import refdump
from alphasparse_b200 import capi
from golden_util import load_golden

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["uniform1024_f32_S5_K3", "uniform1024_f32_S8_K7", "laplace48_f64_S9_K9"])
def test_static_staging_matches_allocating_entry_point(name):
    m, x, _, man = load_golden(name)
    ctx = capi.Context(0)
    descs, keep = refdump.plan_descs(man)
    if name.endswith("S8_K7"):
        descs[0].is_atom_add = 1  # make the kernel accumulate into y: a stale y would be visible
    g = capi.PlanGroup(ctx, descs, keep)
    y_ref, scale = refdump.csr_ref(m, x)
    tol = refdump.TOL[np.dtype(m.values.dtype)]
    for k, xx in enumerate((x, (2.0 * x + 0.25).astype(x.dtype))):  # two calls in a row, different x
        want = g.spmv_host(xx)
        got = g.spmv_host_static(xx)
        _, scale_k = refdump.csr_ref(m, xx)
        err = refdump.rel_err(got, want.astype(np.float64), scale_k)
        assert err <= tol, f"{name} call {k}: static vs allocating entry point differ by {err:.3e}"
    refdump.assert_y(g.spmv_host_static(x), y_ref, scale, m.values.dtype, name + " vs oracle")
    g.close()
    ctx.close()


def test_static_staging_rejects_oversized_matrices():
    m, x, _, man = load_golden("uniform1024_f32_S5_K3")
    ctx = capi.Context(0)
    descs, keep = refdump.plan_descs(man)
    half = capi.lib().asp_static_stage_bytes() // 2
    descs[0].n_cols = half // 4 + 1  # one f32 element more than the x half holds
    g = capi.PlanGroup(ctx, descs, keep)
    big_x = np.zeros(int(descs[0].n_cols), dtype=np.float32)
    y = np.empty(m.n_rows, dtype=np.float32)
    import ctypes as C

    st = capi.lib().asp_spmv_host_static(ctx.handle, g._plans, g.n, C.c_void_p(big_x.ctypes.data), C.c_void_p(y.ctypes.data))
    assert st == 1
    assert b"static staging area" in capi.lib().asp_last_error()
    g.close()
    ctx.close()
