"""CPU suite, part 2: the C-ABI library loads and exports every declared entry point."""
import os
import re

from alphasparse_b200 import capi


def declared_functions(header="asp_b200.h"):
    hdr = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", header)
    text = open(hdr).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(asp_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    L = capi.lib()
    names = declared_functions()
    assert len(names) >= 15
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/asp_b200.h but not exported"


def test_binding_covers_header():
    assert set(capi.EXPORTS) <= set(declared_functions())


def test_host_header_symbols_are_exported_and_bound():
    from alphasparse_b200 import graph

    L = capi.lib()
    names = [n for n in declared_functions("asp_b200_host.h") if n not in ("asp_time_fn",)]
    assert len(names) >= 25
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/asp_b200_host.h but not exported"
    assert set(graph.HOST_EXPORTS) <= set(names)


def test_built_for_sm100a():
    assert capi.lib().asp_built_for_sm100a() == 1


def test_status_strings():
    L = capi.lib()
    assert L.asp_status_str(0) == b"ok"
    assert L.asp_status_str(5) == b"format array out of bounds"
    assert L.asp_status_str(7) == b"bounded device-side wait expired"


def test_argument_errors_of_the_multi_gpu_entry_points_need_no_device():
    """Bad arguments are refused before anything is launched: more ranks than the barrier has lanes for, a rank
    outside the group, NULL buffers."""
    import ctypes as C

    L = capi.lib()
    buf = (C.c_uint32 * 64)()
    p = C.cast(buf, C.c_void_p)
    assert L.asp_rank_barrier(p, p, 0, 33, 1, p, 0, None) == 1   # world > 32
    assert L.asp_rank_barrier(p, p, 2, 2, 1, p, 0, None) == 1    # rank outside the group
    assert L.asp_rank_barrier(None, p, 0, 2, 1, p, 0, None) == 1
    assert L.asp_spmv_publish(None, None, 0, None, None, None) == 1
    assert L.asp_multicast_store(None, None, 16, None, 0) == 1
    assert L.asp_multicast_store(p, p, 0, None, 0) == 0          # nothing to store
    assert L.asp_plan_descs_validate(None, 0) == 1
    # the native loop of the sharded SpMV
    out = C.c_void_p(1)
    assert L.asp_dist_create(None, None, C.byref(out)) == 1 and not out.value
    assert L.asp_dist_spmv(None, p, p, p) == 1
    assert L.asp_dist_spmv_iter(None, p, None, None, 1, None) == 1
    assert L.asp_dist_status(None, None) == 1
    L.asp_dist_destroy(None)
    assert L.asp_spmv_host_pipelined(None, None, 0, p, p) == 1
