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
