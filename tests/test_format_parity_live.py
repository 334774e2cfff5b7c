"""CPU suite, part 4: native operators against the reference host code, run live.

Needs oracle/_ref/ref_dump (built from the reference tree by oracle/Makefile); skipped where
it is absent. Sweeps node parameters the committed fixtures do not cover."""
import numpy as np
import pytest

import refdump
from alphasparse_b200 import matrices as M
from alphasparse_b200.graph import Matrix
from test_format_parity import compare_with_manifest

pytestmark = pytest.mark.skipif(not refdump.have_ref_dump(), reason="reference format oracle not built")


def _uniform():
    return M.uniform_random(768, 12, seed=11)[0]


def _long_rows():
    rng = np.random.default_rng(5)
    return M.from_row_lengths(rng.integers(40, 300, size=512), 4096, seed=6, dtype=np.float64)[0]


def _mixed():
    rng = np.random.default_rng(7)
    lengths = np.concatenate([rng.integers(520, 900, size=16), rng.integers(130, 500, size=120), rng.integers(33, 127, size=400),
                              np.minimum(rng.zipf(2.0, size=3000), 31)])
    rng.shuffle(lengths)
    return M.from_row_lengths(lengths, 8192, seed=8)[0]


CASES = [
    ("uniform", _uniform, "dense compress\nsub all row_padding 192 1\nsub all blb_row_evenly 192\nsub all tlb_row\nsub all template K2"),
    ("uniform", _uniform, "dense compress\nsub all row_padding 64 1\nsub all blb_row_evenly 64\nsub all tlb_col_fixed 7\nsub all template K6"),
    ("uniform", _uniform, "dense compress\nsub all row_padding 32 1\nsub all blb_row_evenly 32\nsub all tlb_col_fixed 1\nsub all template K6"),
    ("uniform", _uniform, "dense compress\nsub all blb_row_nnz 128\nsub all tlb_col_fixed 2\nsub all template K6"),
    ("uniform", _uniform, "dense compress\nsub all tlb_nnz 2\nsub all template K9"),
    ("uniform", _uniform, "dense compress\nsub all tlb_nnz 7\nsub all template K10"),
    ("uniform", _uniform, "dense compress\nsub all tlb_nnz 16\nsub all template K9"),
    ("uniform", _uniform, "dense compress\nsub all blb_row_evenly 96\nsub all wlb_row_evenly 32\nsub all tlb_col_fixed 3\nsub all template K1"),
    ("uniform", _uniform, "dense compress\nsub all blb_row_evenly 128\nsub all wlb_row_evenly 8\nsub all tlb_row\nsub all template K5"),
    ("long", _long_rows, "dense compress\nsub all wlb_col_fixed 64\nsub all template K4"),
    ("long", _long_rows, "dense compress\nsub all wlb_col_fixed 96\nsub all template K4"),
    ("long", _long_rows, "dense compress\nsub all row_padding 2 1\nsub all blb_row_evenly 2\nsub all wlb_col_fixed 64\nsub all template K8"),
    ("long", _long_rows, "dense compress\nsub all blb_row_nnz 896\nsub all wlb_col_fixed 128\nsub all template K8"),
    ("long", _long_rows, "dense compress\nsub all blb_col_fixed 64\nsub all template K7"),
    ("long", _long_rows, "dense compress\nsub all blb_col_fixed 256\nsub all template K7"),
    ("long", _long_rows, "dense compress\nsub all row_padding 32 1\nsub all tlb_row\nsub all template K3"),
    ("mixed", _mixed, "dense sort 1\ndense compress\nsub all row_padding 64 1\nsub all blb_row_evenly 64\nsub all tlb_col_fixed 4\nsub all template K6"),
    ("mixed", _mixed, "dense sort 1\ndense compress\nsub all blb_col_fixed 128\nsub all template K7"),
    ("mixed", _mixed, "dense sort 1\ndense compress\nsub all wlb_col_fixed 32\nsub all template K4"),
    ("mixed", _mixed, "dense sort 1\ndense compress\nsub all blb_row_nnz 4096\nsub all wlb_col_fixed 32\nsub all template K8"),
    ("mixed", _mixed, "dense sort 1\ndense rowdiv_exp 128 4096 8\ndense compress\nsub all row_padding 32 1\nsub all blb_row_evenly 32\nsub all tlb_col_fixed 4\nsub all template K6"),
    ("mixed", _mixed, "dense sort 1\ndense rowdiv_exp 512 4096 16\ndense compress\nsub all blb_row_nnz 4096\nsub all wlb_col_fixed 64\nsub all template K8"),
    # one-bin coarse sort = stable partition that only moves rows without non-zeros to the end
    ("rmat", lambda: M.rmat(11, 8, seed=4)[0], "dense sort 1073741824\ndense compress\nsub all tlb_nnz 8\nsub all template K9"),
    ("rmat", lambda: M.rmat(11, 8, seed=4)[0], "dense sort 1073741824\ndense compress\nsub all tlb_nnz 32\nsub all template K10"),
]
_cache = {}


@pytest.mark.parametrize("idx", range(len(CASES)))
def test_native_equals_reference_live(idx):
    name, gen, spec = CASES[idx]
    if name not in _cache:
        _cache[name] = gen()
    m = _cache[name]
    man = refdump.run_ref_dump(m, spec)
    fmt = Matrix.from_csr(m).execute(spec)
    compare_with_manifest(fmt, man, f"{name}: {spec!r}")


def test_seeded_sweep_of_random_matrices_and_strategies():
    """60 seeded (matrix, strategy, sort) draws: wherever the reference runs to completion the native
    arrays equal its arrays bit for bit, except for the one documented repair (the SELL-like TLB-size
    array typed by its largest entry where the reference's type truncates it)."""
    import specs

    names = sorted(specs.COMPRESSED_SPECS)
    rng0 = np.random.default_rng(7)
    equal = aborted = repaired = 0
    for _ in range(60):
        seed = int(rng0.integers(0, 1 << 30))
        rng = np.random.default_rng(seed)
        n = int(rng.integers(300, 1500))
        kind = int(rng.integers(0, 3))
        if kind == 0:
            lengths = rng.integers(1, 14, size=n)
        elif kind == 1:
            lengths = np.minimum(rng.zipf(1.8, size=n), n // 3).clip(min=1)
        else:
            lengths = rng.integers(33, 160, size=n)
        m = M.from_row_lengths(lengths.astype(np.int64), n, seed=seed % 1000, dtype=[np.float32, np.float64][int(rng.integers(0, 2))])[0]
        spec = specs.full_spec(names[int(rng.integers(0, len(names)))], ["dense compress", "dense sort 1\ndense compress"][int(rng.integers(0, 2))])
        try:
            man = refdump.run_ref_dump(m, spec)
        except Exception:
            aborted += 1  # an assert of the reference on this input
            continue
        fmt = Matrix.from_csr(m).execute(spec)
        try:
            compare_with_manifest(fmt, man, f"seed {seed}: {spec!r}")
            equal += 1
        except AssertionError as e:
            ref_sizes = man.sub_arrays(0).get("thread_block_size_in_block")
            mine = fmt.arrays(0).get("thread_block_size_in_block")
            truncated = ref_sizes is not None and mine is not None and ref_sizes[0].dtype == np.uint8 and int(mine[0].max()) > 255
            assert truncated and "thread_block_size_in_block" in str(e), e
            repaired += 1
    assert equal >= 40 and equal + aborted + repaired == 60
