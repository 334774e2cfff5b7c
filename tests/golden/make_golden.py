"""Regenerates the golden fixtures in this directory.

Runs the reference's own host pipeline (oracle/_ref/ref_dump, built from the reference
sources by oracle/Makefile) on small seeded matrices and stores, per case, the input CSR, x,
the graph spec, and every template array the reference produced (manifest + raw bytes).
Needs the reference tree; the fixtures themselves are what travels.

    python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

import refdump  # noqa: E402
import specs  # noqa: E402
from alphasparse_b200 import matrices as M  # noqa: E402


def save(name, m, x, spec, man):
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"),
        indptr=m.indptr, indices=m.indices, values=m.values, x=x, shape=np.array([m.n_rows, m.n_cols]),
        spec=np.frombuffer(spec.encode(), dtype=np.uint8), manifest=np.frombuffer(json.dumps(man.meta).encode(), dtype=np.uint8),
        blob=man.blob)


def mixed_rows():
    """4096 rows in shuffled order: a few very long rows, some long, some medium, many short
    (power-law-like), so that a descending sort + exponential row division yields four strips
    with at least three BLBs each (the reference aborts on strips with fewer)."""
    rng = np.random.default_rng(2)
    lengths = np.concatenate([
        rng.integers(520, 700, size=12), rng.integers(130, 400, size=100), rng.integers(33, 120, size=300),
        np.minimum(rng.zipf(2.1, size=4096 - 412), 31)])
    rng.shuffle(lengths)
    return M.from_row_lengths(lengths, 4096, seed=2)


def main():
    refdump.build_oracles()
    cases = []
    m, x = M.uniform_random(1024, 16, seed=0)
    for k in specs.COMPRESSED_SPECS:
        cases.append((f"uniform1024_f32_{k}", m, x, specs.full_spec(k)))
    m, x = M.laplacian_2d(48, seed=1)
    for k in ("S5_K3", "S1_K2", "S2_K6", "S9_K9", "S9_K10"):
        cases.append((f"laplace48_f64_{k}", m, x, specs.full_spec(k)))
    m, x = M.block_fem(128, 27, 32, seed=3)
    for k in ("S5_K3", "S4_K4", "S6_K8", "S8_K7"):
        cases.append((f"fem128_f64_{k}", m, x, specs.full_spec(k)))
    m, x = mixed_rows()
    cases.append(("mixed4096_f32_sorted_split", m, x, specs.SORTED_SPLIT_SPEC))
    cases.append(("mixed4096_f32_split", m, x, specs.SPLIT_SPEC))
    for name, m, x, spec in cases:
        man = refdump.run_ref_dump(m, spec)
        save(name, m, x, spec, man)
        print(name, m.nnz, len(man.blob))


if __name__ == "__main__":
    main()
