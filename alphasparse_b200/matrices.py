"""Seeded synthetic inputs for the five benchmark configurations, and the `.mtx.coo` text format.

The reference was evaluated on SuiteSparse matrices that are not available offline; these
generators stand in for them with the shapes and distributions the benchmark configs name.
Every generator returns a `CsrMatrix` (row offsets int64, column indices uint32, values in
the config's dtype) plus the dense vector x, and is deterministic in its seed.

`.mtx.coo` grammar (reference `struct.cc:92-174`): first line `rows cols ...`, then one
`row col val` triple per line, 1-based, sorted by row then column, single-space separated.
"""
from __future__ import annotations

import dataclasses

import numpy as np


@dataclasses.dataclass
class CsrMatrix:
    n_rows: int
    n_cols: int
    indptr: np.ndarray  # int64 [n_rows + 1]
    indices: np.ndarray  # uint32 [nnz], sorted within a row
    values: np.ndarray  # float32 | float64 [nnz]

    @property
    def nnz(self) -> int:
        return int(self.indptr[-1])

    @property
    def dtype(self):
        return self.values.dtype

    def row_lengths(self) -> np.ndarray:
        return np.diff(self.indptr)

    def algorithmic_bytes(self) -> int:
        """Canonical-CSR bytes of one SpMV: nnz*(s_v+4) + 4*(M+1) + s_v*(N+M)."""
        sv = self.values.dtype.itemsize
        return self.nnz * (sv + 4) + 4 * (self.n_rows + 1) + sv * (self.n_cols + self.n_rows)

    def row_slice(self, r0: int, r1: int) -> "CsrMatrix":
        a, b = int(self.indptr[r0]), int(self.indptr[r1])
        return CsrMatrix(r1 - r0, self.n_cols, self.indptr[r0 : r1 + 1] - a, self.indices[a:b], self.values[a:b])


def _from_lengths(lengths: np.ndarray) -> np.ndarray:
    indptr = np.zeros(lengths.shape[0] + 1, dtype=np.int64)
    np.cumsum(lengths, out=indptr[1:])
    return indptr


def _sorted_unique_columns(rng, lengths: np.ndarray, n_cols: int):
    """Uniform columns, sorted inside each row; duplicates inside a row are dropped."""
    indptr = _from_lengths(lengths)
    nnz = int(indptr[-1])
    rows = np.repeat(np.arange(lengths.shape[0], dtype=np.int64), lengths)
    cols = rng.integers(0, n_cols, size=nnz, dtype=np.int64)
    key = rows * np.int64(n_cols) + cols
    key.sort()
    keep = np.ones(nnz, dtype=bool)
    keep[1:] = key[1:] != key[:-1]
    key = key[keep]
    rows = key // n_cols
    cols = (key - rows * n_cols).astype(np.uint32)
    new_len = np.bincount(rows, minlength=lengths.shape[0]).astype(np.int64)
    return _from_lengths(new_len), cols


def from_row_lengths(lengths, n_cols: int, seed: int, dtype=np.float32):
    """A matrix with the given row lengths (before duplicate-column removal), uniform sorted
    columns, values and x ~ U[-1,1]. Used for small hand-shaped test matrices."""
    rng = np.random.default_rng(seed)
    lengths = np.asarray(lengths, dtype=np.int64)
    indptr, cols = _sorted_unique_columns(rng, lengths, n_cols)
    vals = rng.uniform(-1.0, 1.0, size=cols.shape[0]).astype(dtype)
    x = rng.uniform(-1.0, 1.0, size=n_cols).astype(dtype)
    return CsrMatrix(lengths.shape[0], n_cols, indptr, cols, vals), x


def uniform_random(n: int = 4096, mean_nnz: float = 16.0, seed: int = 0, dtype=np.float32):
    """Config 1: per-row nnz ~ Poisson(mean) clipped to >= 1 (the reference rejects empty rows,
    main.cc:604-621), columns uniform without replacement and sorted, values and x ~ U[-1,1]."""
    rng = np.random.default_rng(seed)
    lengths = np.maximum(rng.poisson(mean_nnz, size=n), 1).astype(np.int64)
    lengths = np.minimum(lengths, n)
    indptr = _from_lengths(lengths)
    cols = np.empty(int(indptr[-1]), dtype=np.uint32)
    for r in range(n):
        c = rng.choice(n, size=int(lengths[r]), replace=False)
        c.sort()
        cols[indptr[r] : indptr[r + 1]] = c
    vals = rng.uniform(-1.0, 1.0, size=cols.shape[0]).astype(dtype)
    x = rng.uniform(-1.0, 1.0, size=n).astype(dtype)
    return CsrMatrix(n, n, indptr, cols, vals), x


def laplacian_2d(grid: int = 2048, seed: int = 1, dtype=np.float64, grid_y: int | None = None, rows: tuple | None = None):
    """Config 2: 5-point Laplacian on a grid x grid_y mesh, natural ordering, diagonal 4,
    neighbours -1; x ~ U[-1,1]. Row i = iy*grid + ix. With rows=(r0, r1) only that row block is
    built (global column indices, the full x): what one rank of a sharded run needs."""
    gx = grid
    gy = grid if grid_y is None else grid_y
    n = gx * gy
    r0, r1 = (0, n) if rows is None else (int(rows[0]), int(rows[1]))
    i = np.arange(r0, r1, dtype=np.int64)
    ix = i % gx
    iy = i // gx
    # candidate neighbours in ascending column order: i-gx, i-1, i, i+1, i+gx
    cand = np.stack([i - gx, i - 1, i, i + 1, i + gx], axis=1)
    ok = np.stack([iy > 0, ix > 0, np.ones(i.shape[0], bool), ix < gx - 1, iy < gy - 1], axis=1)
    val = np.array([-1.0, -1.0, 4.0, -1.0, -1.0], dtype=dtype)
    lengths = ok.sum(axis=1).astype(np.int64)
    indptr = _from_lengths(lengths)
    cols = cand[ok].astype(np.uint32)
    vals = np.broadcast_to(val, (i.shape[0], 5))[ok].astype(dtype)
    rng = np.random.default_rng(seed)
    x = rng.uniform(-1.0, 1.0, size=n).astype(dtype)
    return CsrMatrix(r1 - r0, n, indptr, cols, vals), x


def power_law(n: int = 8_388_608, exponent: float = 2.1, cap: int = 500_000, seed: int = 2, dtype=np.float32):
    """Config 3: row lengths ~ min(Zipf(exponent), cap) (min 1), columns uniform and sorted per
    row (duplicates dropped), values and x ~ U[-1,1]."""
    rng = np.random.default_rng(seed)
    lengths = np.minimum(rng.zipf(exponent, size=n), min(cap, n)).astype(np.int64)
    indptr, cols = _sorted_unique_columns(rng, lengths, n)
    vals = rng.uniform(-1.0, 1.0, size=cols.shape[0]).astype(dtype)
    x = rng.uniform(-1.0, 1.0, size=n).astype(dtype)
    return CsrMatrix(n, n, indptr, cols, vals), x


def block_fem(block_rows: int = 1_048_576, blocks_per_row: int = 27, half_band: int = 4096, seed: int = 3, dtype=np.float64):
    """Config 4: dense 3x3 blocks, `blocks_per_row` blocks per block row at distinct block
    columns inside a window of 2*half_band+1 block columns around the diagonal (the window is
    shifted, not clipped, at the matrix edges; the diagonal block is always present), values
    N(0,1) with the diagonal raised above the row's absolute sum; x ~ U[-1,1]."""
    rng = np.random.default_rng(seed)
    nb = block_rows
    w = min(2 * half_band + 1, nb)
    k = min(blocks_per_row, w)
    i = np.arange(nb, dtype=np.int64)
    start = np.clip(i - half_band, 0, nb - w)
    diag_off = i - start  # position of the diagonal inside the window
    # k-1 distinct offsets != diag_off: draw, then redraw rows that collide until clean
    off = rng.integers(0, w - 1, size=(nb, k - 1), dtype=np.int64)
    while True:
        off.sort(axis=1)
        dup = (off[:, 1:] == off[:, :-1]).any(axis=1) if k > 2 else np.zeros(nb, bool)
        bad = np.nonzero(dup)[0]
        if bad.size == 0:
            break
        off[bad] = rng.integers(0, w - 1, size=(bad.size, k - 1), dtype=np.int64)
    off = off + (off >= diag_off[:, None])  # skip the diagonal slot
    bcols = np.concatenate([off, diag_off[:, None]], axis=1)
    bcols.sort(axis=1)
    bcols += start[:, None]
    # expand to scalar rows: row 3*i+a has columns 3*bc+b for every block, b = 0..2
    cols_row = (bcols[:, :, None] * 3 + np.arange(3, dtype=np.int64)[None, None, :]).reshape(nb, 3 * k)
    cols = np.repeat(cols_row, 3, axis=0).astype(np.uint32).reshape(-1)
    n = 3 * nb
    per_row = 3 * k
    vals = rng.standard_normal(size=(n, per_row)).astype(dtype)
    rows = np.arange(n, dtype=np.int64)
    is_diag = cols.reshape(n, per_row) == rows[:, None].astype(np.uint32)
    rowsum = np.abs(vals).sum(axis=1)
    vals[is_diag] = (rowsum + 1.0).astype(dtype)
    indptr = np.arange(n + 1, dtype=np.int64) * per_row
    x = rng.uniform(-1.0, 1.0, size=n).astype(dtype)
    return CsrMatrix(n, n, indptr, cols, vals.reshape(-1)), x


def rmat_edges(scale: int, n_edges: int, seed: int, a=0.57, b=0.19, c=0.19, chunk_id: int = 0):
    """One chunk of R-MAT edges as (row, col) int64 arrays: every level draws the quadrant
    with probabilities a, b, c, d = 1-a-b-c (row bit = quadrant in {c, d}, col bit = quadrant
    in {b, d})."""
    rng = np.random.default_rng([seed, chunk_id])
    rows = np.zeros(n_edges, dtype=np.int64)
    cols = np.zeros(n_edges, dtype=np.int64)
    for _ in range(scale):
        u = rng.random(n_edges)
        rbit = u >= (a + b)
        cbit = ((u >= a) & (u < a + b)) | (u >= a + b + c)
        rows = (rows << 1) | rbit
        cols = (cols << 1) | cbit
    return rows, cols


def rmat(scale: int = 26, edge_factor: int = 16, seed: int = 4, dtype=np.float32, chunk: int = 1 << 24):
    """Config 5 on the host (for scaled-down instances): R-MAT adjacency, duplicate edges
    merged, values and x ~ U(0,1]. Rows without edges stay empty."""
    n = 1 << scale
    total = n * edge_factor
    keys = []
    done = 0
    cid = 0
    while done < total:
        m = min(chunk, total - done)
        r, c = rmat_edges(scale, m, seed, chunk_id=cid)
        keys.append(r * n + c)
        done += m
        cid += 1
    key = np.unique(np.concatenate(keys))
    rows = key // n
    cols = (key - rows * n).astype(np.uint32)
    indptr = _from_lengths(np.bincount(rows, minlength=n).astype(np.int64))
    rng = np.random.default_rng([seed, 1 << 20])
    vals = (1.0 - rng.random(cols.shape[0])).astype(dtype)
    x = (1.0 - rng.random(n)).astype(dtype)
    return CsrMatrix(n, n, indptr, cols, vals), x


def write_mtx_coo(path: str, m: CsrMatrix) -> None:
    """Write the reference's `.mtx.coo` text format (1-based, row-major, sorted)."""
    rows = np.repeat(np.arange(m.n_rows, dtype=np.int64), m.row_lengths()) + 1
    cols = m.indices.astype(np.int64) + 1
    fmt = "%.9g" if m.values.dtype == np.float32 else "%.17g"
    with open(path, "w") as f:
        f.write(f"{m.n_rows} {m.n_cols} {m.nnz}\n")
        block = 1 << 20
        for s in range(0, m.nnz, block):
            e = min(m.nnz, s + block)
            lines = [f"{r} {c} {fmt % v}" for r, c, v in zip(rows[s:e].tolist(), cols[s:e].tolist(), m.values[s:e].tolist())]
            f.write("\n".join(lines))
            f.write("\n")


def read_mtx_coo(path: str, dtype=np.float32) -> CsrMatrix:
    """Parse `.mtx.coo` (same grammar as the writer)."""
    with open(path) as f:
        head = f.readline().split()
        n_rows, n_cols = int(head[0]), int(head[1])
        data = np.loadtxt(f, dtype=np.float64, ndmin=2)
    rows = data[:, 0].astype(np.int64) - 1
    cols = (data[:, 1].astype(np.int64) - 1).astype(np.uint32)
    vals = data[:, 2].astype(dtype)
    indptr = _from_lengths(np.bincount(rows, minlength=n_rows).astype(np.int64))
    return CsrMatrix(n_rows, n_cols, indptr, cols, vals)
