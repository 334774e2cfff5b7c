"""R-MAT generator on the GPU (torch), for the graph configuration that is too large for numpy.

Edges are generated in fixed-size chunks whose random streams depend only on (seed, chunk id), a
rank keeps the edges whose row falls in its row range, duplicates are merged, and the value of an
edge is a hash of (row, col): the matrix does not depend on how many ranks generate it.
"""
from __future__ import annotations

import numpy as np
import torch

from .matrices import CsrMatrix

CHUNK = 1 << 25


def _chunk_edges(scale: int, n_edges: int, seed: int, chunk_id: int, device, a=0.57, b=0.19, c=0.19):
    g = torch.Generator(device=device)
    g.manual_seed((seed << 20) + chunk_id)
    rows = torch.zeros(n_edges, dtype=torch.int64, device=device)
    cols = torch.zeros(n_edges, dtype=torch.int64, device=device)
    for _ in range(scale):
        u = torch.rand(n_edges, generator=g, device=device)
        rbit = (u >= a + b).to(torch.int64)
        cbit = (((u >= a) & (u < a + b)) | (u >= a + b + c)).to(torch.int64)
        rows = (rows << 1) | rbit
        cols = (cols << 1) | cbit
    return rows, cols


def _hash01(key: torch.Tensor, salt: int) -> torch.Tensor:
    """(0, 1] from a 64-bit mix of the key (splitmix64 finaliser on int64 with wrap-around)."""
    z = key + salt
    z = (z ^ (z >> 30)) * -4658895280553007687  # 0xBF58476D1CE4E5B9
    z = (z ^ (z >> 27)) * -7723592293110705685  # 0x94D049BB133111EB
    z = z ^ (z >> 31)
    m = (z & ((1 << 24) - 1)).to(torch.float32)
    return (m + 1.0) / float(1 << 24)


def rmat_degrees(scale: int, edge_factor: int, seed: int, device, chunk_ids=None, columns: bool = True):
    """(edges per row, edges per column) before duplicate removal over the given chunks (all chunks when None)."""
    n = 1 << scale
    total = n * edge_factor
    n_chunks = (total + CHUNK - 1) // CHUNK
    deg = torch.zeros(n, dtype=torch.int64, device=device)
    cdeg = torch.zeros(n, dtype=torch.int64, device=device) if columns else None
    for cid in (range(n_chunks) if chunk_ids is None else chunk_ids):
        m = min(CHUNK, total - cid * CHUNK)
        r, c = _chunk_edges(scale, m, seed, cid, device)
        deg += torch.bincount(r, minlength=n)
        if columns:
            cdeg += torch.bincount(c, minlength=n)
    return deg, cdeg


def rmat_row_degrees(scale: int, edge_factor: int, seed: int, device, chunk_ids=None) -> torch.Tensor:
    """Edges per row before duplicate removal over the given chunks (all chunks when None)."""
    return rmat_degrees(scale, edge_factor, seed, device, chunk_ids, columns=False)[0]


def hotness_labels(col_degrees: torch.Tensor, row_degrees: torch.Tensor | None = None):
    """Relabelling of the vertices of a square matrix by how often their column is read: the vertex with the
    most column entries gets label 0. Returns (labels, inverse): labels[v] = new label of vertex v,
    inverse[k] = vertex that carries label k (ties keep the original order, so the result depends on the
    counts only). In the relabelled matrix P A P^T the entries of x that most gathers read are contiguous:
    whole cache lines of x are hot, and the part of x that an L2 smaller than x keeps is the part that is read.
    With `row_degrees`, vertices whose row has no entries come last (in the same order among themselves): their
    rows of A x are zero for every x, so a loop x <- A x neither computes nor exchanges that suffix."""
    inverse = torch.argsort(col_degrees, descending=True, stable=True)
    if row_degrees is not None:
        has_row = row_degrees[inverse] > 0
        inverse = torch.cat([inverse[has_row], inverse[~has_row]])
    labels = torch.empty_like(inverse)
    labels[inverse] = torch.arange(inverse.shape[0], dtype=inverse.dtype, device=inverse.device)
    return labels, inverse


def rmat_block(scale: int, edge_factor: int, seed: int, r0: int, r1: int, device, labels=None, inverse=None):
    """CSR of rows [r0, r1) of the R-MAT matrix with GLOBAL column indices, as torch tensors on
    `device`: (indptr int64 [r1-r0+1], indices int32-valued int64, values float32). With `labels` /
    `inverse` (hotness_labels) rows and columns are those of the relabelled matrix P A P^T: the same
    edges and the same values (hashed from the ORIGINAL row and column), under new vertex numbers."""
    n = 1 << scale
    total = n * edge_factor
    n_chunks = (total + CHUNK - 1) // CHUNK
    keys = []
    for cid in range(n_chunks):
        m = min(CHUNK, total - cid * CHUNK)
        r, c = _chunk_edges(scale, m, seed, cid, device)
        if labels is not None:
            r, c = labels[r], labels[c]
        if r0 > 0 or r1 < n:
            keep = (r >= r0) & (r < r1)
            r, c = r[keep], c[keep]
        keys.append(torch.unique(r * n + c))
        del r, c
    key = torch.unique(torch.cat(keys))
    del keys
    rows = torch.div(key, n, rounding_mode="floor")
    cols = key - rows * n
    counts = torch.bincount(rows - r0, minlength=r1 - r0)
    indptr = torch.zeros(r1 - r0 + 1, dtype=torch.int64, device=device)
    torch.cumsum(counts, 0, out=indptr[1:])
    vals = _hash01(key if inverse is None else inverse[rows] * n + inverse[cols], seed * 7919 + 13)
    return indptr, cols, vals


def rmat_x(scale: int, seed: int, device) -> torch.Tensor:
    idx = torch.arange(1 << scale, dtype=torch.int64, device=device)
    return _hash01(idx, seed * 104729 + 71)


def to_host_csr(indptr, cols, vals, n_cols: int) -> CsrMatrix:
    return CsrMatrix(int(indptr.shape[0] - 1), n_cols, indptr.cpu().numpy(), cols.to(torch.int32).cpu().numpy().view(np.uint32), vals.cpu().numpy())
