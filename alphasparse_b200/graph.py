"""Host side of the library: matrices, Operator Graph execution, lowering to plans.

Thin ctypes layer over include/asp_b200_host.h; all format work happens in the C++ library.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import capi
from .matrices import CsrMatrix


class SubInfo(C.Structure):
    _fields_ = [("min_row", C.c_uint64), ("max_row", C.c_uint64), ("min_col", C.c_uint64), ("max_col", C.c_uint64),
                ("begin_coo", C.c_uint64), ("end_coo", C.c_uint64), ("n_blb", C.c_uint64), ("n_wlb", C.c_uint64),
                ("n_tlb", C.c_uint64), ("template_type", C.c_int32), ("n_arrays", C.c_int32)]


HOST_EXPORTS = [
    "asp_matrix_from_csr", "asp_matrix_from_coo_file", "asp_matrix_destroy", "asp_matrix_rows", "asp_matrix_cols",
    "asp_matrix_nnz", "asp_graph_execute", "asp_format_destroy", "asp_format_num_subs", "asp_format_global_perm",
    "asp_format_sub_info", "asp_format_plan_descs", "asp_format_padding_rate", "asp_host_last_error",
    "asp_dense_execute", "asp_matrix_num_subs", "asp_matrix_sub_rows", "asp_partition_rows_by_nnz", "asp_matrix_relabel_by_column_count", "asp_format_id", "asp_format_save", "asp_format_load",
    "asp_search", "asp_search_result_destroy", "asp_search_result_dense", "asp_search_result_num_subs", "asp_search_result_sub_spec",
    "asp_search_result_sub_name", "asp_search_result_sub_launch", "asp_search_result_ms", "asp_search_result_num_trials",
    "asp_search_result_trial", "asp_search_candidates", "asp_search_derive_tblock",
]

LOG_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_char_p)
# int time_fn(user, fmt, tblock[], threads[], reduce[], warmup, reps, *ms)
TIME_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.c_int, C.c_int, C.POINTER(C.c_float))


class SearchOptions(C.Structure):
    """asp_search_options"""
    _fields_ = [("quick", C.c_int32), ("warmup", C.c_int32), ("reps", C.c_int32), ("max_subs", C.c_int32), ("struggle_step_num", C.c_int32),
                ("time_limit_s", C.c_double), ("padding_rate_up_bound", C.c_double), ("prune_gbs", C.c_double), ("prune_min_bytes", C.c_uint64),
                ("log_fn", LOG_FN), ("log_user", C.c_void_p), ("strategy_mask", C.c_uint32), ("checkpoint_path", C.c_char_p)]

_bound = False


def _lib():
    global _bound
    L = capi.lib()
    if not _bound:
        L.asp_matrix_from_csr.argtypes = [C.c_uint64, C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.POINTER(C.c_void_p)]
        L.asp_matrix_from_csr.restype = C.c_int
        L.asp_matrix_from_coo_file.argtypes = [C.c_char_p, C.c_int, C.POINTER(C.c_void_p)]
        L.asp_matrix_from_coo_file.restype = C.c_int
        L.asp_matrix_destroy.argtypes = [C.c_void_p]
        L.asp_matrix_destroy.restype = None
        for fn in (L.asp_matrix_rows, L.asp_matrix_cols, L.asp_matrix_nnz):
            fn.argtypes = [C.c_void_p]
            fn.restype = C.c_uint64
        L.asp_graph_execute.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_void_p)]
        L.asp_graph_execute.restype = C.c_int
        L.asp_dense_execute.argtypes = [C.c_void_p, C.c_char_p, C.POINTER(C.c_void_p)]
        L.asp_dense_execute.restype = C.c_int
        L.asp_matrix_num_subs.argtypes = [C.c_void_p]
        L.asp_matrix_num_subs.restype = C.c_int
        L.asp_matrix_sub_rows.argtypes = [C.c_void_p, C.c_int] + [C.POINTER(C.c_uint64)] * 4
        L.asp_matrix_sub_rows.restype = C.c_int
        L.asp_partition_rows_by_nnz.argtypes = [C.c_uint64, C.c_void_p, C.c_int, C.c_void_p]
        L.asp_partition_rows_by_nnz.restype = C.c_int
        L.asp_matrix_relabel_by_column_count.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_void_p), C.c_void_p, C.POINTER(C.c_uint64)]
        L.asp_matrix_relabel_by_column_count.restype = C.c_int
        L.asp_format_destroy.argtypes = [C.c_void_p]
        L.asp_format_destroy.restype = None
        L.asp_format_num_subs.argtypes = [C.c_void_p]
        L.asp_format_num_subs.restype = C.c_int
        L.asp_format_global_perm.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_int), C.POINTER(C.c_uint64)]
        L.asp_format_global_perm.restype = C.c_int
        L.asp_format_sub_info.argtypes = [C.c_void_p, C.c_int, C.POINTER(SubInfo)]
        L.asp_format_sub_info.restype = C.c_int
        L.asp_format_plan_descs.argtypes = [C.c_void_p, C.POINTER(capi.PlanDesc)]
        L.asp_format_plan_descs.restype = C.c_int
        L.asp_format_padding_rate.argtypes = [C.c_void_p, C.c_int]
        L.asp_format_padding_rate.restype = C.c_double
        L.asp_host_last_error.argtypes = []
        L.asp_host_last_error.restype = C.c_char_p
        L.asp_format_id.argtypes = [C.c_void_p]
        L.asp_format_id.restype = C.c_uint64
        L.asp_format_save.argtypes = [C.c_void_p, C.c_char_p]
        L.asp_format_save.restype = C.c_int
        L.asp_format_load.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
        L.asp_format_load.restype = C.c_int
        L.asp_search.argtypes = [C.c_void_p, C.POINTER(SearchOptions), TIME_FN, C.c_void_p, C.POINTER(C.c_void_p)]
        L.asp_search.restype = C.c_int
        L.asp_search_gpu.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(SearchOptions), C.POINTER(C.c_void_p)]
        L.asp_search_gpu.restype = C.c_int
        L.asp_search_result_destroy.argtypes = [C.c_void_p]
        L.asp_search_result_destroy.restype = None
        L.asp_search_result_dense.argtypes = [C.c_void_p]
        L.asp_search_result_dense.restype = C.c_char_p
        L.asp_search_result_num_subs.argtypes = [C.c_void_p]
        L.asp_search_result_num_subs.restype = C.c_int
        for fn in (L.asp_search_result_sub_spec, L.asp_search_result_sub_name, L.asp_search_result_trial):
            fn.argtypes = [C.c_void_p, C.c_int]
            fn.restype = C.c_char_p
        L.asp_search_result_sub_launch.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
        L.asp_search_result_sub_launch.restype = C.c_int
        L.asp_search_result_ms.argtypes = [C.c_void_p]
        L.asp_search_result_ms.restype = C.c_float
        L.asp_search_result_num_trials.argtypes = [C.c_void_p]
        L.asp_search_result_num_trials.restype = C.c_int
        L.asp_search_candidates.argtypes = [C.c_uint64, C.c_uint64, C.c_double, C.c_int, C.c_int]
        L.asp_search_candidates.restype = C.c_char_p
        L.asp_search_derive_tblock.argtypes = [C.c_int, C.c_uint64, C.c_uint64, C.c_uint64, C.c_int64]
        L.asp_search_derive_tblock.restype = C.c_int64
        _bound = True
    return L


def _check(status: int):
    if status != 0:
        L = _lib()
        raise capi.AspError(status, f"{L.asp_status_str(status).decode()}: {L.asp_host_last_error().decode()}")


_NP_OF_DT = {capi.U8: np.uint8, capi.U16: np.uint16, capi.U32: np.uint32, capi.U64: np.uint64, capi.F32: np.float32, capi.F64: np.float64}
_ROLE_NAME = {v: k for k, v in capi.ROLE.items()}
_KIND_NAME = {v: k for k, v in capi.COMPRESS.items()}


def partition_rows_by_nnz(indptr: np.ndarray, parts: int) -> np.ndarray:
    """Row bounds (parts + 1 entries) of contiguous row blocks with about nnz / parts non-zeros each."""
    ip = np.ascontiguousarray(indptr, dtype=np.int64)
    out = np.zeros(parts + 1, dtype=np.uint64)
    _check(_lib().asp_partition_rows_by_nnz(ip.shape[0] - 1, ip.ctypes.data, parts, out.ctypes.data))
    return out.astype(np.int64)


class Matrix:
    """asp_matrix: the input of an Operator Graph (BEGIN_MEMORY_CACHE_INPUT_FILE / BEGIN_INPUT_FILE)."""

    def __init__(self, handle):
        self._h = handle

    @staticmethod
    def from_csr(m: CsrMatrix) -> "Matrix":
        indptr = np.ascontiguousarray(m.indptr, dtype=np.int64)
        idx = np.ascontiguousarray(m.indices, dtype=np.uint32)
        vals = np.ascontiguousarray(m.values)
        h = C.c_void_p()
        _check(_lib().asp_matrix_from_csr(m.n_rows, m.n_cols, indptr.ctypes.data, idx.ctypes.data, vals.ctypes.data,
                                          capi.DTYPE_OF_NP[vals.dtype], C.byref(h)))
        return Matrix(h)

    @staticmethod
    def from_coo_file(path: str, dtype=np.float32) -> "Matrix":
        h = C.c_void_p()
        _check(_lib().asp_matrix_from_coo_file(path.encode(), capi.DTYPE_OF_NP[np.dtype(dtype)], C.byref(h)))
        return Matrix(h)

    def relabel_by_column_count(self, empty_rows_last: bool = True):
        """(P A P^T as a new Matrix, labels, rows with non-zeros): vertices renumbered by column count, most frequent
        first; labels[v] = new number of vertex v (asp_matrix_relabel_by_column_count)."""
        n = self.shape[0]
        labels = np.zeros(n, dtype=np.uint32)
        h, active = C.c_void_p(), C.c_uint64()
        _check(_lib().asp_matrix_relabel_by_column_count(self._h, 1 if empty_rows_last else 0, C.byref(h), labels.ctypes.data, C.byref(active)))
        return Matrix(h), labels, int(active.value)

    @property
    def shape(self):
        L = _lib()
        return int(L.asp_matrix_rows(self._h)), int(L.asp_matrix_cols(self._h))

    @property
    def nnz(self):
        return int(_lib().asp_matrix_nnz(self._h))

    def dense(self, dense_spec: str = "dense compress") -> "Matrix":
        """Run only the dense-view nodes (sort / row division / compress); the result can be lowered
        repeatedly with execute() on `sub ...` lines."""
        h = C.c_void_p()
        _check(_lib().asp_dense_execute(self._h, dense_spec.encode(), C.byref(h)))
        return Matrix(h)

    @property
    def n_subs(self) -> int:
        return int(_lib().asp_matrix_num_subs(self._h))

    def sub_rows(self, i: int):
        """(rows, nnz, min row nnz, max row nnz) of sub-matrix i of a compressed matrix."""
        v = [C.c_uint64() for _ in range(4)]
        _check(_lib().asp_matrix_sub_rows(self._h, i, *[C.byref(x) for x in v]))
        return tuple(int(x.value) for x in v)

    def execute(self, spec: str) -> "Format":
        """Run an Operator Graph (see include/asp_b200_host.h for the spec grammar)."""
        f = C.c_void_p()
        _check(_lib().asp_graph_execute(self._h, spec.encode(), C.byref(f)))
        return Format(f)

    def close(self):
        if self._h:
            _lib().asp_matrix_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Format:
    """asp_format: one lowered template per sub-matrix."""

    def __init__(self, handle, owned: bool = True):
        self._h = handle
        self._owned = owned
        L = _lib()
        self.n_subs = L.asp_format_num_subs(handle)
        self._descs = (capi.PlanDesc * self.n_subs)()
        _check(L.asp_format_plan_descs(handle, self._descs))

    @staticmethod
    def borrowed(handle) -> "Format":
        """View of an asp_format that somebody else owns (a timing callback of asp_search)."""
        return Format(C.c_void_p(handle) if isinstance(handle, int) else handle, owned=False)

    @property
    def id(self) -> int:
        return int(_lib().asp_format_id(self._h))

    def save(self, path: str) -> None:
        """asp_format_save: everything needed to upload this format later, in one binary file."""
        _check(_lib().asp_format_save(self._h, path.encode()))

    @staticmethod
    def load(path: str) -> "Format":
        h = C.c_void_p()
        _check(_lib().asp_format_load(path.encode(), C.byref(h)))
        return Format(h)

    def plan_descs(self):
        return [self._descs[i] for i in range(self.n_subs)]

    def sub_info(self, i: int) -> SubInfo:
        s = SubInfo()
        _check(_lib().asp_format_sub_info(self._h, i, C.byref(s)))
        return s

    def padding_rate(self, i: int) -> float:
        return float(_lib().asp_format_padding_rate(self._h, i))

    def global_perm(self):
        p, dt, n = C.c_void_p(), C.c_int(), C.c_uint64()
        _check(_lib().asp_format_global_perm(self._h, C.byref(p), C.byref(dt), C.byref(n)))
        if not p.value:
            return None
        t = np.dtype(_NP_OF_DT[dt.value])
        return np.frombuffer((C.c_char * (n.value * t.itemsize)).from_address(p.value), dtype=t).copy()

    def arrays(self, i: int) -> dict:
        """name -> (numpy copy or None, closed-form dict, dtype id, length) of sub-matrix i."""
        d = self._descs[i]
        out = {}
        for k in range(d.n_arrays):
            a = d.arrays[k]
            t = np.dtype(_NP_OF_DT[a.dtype])
            arr = None
            if a.host_ptr:
                arr = np.frombuffer((C.c_char * (a.len * t.itemsize)).from_address(a.host_ptr), dtype=t).copy()
            comp = {"kind": _KIND_NAME[a.compress]}
            if comp["kind"] in ("linear", "cycle_linear"):
                comp["coef"] = int(a.coef)
            if comp["kind"] in ("linear", "constant", "cycle_linear", "cycle_increase"):
                comp["icpt"] = int(a.icpt)
            if comp["kind"] in ("cycle_linear", "cycle_increase"):
                comp["cycle"] = int(a.cycle)
            if comp["kind"] == "branch":
                comp["lo"] = [int(a.branch_lo[j]) for j in range(a.n_branch)]
                comp["hi"] = [int(a.branch_hi[j]) for j in range(a.n_branch)]
                comp["val"] = [int(a.branch_val[j]) for j in range(a.n_branch)]
            out[_ROLE_NAME[a.role]] = (arr, comp, int(a.dtype), int(a.len))
        return out

    def upload(self, ctx: capi.Context) -> capi.PlanGroup:
        """asp_plan_group_create over every sub-matrix of this format."""
        return capi.PlanGroup(ctx, self.plan_descs(), keepalive=self)

    def close(self):
        if self._h and self._owned:
            _lib().asp_format_destroy(self._h)
        self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
