"""ctypes binding of the C ABI declared in include/asp_b200.h.

The library must have been built (`python -c "import __graft_entry__ as g; g.build()"`);
a missing library is an error, never a fallback.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libasp_b200.so")

ASP_MAX_BRANCH = 5
U8, U16, U32, U64, F32, F64 = range(6)
DTYPE_OF_NP = {np.dtype(np.uint8): U8, np.dtype(np.uint16): U16, np.dtype(np.uint32): U32, np.dtype(np.uint64): U64,
               np.dtype(np.float32): F32, np.dtype(np.float64): F64}
NP_OF_NAME = {"u8": np.uint8, "u16": np.uint16, "u32": np.uint32, "u64": np.uint64, "f32": np.float32, "f64": np.float64}
COMPRESS = {"none": 0, "linear": 1, "constant": 2, "branch": 3, "cycle_linear": 4, "cycle_increase": 5}
TEMPLATE = {"K1": 0, "K2": 1, "K3": 2, "K5": 3, "K6": 4, "K7": 5, "K8": 6, "K4": 7, "K9": 8, "K10": 9, "EMPTY": 10, "B1": 11, "D1": 12}
TEMPLATE_NAME = {
    0: "DIRECT_ATOM_TEMPLATE", 1: "DIRECT_ATOM_TEMPLATE_WARP_COMPRESS", 2: "DIRECT_ATOM_TEMPLATE_WARP_BLOCK_COMPRESS",
    3: "SHARED_MEMORY_TEMPLATE", 4: "SHARED_MEMORY_TEMPLATE_WARP_COMPRESS", 5: "SHARED_MEMORY_LONG_ROW_TEMPLATE",
    6: "SHARED_MEMORY_TOTAL_WARP_REDUCE_TEMPLATE", 7: "DIRECT_ATOM_TOTAL_WARP_REDUCE_TEMPLATE",
    8: "UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE", 9: "UNALIGNED_WARP_REDUCE_SAME_TLB_SIZE_TEMPLATE_WITH_WARP_REDUCE",
    10: "EMPTY_TEMPLATE", 11: "BLOCK_ELL_TEMPLATE", 12: "DIAG_TEMPLATE",
}
ROLE = {
    "val_arr": 0, "col_index_arr": 1, "row_index_before_sort": 2, "global_row_index_of_thread_level_block": 3,
    "block_begin_warp_index_offset": 4, "warp_begin_thread_index_offset": 5, "thread_block_size_in_warp": 6,
    "block_nz_begin_offset": 7, "warp_nz_begin_offset": 8, "block_begin_thread_index_offset": 9,
    "thread_block_size_in_block": 10, "global_row_index_of_warp_level_block": 11, "global_warp_nz_begin_offset": 12,
    "row_offset_in_thread_tmp_result": 13, "block_first_row_index": 14, "row_index_of_block_level_block": 15,
    "row_offset_in_warp_tmp_result": 16, "global_warp_block_first_nz": 17,
    "global_first_row_index_of_warp_level_block": 18, "combine_meta_of_thread_level_block": 19,
}
SORT_NONE, SORT_GLOBAL, SORT_LOCAL = 0, 1, 2


class ArrayDesc(C.Structure):
    _fields_ = [("role", C.c_int32), ("dtype", C.c_int32), ("host_ptr", C.c_void_p), ("len", C.c_uint64),
                ("compress", C.c_int32), ("n_branch", C.c_int32), ("coef", C.c_uint64), ("icpt", C.c_uint64),
                ("cycle", C.c_uint64), ("branch_lo", C.c_uint64 * ASP_MAX_BRANCH), ("branch_hi", C.c_uint64 * ASP_MAX_BRANCH),
                ("branch_val", C.c_uint64 * ASP_MAX_BRANCH)]


class PlanDesc(C.Structure):
    _fields_ = [("template_type", C.c_int32), ("val_dtype", C.c_int32), ("n_rows", C.c_uint64), ("n_cols", C.c_uint64),
                ("first_row", C.c_uint64), ("first_col", C.c_uint64), ("true_nnz", C.c_uint64), ("n_arrays", C.c_int32),
                ("arrays", C.POINTER(ArrayDesc)), ("effective_num", C.c_uint64), ("tlb_size", C.c_uint64),
                ("bits_word", C.c_int32), ("bits_flag", C.c_int32), ("bits_row", C.c_int32), ("bits_off", C.c_int32),
                ("is_atom_add", C.c_int32), ("sort_kind", C.c_int32), ("tblock_num", C.c_int64),
                ("thread_num_in_block", C.c_int64), ("thread_num_of_row_reduce", C.c_int64)]


EXPORTS = [
    "asp_ctx_create", "asp_multicast_store", "asp_spmv_publish", "asp_plan_end_rows", "asp_rank_barrier", "asp_ctx_destroy", "asp_ctx_stream", "asp_plan_group_create", "asp_plan_descs_validate", "asp_plan_destroy",
    "asp_plan_set_launch", "asp_plan_get_launch", "asp_plan_set_tuning", "asp_plan_format_bytes", "asp_plan_launches", "asp_spmv", "asp_spmv_host", "asp_time",
    "asp_synchronize", "asp_status_str", "asp_last_error", "asp_built_for_sm100a", "asp_spmv_host_static",
    "asp_static_stage_bytes", "asp_search_gpu", "asp_spmv_host_pipelined", "asp_dist_create", "asp_dist_destroy", "asp_dist_spmv", "asp_dist_spmv_iter", "asp_dist_status",
]

_lib = None


class DistChunk(C.Structure):
    """asp_dist_chunk"""
    _fields_ = [("plans", C.POINTER(C.c_void_p)), ("n_plans", C.c_int), ("row_lo", C.c_uint64), ("row_hi", C.c_uint64)]


class HostChunk(C.Structure):
    """asp_host_chunk"""
    _fields_ = [("plans", C.POINTER(C.c_void_p)), ("n_plans", C.c_int), ("row_lo", C.c_uint64), ("row_hi", C.c_uint64), ("col_hi", C.c_uint64)]


class DistDesc(C.Structure):
    """asp_dist_desc"""
    _fields_ = [("rank", C.c_int), ("world", C.c_int), ("value_is_f64", C.c_int), ("n", C.c_uint64), ("chunks", C.POINTER(DistChunk)),
                ("n_chunks", C.c_int), ("flags_local", C.c_void_p), ("flags_multicast", C.c_void_p), ("max_polls", C.c_uint)]


class AspError(RuntimeError):
    def __init__(self, status: int, msg: str):
        super().__init__(f"asp status {status}: {msg}")
        self.status = status


def lib() -> C.CDLL:
    """Load libasp_b200.so (once). Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FileNotFoundError(f"{LIB_PATH} is missing: build the CUDA library first (__graft_entry__.build()); there is no CPU fallback")
    L = C.CDLL(LIB_PATH)
    L.asp_ctx_create.argtypes = [C.c_int, C.POINTER(C.c_void_p)]
    L.asp_ctx_create.restype = C.c_int
    L.asp_multicast_store.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_int]
    L.asp_multicast_store.restype = C.c_int
    L.asp_spmv_publish.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
    L.asp_spmv_publish.restype = C.c_int
    L.asp_plan_end_rows.argtypes = [C.c_void_p]
    L.asp_plan_end_rows.restype = C.c_uint64
    L.asp_rank_barrier.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_uint, C.c_void_p, C.c_uint, C.c_void_p]
    L.asp_rank_barrier.restype = C.c_int
    L.asp_ctx_destroy.argtypes = [C.c_void_p]
    L.asp_ctx_destroy.restype = None
    L.asp_ctx_stream.argtypes = [C.c_void_p]
    L.asp_ctx_stream.restype = C.c_void_p
    L.asp_plan_group_create.argtypes = [C.c_void_p, C.POINTER(PlanDesc), C.c_int, C.POINTER(C.c_void_p)]
    L.asp_plan_group_create.restype = C.c_int
    L.asp_plan_descs_validate.argtypes = [C.POINTER(PlanDesc), C.c_int]
    L.asp_plan_descs_validate.restype = C.c_int
    L.asp_plan_destroy.argtypes = [C.c_void_p]
    L.asp_plan_destroy.restype = None
    L.asp_plan_set_launch.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_int64]
    L.asp_plan_set_launch.restype = C.c_int
    L.asp_plan_get_launch.argtypes = [C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
    L.asp_plan_get_launch.restype = C.c_int
    L.asp_plan_set_tuning.argtypes = [C.c_void_p, C.c_int, C.c_int]
    L.asp_plan_set_tuning.restype = C.c_int
    L.asp_plan_format_bytes.argtypes = [C.c_void_p]
    L.asp_plan_format_bytes.restype = C.c_uint64
    L.asp_plan_launches.argtypes = [C.c_void_p]
    L.asp_plan_launches.restype = C.c_int
    L.asp_spmv.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_void_p, C.c_void_p, C.c_int]
    L.asp_spmv.restype = C.c_int
    L.asp_spmv_host.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_void_p, C.c_void_p]
    L.asp_spmv_host.restype = C.c_int
    L.asp_spmv_host_static.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_void_p, C.c_void_p]
    L.asp_spmv_host_static.restype = C.c_int
    L.asp_static_stage_bytes.argtypes = []
    L.asp_static_stage_bytes.restype = C.c_uint64
    L.asp_time.argtypes = [C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_int, C.c_int, C.c_double,
                           C.POINTER(C.c_float), C.POINTER(C.c_float)]
    L.asp_time.restype = C.c_int
    L.asp_synchronize.argtypes = [C.c_void_p]
    L.asp_synchronize.restype = C.c_int
    L.asp_status_str.argtypes = [C.c_int]
    L.asp_status_str.restype = C.c_char_p
    L.asp_last_error.argtypes = []
    L.asp_last_error.restype = C.c_char_p
    L.asp_built_for_sm100a.argtypes = []
    L.asp_built_for_sm100a.restype = C.c_int
    L.asp_spmv_host_pipelined.argtypes = [C.c_void_p, C.POINTER(HostChunk), C.c_int, C.c_void_p, C.c_void_p]
    L.asp_spmv_host_pipelined.restype = C.c_int
    L.asp_dist_create.argtypes = [C.c_void_p, C.POINTER(DistDesc), C.POINTER(C.c_void_p)]
    L.asp_dist_create.restype = C.c_int
    L.asp_dist_destroy.argtypes = [C.c_void_p]
    L.asp_dist_destroy.restype = None
    L.asp_dist_spmv.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    L.asp_dist_spmv.restype = C.c_int
    L.asp_dist_spmv_iter.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int, C.POINTER(C.c_int)]
    L.asp_dist_spmv_iter.restype = C.c_int
    L.asp_dist_status.argtypes = [C.c_void_p, C.POINTER(C.c_int)]
    L.asp_dist_status.restype = C.c_int
    _lib = L
    return L


def check(status: int) -> None:
    if status != 0:
        L = lib()
        raise AspError(status, f"{L.asp_status_str(status).decode()}: {L.asp_last_error().decode()}")


def multicast_store(src_ptr: int, multicast_ptr: int, nbytes: int, stream: int, ctas: int = 0) -> None:
    """asp_multicast_store: one-to-all store of a slice through an NVLink multicast address."""
    check(lib().asp_multicast_store(src_ptr, multicast_ptr, nbytes, stream, ctas))


def rank_barrier(flags_local: int, flags_multicast: int, rank: int, world: int, epoch: int, status_ptr: int, stream: int, max_polls: int = 0) -> None:
    """asp_rank_barrier: bounded-wait barrier of the ranks of a multicast group, enqueued on `stream`."""
    check(lib().asp_rank_barrier(flags_local, flags_multicast, rank, world, epoch & 0xFFFFFFFF, status_ptr, max_polls, stream))


class Context:
    """One per GPU: stream, events, scratch x / y (asp_ctx)."""

    def __init__(self, device: int = 0):
        self._h = C.c_void_p()
        check(lib().asp_ctx_create(device, C.byref(self._h)))
        self.device = device

    @property
    def handle(self):
        return self._h

    @property
    def stream(self) -> int:
        return lib().asp_ctx_stream(self._h) or 0

    def synchronize(self):
        check(lib().asp_synchronize(self._h))

    def close(self):
        if self._h:
            lib().asp_ctx_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def make_array_desc(name: str, arr, compress: dict | None, length: int | None = None, dtype: int | None = None) -> ArrayDesc:
    """Describe one template array. `arr` may be None for a closed form."""
    d = ArrayDesc()
    d.role = ROLE[name]
    if arr is not None:
        assert arr.flags["C_CONTIGUOUS"]
        d.dtype = DTYPE_OF_NP[arr.dtype]
        d.host_ptr = arr.ctypes.data
        d.len = arr.shape[0] if length is None else length
    else:
        d.dtype = U32 if dtype is None else dtype
        d.host_ptr = None
        d.len = length or 0
    c = compress or {"kind": "none"}
    d.compress = COMPRESS[c["kind"]]
    d.coef = int(c.get("coef", 0))
    d.icpt = int(c.get("icpt", 0))
    d.cycle = int(c.get("cycle", 0))
    if c["kind"] == "branch":
        d.n_branch = len(c["val"])
        for i in range(d.n_branch):
            d.branch_lo[i] = int(c["lo"][i])
            d.branch_hi[i] = int(c["hi"][i])
            d.branch_val[i] = int(c["val"][i])
    return d


def validate_descs(descs: list[PlanDesc]) -> None:
    """asp_plan_descs_validate: the checks of PlanGroup() without a GPU; raises AspError."""
    n = len(descs)
    arr = (PlanDesc * n)(*descs)
    check(lib().asp_plan_descs_validate(arr, n))


class PlanGroup:
    """All sub-matrix plans of one matrix (asp_plan_group_create). Keeps the host arrays alive
    until upload has finished."""

    def __init__(self, ctx: Context, descs: list[PlanDesc], keepalive=None):
        self.ctx = ctx
        n = len(descs)
        self._descs = (PlanDesc * n)(*descs)
        self._plans = (C.c_void_p * n)()
        self._keep = keepalive
        check(lib().asp_plan_group_create(ctx.handle, self._descs, n, self._plans))
        self.n = n
        self.val_dtype = np.float64 if descs[0].val_dtype == F64 else np.float32
        self.n_rows = int(descs[0].n_rows)
        self.n_cols = int(descs[0].n_cols)
        self._keep = None

    def set_launch(self, i: int, tblock: int, threads: int, reduce: int = 1):
        check(lib().asp_plan_set_launch(self._plans[i], tblock, threads, reduce))

    def get_launch(self, i: int):
        """(tblock_num, thread_num_in_block, thread_num_of_row_reduce) the kernel of plan i is launched with."""
        a, b, c = C.c_int64(), C.c_int64(), C.c_int64()
        check(lib().asp_plan_get_launch(self._plans[i], C.byref(a), C.byref(b), C.byref(c)))
        return a.value, b.value, c.value

    def set_tuning(self, i: int, vec: int = 0, path: int = -1):
        check(lib().asp_plan_set_tuning(self._plans[i], vec, path))

    def format_bytes(self) -> int:
        return sum(lib().asp_plan_format_bytes(self._plans[i]) for i in range(self.n))

    def launches(self) -> int:
        return sum(lib().asp_plan_launches(self._plans[i]) for i in range(self.n))

    def spmv(self, d_x: int, d_y: int, zero_y=True):
        """Asynchronous y (+)= A x on device pointers (ints). zero_y: False / True / "auto"
        (clear y only when a plan accumulates with atomics)."""
        z = 2 if zero_y == "auto" else (1 if zero_y else 0)
        check(lib().asp_spmv(self.ctx.handle, self._plans, self.n, C.c_void_p(d_x), C.c_void_p(d_y), z))

    def spmv_publish(self, d_x: int, d_y: int, d_y_multicast: int):
        """asp_spmv_publish: y = A x computed and sent to every rank of the multicast group from one kernel."""
        check(lib().asp_spmv_publish(self.ctx.handle, self._plans, self.n, C.c_void_p(d_x), C.c_void_p(d_y), C.c_void_p(d_y_multicast)))

    def end_rows(self) -> int:
        return sum(lib().asp_plan_end_rows(self._plans[i]) for i in range(self.n))

    def spmv_host(self, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=self.val_dtype)
        assert x.shape[0] == self.n_cols
        y = np.empty(self.n_rows, dtype=self.val_dtype)
        check(lib().asp_spmv_host(self.ctx.handle, self._plans, self.n, C.c_void_p(x.ctypes.data), C.c_void_p(y.ctypes.data)))
        return y

    def spmv_host_static(self, x: np.ndarray) -> np.ndarray:
        """spmv_host without any device allocation: x and y are staged in the library's fixed
        device array (see asp_spmv_host_static in include/asp_b200.h for who needs this and for
        the size limit)."""
        x = np.ascontiguousarray(x, dtype=self.val_dtype)
        assert x.shape[0] == self.n_cols
        y = np.empty(self.n_rows, dtype=self.val_dtype)
        check(lib().asp_spmv_host_static(self.ctx.handle, self._plans, self.n, C.c_void_p(x.ctypes.data), C.c_void_p(y.ctypes.data)))
        return y

    def time(self, warmup: int = 3, reps: int = 20, zero_y="auto", gflops_up_bound: float = 0.0):
        ms = C.c_float()
        gf = C.c_float()
        z = 2 if zero_y == "auto" else (1 if zero_y else 0)
        check(lib().asp_time(self.ctx.handle, self._plans, self.n, warmup, reps, z, gflops_up_bound, C.byref(ms), C.byref(gf)))
        return ms.value, gf.value

    def close(self):
        for i in range(self.n):
            if self._plans[i]:
                lib().asp_plan_destroy(self._plans[i])
                self._plans[i] = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class DistLoop:
    """The sharded repeated SpMV of one rank as a native loop (asp_dist_*). `chunks`: [(PlanGroup or None,
    first global row, end global row)] in the order they are computed; vectors and flags are device
    pointers (ints) of symmetric memory the caller owns."""

    def __init__(self, ctx: Context, chunks, n: int, rank: int = 0, world: int = 1, f64: bool = False, flags_local: int = 0, flags_multicast: int = 0,
                 max_polls: int = 0):
        self.ctx = ctx
        self._groups = [g for g, _, _ in chunks]  # keep the plan groups alive
        arr = (DistChunk * len(chunks))()
        for i, (g, lo, hi) in enumerate(chunks):
            arr[i].plans = C.cast(g._plans, C.POINTER(C.c_void_p)) if g is not None else None
            arr[i].n_plans = g.n if g is not None else 0
            arr[i].row_lo, arr[i].row_hi = int(lo), int(hi)
        d = DistDesc(rank, world, 1 if f64 else 0, int(n), arr, len(chunks), flags_local or None, flags_multicast or None, max_polls)
        self._h = C.c_void_p()
        check(lib().asp_dist_create(ctx.handle, C.byref(d), C.byref(self._h)))

    def spmv(self, d_x: int, d_y: int, d_y_multicast: int = 0) -> None:
        check(lib().asp_dist_spmv(self._h, C.c_void_p(d_x), C.c_void_p(d_y), C.c_void_p(d_y_multicast or None)))

    def iterate(self, d_x0: int, bufs, bufs_multicast, iters: int) -> int:
        """x <- A x `iters` times from d_x0; returns the index (0 / 1) of the buffer that holds the result."""
        b = (C.c_void_p * 2)(bufs[0], bufs[1])
        m = (C.c_void_p * 2)(bufs_multicast[0] or None, bufs_multicast[1] or None) if bufs_multicast else None
        last = C.c_int(-1)
        check(lib().asp_dist_spmv_iter(self._h, C.c_void_p(d_x0), b, m, iters, C.byref(last)))
        return last.value

    def status(self) -> None:
        """Waits for the stream; raises AspError (status 7) when a barrier gave up waiting for a rank."""
        w = C.c_int(-1)
        check(lib().asp_dist_status(self._h, C.byref(w)))

    def close(self):
        if self._h:
            lib().asp_dist_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def spmv_host_pipelined(ctx: Context, chunks, h_x_ptr: int, h_y_ptr: int) -> None:
    """asp_spmv_host_pipelined: `chunks` = [(PlanGroup, first row, end row, col_hi)] in ascending row order; h_x / h_y are host
    pointers (pinned memory for real overlap)."""
    arr = (HostChunk * len(chunks))()
    for i, (g, lo, hi, col_hi) in enumerate(chunks):
        arr[i].plans = C.cast(g._plans, C.POINTER(C.c_void_p))
        arr[i].n_plans = g.n
        arr[i].row_lo, arr[i].row_hi, arr[i].col_hi = int(lo), int(hi), int(col_hi)
    check(lib().asp_spmv_host_pipelined(ctx.handle, arr, len(chunks), C.c_void_p(h_x_ptr), C.c_void_p(h_y_ptr)))
