"""Test-side helpers around the oracles.

* format oracle: runs `oracle/_ref/ref_dump` (the reference's own host code) on a matrix and a
  graph spec, and loads the resulting manifest + arrays;
* y oracle: `oracle/_build/libasp_oracle.so`, CSR SpMV with double accumulation;
* conversion of a manifest into the C ABI's plan descriptors.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import subprocess
import sys
import tempfile

import numpy as np

from alphasparse_b200 import capi
from alphasparse_b200.matrices import CsrMatrix, write_mtx_coo

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_DIR = os.path.join(ROOT, "oracle", "_ref")
REF_DUMP = os.path.join(REF_DIR, "ref_dump")
ORACLE_LIB = os.path.join(ROOT, "oracle", "_build", "libasp_oracle.so")
GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")

TOL = {np.dtype(np.float32): 1e-5, np.dtype(np.float64): 1e-12}


def have_ref_dump() -> bool:
    return os.path.exists(REF_DUMP)


def build_oracles() -> None:
    """Compile the C y-oracle, and the reference format oracle when the reference tree exists."""
    subprocess.run(["make", "-s", "-C", os.path.join(ROOT, "oracle"), "cpu"], check=True)
    sys.path.insert(0, ROOT)
    from __graft_entry__ import reference_dir

    ref = reference_dir()
    if ref:
        subprocess.run(["make", "-s", "-j8", "-C", os.path.join(ROOT, "oracle"), "ref", "REF=" + ref], check=True)


_olib = None


def oracle_lib():
    global _olib
    if _olib is None:
        if not os.path.exists(ORACLE_LIB):
            build_oracles()
        _olib = C.CDLL(ORACLE_LIB)
        _olib.asp_oracle_max_threads.restype = C.c_int
    return _olib


def csr_ref(m: CsrMatrix, x: np.ndarray):
    """(y_ref, scale): y in double accumulation and sum |a||x| per row."""
    L = oracle_lib()
    fn = L.asp_oracle_spmv_f64_ref if m.values.dtype == np.float64 else L.asp_oracle_spmv_f32_ref
    y = np.zeros(m.n_rows, dtype=np.float64)
    sc = np.zeros(m.n_rows, dtype=np.float64)
    indptr = np.ascontiguousarray(m.indptr, dtype=np.int64)
    idx = np.ascontiguousarray(m.indices, dtype=np.uint32)
    vals = np.ascontiguousarray(m.values)
    xx = np.ascontiguousarray(x, dtype=m.values.dtype)
    fn(C.c_int64(m.n_rows), C.c_void_p(indptr.ctypes.data), C.c_void_p(idx.ctypes.data), C.c_void_p(vals.ctypes.data),
       C.c_void_p(xx.ctypes.data), C.c_void_p(y.ctypes.data), C.c_void_p(sc.ctypes.data))
    return y, sc


def csr_native(m: CsrMatrix, x: np.ndarray) -> np.ndarray:
    """The timed CPU baseline loop (accumulation in the value dtype, OpenMP)."""
    L = oracle_lib()
    fn = L.asp_oracle_spmv_f64_native if m.values.dtype == np.float64 else L.asp_oracle_spmv_f32_native
    y = np.zeros(m.n_rows, dtype=m.values.dtype)
    indptr = np.ascontiguousarray(m.indptr, dtype=np.int64)
    idx = np.ascontiguousarray(m.indices, dtype=np.uint32)
    vals = np.ascontiguousarray(m.values)
    xx = np.ascontiguousarray(x, dtype=m.values.dtype)
    fn(C.c_int64(m.n_rows), C.c_void_p(indptr.ctypes.data), C.c_void_p(idx.ctypes.data), C.c_void_p(vals.ctypes.data),
       C.c_void_p(xx.ctypes.data), C.c_void_p(y.ctypes.data))
    return y


def rel_err(y: np.ndarray, y_ref: np.ndarray, scale: np.ndarray) -> float:
    """max_i |y_i - y_ref_i| / sum_j |a_ij||x_j| (rows with zero scale must match exactly)."""
    d = np.abs(y.astype(np.float64) - y_ref)
    nz = scale > 0
    worst = float((d[nz] / scale[nz]).max()) if nz.any() else 0.0
    if (~nz).any() and d[~nz].max() > 0:
        return float("inf")
    return worst


def assert_y(y, y_ref, scale, dtype, what=""):
    e = rel_err(y, y_ref, scale)
    tol = TOL[np.dtype(dtype)]
    assert e <= tol, f"{what}: max |y-y_ref|/(|A||x|) = {e:.3e} > {tol:g}"


class Manifest:
    """manifest.json + arrays.bin of one ref_dump run (or of a golden fixture)."""

    def __init__(self, meta: dict, blob: np.ndarray):
        self.meta = meta
        self.blob = blob

    def array(self, desc: dict) -> np.ndarray:
        dt = np.dtype(capi.NP_OF_NAME[desc["dtype"]])
        n = int(desc["len"])
        return self.blob[desc["offset"] : desc["offset"] + n * dt.itemsize].view(dt)

    @property
    def subs(self):
        return self.meta["subs"]

    def global_perm(self):
        for g in self.meta["global"]:
            if g["name"] == "sorted_row_index":
                return self.array(g)
        return None

    def sub_arrays(self, i: int) -> dict:
        return {a["name"]: (self.array(a), a["compress"], a) for a in self.subs[i]["arrays"]}

    @staticmethod
    def load(dirname: str) -> "Manifest":
        with open(os.path.join(dirname, "manifest.json")) as f:
            meta = json.load(f)
        blob = np.fromfile(os.path.join(dirname, "arrays.bin"), dtype=np.uint8)
        return Manifest(meta, blob)


def run_ref_dump(m: CsrMatrix, spec: str, keep_dir: str | None = None) -> Manifest:
    """Run the reference host pipeline on `m` with graph `spec` (see oracle/ref_dump.cc)."""
    assert have_ref_dump(), "oracle/_ref/ref_dump not built"
    tmp = keep_dir or tempfile.mkdtemp(prefix="asp_ref_")
    os.makedirs(tmp, exist_ok=True)
    mtx = os.path.join(tmp, "m.mtx.coo")
    write_mtx_coo(mtx, m)
    dt = "double" if m.values.dtype == np.float64 else "float"
    with open(os.path.join(tmp, "spec"), "w") as f:
        f.write(f"dtype {dt}\n{spec}\n")
    r = subprocess.run([REF_DUMP, mtx, os.path.join(tmp, "spec"), tmp], cwd=REF_DIR, stdout=subprocess.DEVNULL, stderr=subprocess.PIPE)
    if r.returncode != 0:
        raise RuntimeError(f"ref_dump failed ({r.returncode}): {r.stderr.decode()[-500:]}")
    man = Manifest.load(tmp)
    if keep_dir is None:
        for fn in os.listdir(tmp):
            os.remove(os.path.join(tmp, fn))
        os.rmdir(tmp)
    return man


def plan_descs(man: Manifest, launch: dict | None = None):
    """C-ABI descriptors for every sub-matrix of a manifest. Returns (descs, keepalive)."""
    keep = []
    descs = []
    meta = man.meta
    val_dtype = capi.F64 if meta["val_dtype"] == "f64" else capi.F32
    for i, s in enumerate(man.subs):
        arrs = []
        for a in s["arrays"]:
            if a["name"] in ("first_relative_reduce_row_of_thread_level_block", "tmp_result_reduce_offset_of_thread_level_block"):
                continue  # host-side intermediates of the CSR5-like templates, never uploaded by the reference either
            arr = np.ascontiguousarray(man.array(a))
            keep.append(arr)
            arrs.append(capi.make_array_desc(a["name"], arr, a["compress"]))
        arr_t = (capi.ArrayDesc * len(arrs))(*arrs)
        keep.append(arr_t)
        d = capi.PlanDesc()
        d.template_type = capi.TEMPLATE[s["template"]]
        d.val_dtype = val_dtype
        d.n_rows = meta["rows"]
        d.n_cols = meta["cols"]
        d.first_row = s["first_row"]
        d.first_col = s["first_col"]
        d.true_nnz = s["end_coo"] - s["begin_coo"] + 1
        d.n_arrays = len(arrs)
        d.arrays = arr_t
        d.effective_num = s.get("effective_TLB_num", s.get("effective_WLB_num", s.get("effective_row_num", 0)))
        d.tlb_size = s.get("thread_block_size_in_block", s.get("tlb_size", 0))
        d.bits_word = s.get("bits_word", 0)
        d.bits_flag = s.get("bits_flag", 0)
        d.bits_row = s.get("bits_row", 0)
        d.bits_off = s.get("bits_off", 0)
        d.is_atom_add = s.get("is_atom_add", s.get("is_all_force_atom_add", 0))
        d.sort_kind = capi.SORT_GLOBAL if s["global_sort"] else (capi.SORT_LOCAL if s["local_sort"] else capi.SORT_NONE)
        lp = (launch or {}).get(i, {})
        threads = lp.get("threads", s.get("threads", 256))
        tblock = lp.get("tblock", s.get("tblock", 0))
        if not tblock:  # the second CSR5-like template derives its grid from the block size
            n_tlb = [a["len"] for a in s["arrays"] if a["name"] == "combine_meta_of_thread_level_block"][0]
            tblock = (n_tlb + threads - 1) // threads
        d.tblock_num = tblock
        d.thread_num_in_block = threads
        d.thread_num_of_row_reduce = lp.get("reduce", s.get("row_reduce", 1))
        descs.append(d)
    return descs, keep
