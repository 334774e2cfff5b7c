"""CPU interpreter of the ten template formats (test infrastructure).

Given the arrays of one template exactly as the reference's host code produced them, compute
y = A x by walking the arrays the way the emitted kernels do (reference emitters:
direct_atom_op*.cc, shared_memory_*.cc, unaligned_warp_reduce_same_TLB_size_op*.cc,
code_of_template_kernal). It documents the array semantics the CUDA kernels rely on and lets
the CPU-only suite check "reference arrays + these semantics == CSR SpMV" without a GPU.
Accumulation is in double; only small matrices are meant to go through here.
"""
from __future__ import annotations

import numpy as np


class MetaArr:
    """A metadata array or the closed form that replaced it (arr_optimization.cc)."""

    def __init__(self, arr, comp):
        self.arr = arr
        self.c = comp or {"kind": "none"}

    def __getitem__(self, i):
        k = self.c["kind"]
        i = int(i)
        if k == "none":
            return int(self.arr[i])
        if k == "linear":
            return i * int(self.c["coef"]) + int(self.c["icpt"])
        if k == "constant":
            return int(self.c["icpt"])
        if k == "cycle_linear":
            return (i % int(self.c["cycle"])) * int(self.c["coef"]) + int(self.c["icpt"])
        if k == "cycle_increase":
            return i // int(self.c["cycle"]) + int(self.c["icpt"])
        if k == "branch":
            for lo, hi, v in zip(self.c["lo"], self.c["hi"], self.c["val"]):
                if lo <= i <= hi:
                    return int(v)
            raise IndexError(i)
        raise ValueError(k)

    def __len__(self):
        return len(self.arr)


def closed_form_matches(arr: np.ndarray, comp: dict) -> bool:
    """True when the closed form reproduces every element of the array it replaces."""
    m = MetaArr(arr, comp)
    return all(m[i] == int(arr[i]) for i in range(len(arr)))


def interpret(man, x: np.ndarray) -> np.ndarray:
    """y over all sub-matrices of a manifest."""
    y = np.zeros(man.meta["rows"], dtype=np.float64)
    xd = x.astype(np.float64)
    for i in range(len(man.subs)):
        if man.subs[i]["template"] == "EMPTY":  # a strip that is deliberately not computed
            continue
        _interp_sub(man, i, xd, y)
    return y


def _interp_sub(man, si, x, y):
    s = man.subs[si]
    A = {k: MetaArr(v[0], v[1]) for k, v in man.sub_arrays(si).items()}
    val = man.sub_arrays(si)["val_arr"][0].astype(np.float64)
    col = man.sub_arrays(si)["col_index_arr"][0].astype(np.int64) + s["first_col"]
    first_row = s["first_row"]
    gsort, lsort = s["global_sort"], s["local_sort"]
    perm = A.get("row_index_before_sort")
    t = s["template"]

    def row_host(r):  # permutation already applied by the host (K1, K2, K3, K4, K7)
        return r if gsort else r + first_row

    def row_dev(r):  # permutation applied on the device (K5, K6, K8, K9, K10)
        if gsort:
            return perm[r + first_row]
        if lsort:
            return perm[r] + first_row
        return r + first_row

    prod = val * x[col]

    if t == "K3":
        rm = A["global_row_index_of_thread_level_block"]
        P = int(man.sub_arrays(si)["global_row_index_of_thread_level_block"][2]["len"])
        S = s["thread_block_size_in_block"]
        for tid in range(min(P, s["effective_TLB_num"])):
            y[row_host(rm[tid])] += prod[tid : tid + S * P : P].sum()
    elif t == "K2":
        rm = A["global_row_index_of_thread_level_block"]
        bt, bnz, ts = A["block_begin_thread_index_offset"], A["block_nz_begin_offset"], A["thread_block_size_in_block"]
        B = int(man.sub_arrays(si)["block_nz_begin_offset"][2]["len"])
        for b in range(B):
            t0, t1, nz0, S = bt[b], bt[b + 1], bnz[b], ts[b]
            n = t1 - t0
            for i in range(n):
                if t0 + i >= s["effective_TLB_num"]:
                    break
                y[row_host(rm[t0 + i])] += prod[nz0 + i : nz0 + i + S * n : n].sum()
    elif t == "K1":
        rm = A["global_row_index_of_thread_level_block"]
        bw, wt, ts = A["block_begin_warp_index_offset"], A["warp_begin_thread_index_offset"], A["thread_block_size_in_warp"]
        bnz, wnz = A["block_nz_begin_offset"], A["warp_nz_begin_offset"]
        B = int(man.sub_arrays(si)["block_nz_begin_offset"][2]["len"])
        for b in range(B):
            for w in range(bw[b], bw[b + 1]):
                base, S, t0, t1 = bnz[b] + wnz[w], ts[w], wt[w], wt[w + 1]
                for g in range((t1 - t0) // 32):
                    for lane in range(32):
                        nz = base + g * 32 * S + lane
                        y[row_host(rm[t0 + g * 32 + lane])] += prod[nz : nz + 32 * S : 32].sum()
    elif t == "K4":
        rm, off = A["global_row_index_of_warp_level_block"], A["global_warp_nz_begin_offset"]
        for w in range(s["effective_WLB_num"]):
            y[row_host(rm[w])] += prod[off[w] : off[w + 1]].sum()
    elif t == "K7":
        rm, off = A["row_index_of_block_level_block"], A["block_nz_begin_offset"]
        B = int(man.sub_arrays(si)["row_index_of_block_level_block"][2]["len"])
        for b in range(B):
            y[row_host(rm[b])] += prod[off[b] : off[b + 1]].sum()
    elif t in ("K6", "K5", "K8"):
        roff = A["row_offset_in_thread_tmp_result"] if t != "K8" else A["row_offset_in_warp_tmp_result"]
        br = A["block_first_row_index"]
        B = int(man.sub_arrays(si)["block_first_row_index"][2]["len"]) - 1
        eff = s.get("effective_row_num", 1 << 62)
        for b in range(B):
            r0, r1 = br[b], br[b + 1]
            if t == "K6":
                bt, bnz, ts = A["block_begin_thread_index_offset"], A["block_nz_begin_offset"], A["thread_block_size_in_block"]
                t0, t1, nz0, S = bt[b], bt[b + 1], bnz[b], ts[b]
                n = t1 - t0
                part = np.array([prod[nz0 + i : nz0 + i + S * n : n].sum() for i in range(n)])
            elif t == "K5":
                bw, wt, ts = A["block_begin_warp_index_offset"], A["warp_begin_thread_index_offset"], A["thread_block_size_in_warp"]
                bnz, wnz = A["block_nz_begin_offset"], A["warp_nz_begin_offset"]
                tb0 = wt[bw[b]]
                part = np.zeros(wt[bw[b + 1]] - tb0)
                for w in range(bw[b], bw[b + 1]):
                    base, S, t0, t1 = bnz[b] + wnz[w], ts[w], wt[w], wt[w + 1]
                    n = t1 - t0
                    for i in range(n):
                        part[t0 + i - tb0] = prod[base + i : base + i + S * n : n].sum()
            else:
                bw, fnz = A["block_begin_warp_index_offset"], A["global_warp_block_first_nz"]
                part = np.array([prod[fnz[w] : fnz[w + 1]].sum() for w in range(bw[b], bw[b + 1])])
            g0 = roff[r0]
            for r in range(r0, r1):
                if r >= eff:
                    break
                y[row_dev(r)] += part[roff[r] - g0 : roff[r + 1] - g0].sum()
    elif t in ("K9", "K10"):
        fr = A["global_first_row_index_of_warp_level_block"]
        meta = man.sub_arrays(si)["combine_meta_of_thread_level_block"][0]
        S, bw_, brow, boff = s["tlb_size"], s["bits_word"], s["bits_row"], s["bits_off"]
        T = len(meta)
        for w in range(T // 32):
            R0 = fr[w]
            cur = None  # row currently accumulating (relative to R0); None before the warp's first flag
            for lane in range(32):
                m = int(meta[w * 32 + lane])
                frow = m & ((1 << brow) - 1)
                yo = frow
                seen = False
                for k in range(S):
                    flag = (m >> (bw_ - 1 - k)) & 1
                    if flag:
                        if seen:
                            yo += 1
                        seen = True
                        cur = yo
                    assert cur is not None, "warp does not start with a row-start flag"
                    nz = w * 32 * S + k * 32 + lane
                    y[row_dev(R0 + cur)] += prod[nz]
    else:
        raise ValueError(t)
