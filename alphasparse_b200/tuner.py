"""Enumerate-and-time search over Operator Graphs and launch parameters.

The loop structure follows the reference's tuner (whilte_list_path_impl.cc: one whitelist
strategy per template family, gated on the row-nnz statistics of the sub-matrix;
default_auto_tuner.cc: per-template launch-parameter sweep; param_enumerater.cc: integer
ranges `lo, lo+step, ... <= hi`), but every trial is an in-process upload + CUDA-event timing
through the C ABI instead of an nvcc compile and an ~8 s run of a generated program.
"""
from __future__ import annotations

import dataclasses
import math

import numpy as np

from . import capi
from .graph import Matrix
from .matrices import CsrMatrix

PADDING_RATE_UP_BOUND = 4.0  # global_config.json of the reference
MAX_TBLOCK_NUM = 2**31 - 1  # the reference's 65535 grid cap is obsolete on sm_100


def integer_range(lo: int, hi: int, step: int):
    """register_integer_independ_param_to_enumerater semantics: lo, lo+step, ... while <= hi."""
    v = lo
    while v <= hi:
        yield v
        v += step


@dataclasses.dataclass
class Candidate:
    name: str
    spec: str
    template: str
    launches: list  # [(tblock | None, threads, row_reduce)]


@dataclasses.dataclass
class Trial:
    name: str
    spec: str
    launch: tuple
    ms: float
    gflops: float
    padding_rate: float


def row_stats(m: CsrMatrix):
    l = m.row_lengths()
    return int(l.min()), int(l.max()), float(l.mean())


def _ceil32(v: int) -> int:
    return (v + 31) // 32 * 32


def compressed_candidates(m: CsrMatrix, quick: bool = True) -> list[Candidate]:
    """Whitelist strategies that apply to a sub-matrix with these row-nnz statistics
    (find_best_path_of_compressed_sub_matrix, whilte_list_path_impl.cc:3411-3960). `quick`
    keeps one or two node-parameter points per strategy."""
    mn, mx, avg = row_stats(m)
    out: list[Candidate] = []
    if mx <= 512:
        # strategy 5: ROW_PADDING(32,1) -> TLB_ROW_DIV -> ELL-like; threads 32..256 step 32
        th = [64, 128, 256] if quick else list(integer_range(32, 256, 32))
        out.append(Candidate("S5_K3", "sub all row_padding 32 1\nsub all tlb_row\nsub all template K3", "K3", [(None, t, 1) for t in th]))
        # strategy 1: ROW_PADDING(m,1) -> BLB_ROW_DIV(m) -> TLB_ROW_DIV -> SELL-like, m in {64,128,192,256}
        for mm in ([128, 256] if quick else [64, 128, 192, 256]):
            out.append(Candidate(f"S1_K2_m{mm}", f"sub all row_padding {mm} 1\nsub all blb_row_evenly {mm}\nsub all tlb_row\nsub all template K2", "K2",
                                 [(None, t, 1) for t in sorted({max(32, mm // 4), max(32, mm // 2), mm})]))
    if mx <= 1024:
        # strategy 2: ROW_PADDING(m,1) -> BLB_ROW_DIV(m) -> TLB_COL_DIV(c) -> row-grouped, m in {32,64}
        cs = [c for c in integer_range(1, min(16, max(1, math.ceil(mx / 2))), 3)]
        for mm in ([64] if quick else [32, 64]):
            for c in (cs[:2] if quick else cs):
                out.append(Candidate(f"S2_K6_m{mm}_c{c}", f"sub all row_padding {mm} 1\nsub all blb_row_evenly {mm}\nsub all tlb_col_fixed {c}\nsub all template K6", "K6",
                                     [(None, t, r) for t in (128, 256) for r in (1, 4)]))
    return out


def derive_tblock(template: str, info, n_tlb: int, n_wlb: int, n_blb: int, threads: int) -> int:
    """Launch shapes the reference derives instead of searching (default_auto_tuner.cc:465-498,
    688-693): one CTA per BLB for the CTA-per-BLB templates, ceil(units / threads) otherwise."""
    if template in ("K2", "K6", "K7", "K8", "K1", "K5"):
        n = n_blb
    elif template == "K3":
        n = (n_tlb + threads - 1) // threads
    elif template == "K4":
        n = (32 * n_wlb + threads - 1) // threads
    else:  # K9 / K10: one thread per TLB
        n = (n_tlb + threads - 1) // threads
    return int(max(1, min(n, MAX_TBLOCK_NUM)))


def search(ctx: capi.Context, m: CsrMatrix, candidates: list[Candidate] | None = None, dense: str = "dense compress",
           warmup: int = 2, reps: int = 10, log=None):
    """Time every (graph, launch) point; return (best Format, best PlanGroup, trials)."""
    hm = Matrix.from_csr(m)
    cands = candidates if candidates is not None else compressed_candidates(m)
    best = None
    trials: list[Trial] = []
    for cand in cands:
        spec = dense + "\n" + cand.spec
        try:
            fmt = hm.execute(spec)
        except capi.AspError as e:
            if log:
                log(f"{cand.name}: graph rejected ({e})")
            continue
        rate = max(fmt.padding_rate(i) for i in range(fmt.n_subs))
        if rate > PADDING_RATE_UP_BOUND:
            fmt.close()
            continue
        try:
            group = fmt.upload(ctx)
        except capi.AspError as e:
            if log:
                log(f"{cand.name}: upload rejected ({e})")
            fmt.close()
            continue
        kept = False
        for (tb, th, red) in cand.launches:
            try:
                for i in range(fmt.n_subs):
                    info = fmt.sub_info(i)
                    tbi = tb if tb else derive_tblock(cand.template, info, info.n_tlb, info.n_wlb, info.n_blb, th)
                    group.set_launch(i, tbi, th, red)
                ms, gf = group.time(warmup=warmup, reps=reps)
            except capi.AspError as e:
                if log:
                    log(f"{cand.name} {tb, th, red}: failed ({e})")
                continue
            trials.append(Trial(cand.name, spec, (tb, th, red), ms, gf, rate))
            if log:
                log(f"{cand.name} threads={th} reduce={red}: {ms * 1e3:.1f} us  {gf:.1f} GFLOP/s")
            if best is None or ms < best[2].ms:
                if best is not None and best[1] is not group:
                    best[1].close()
                    best[0].close()
                best = (fmt, group, trials[-1])
                kept = True
        if not kept or best[1] is not group:
            group.close()
            fmt.close()
    hm.close()
    if best is None:
        raise RuntimeError("no graph could be built and timed for this matrix")
    fmt, group, tr = best
    # re-apply the winning launch (later trials of the same group may have changed it)
    for i in range(fmt.n_subs):
        info = fmt.sub_info(i)
        tb, th, red = tr.launch
        tname = [k for k, v in capi.TEMPLATE.items() if v == info.template_type][0]
        group.set_launch(i, tb if tb else derive_tblock(tname, info, info.n_tlb, info.n_wlb, info.n_blb, th), th, red)
    return fmt, group, trials
