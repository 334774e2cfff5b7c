"""Enumerate-and-time search over Operator Graphs and launch parameters.

The loop structure follows the reference's tuner:
  * dense-view strategies (whilte_list_path_impl.cc:4230, 4330, 4579): G1 compress only; G2 exponential
    row division; G3 coarse sort (step 1) + exponential row division with several (min, rate);
  * per sub-matrix, whitelist strategies gated on its row-nnz statistics
    (find_best_path_of_compressed_sub_matrix, whilte_list_path_impl.cc:3411-3960), each a
    compressed-view graph skeleton with a small node-parameter grid and one template;
  * per template, a launch-parameter sweep (default_auto_tuner.cc:449-2030) with integer ranges in
    the param_enumerater.cc sense (`lo, lo+step, ... <= hi`);
  * points whose padded / true nnz exceeds PADDING_RATE_UP_BOUND are skipped.
Every trial is an in-process lowering + upload + CUDA-event timing through the C ABI instead of an
nvcc compile and an ~8 s run of a generated program; sub-matrices not under test carry the EMPTY
template, as in the reference's part_execute_code_builder.
"""
from __future__ import annotations

import dataclasses
import math

from . import capi
from .graph import Format, Matrix
from .matrices import CsrMatrix

PADDING_RATE_UP_BOUND = 4.0  # global_config.json of the reference
MAX_TBLOCK_NUM = 2**31 - 1  # the reference's 65535 grid cap is obsolete on sm_100
TEMPLATE_OF_ID = {v: k for k, v in capi.TEMPLATE.items()}


class SearchStrategy:
    """Stop rule of the reference's search loop (search_strategy.cc:5-80): a budget of steps that is
    refilled whenever a trial beats the best GFLOP/s so far (5 steps per GFLOP/s gained, clamped to
    5..25), then `struggle_step_num` further steps, and a wall-clock limit over everything."""

    def __init__(self, struggle_step_num: int = 10, total_allow_search_time: float = float("inf"), clock=None):
        import time

        self._clock = clock or time.monotonic
        self.remain_step_num = 10
        self.struggle_step_num = int(struggle_step_num)
        self.total_allow_search_time = float(total_allow_search_time)
        self.begin_time = self._clock()
        self.best_gflops = 0.0

    def _out_of_time(self) -> bool:
        return self._clock() - self.begin_time >= self.total_allow_search_time

    def continue_search(self, gflops: float | None = None) -> bool:
        """With a trial's GFLOP/s: account for it, then say whether to go on. Without: only ask."""
        if gflops is None:
            if self._out_of_time():
                return False
            return not (self.remain_step_num == 0 and self.struggle_step_num == 0)
        if gflops > self.best_gflops:
            self.remain_step_num = max(5, min(25, int((gflops - self.best_gflops) * 5)))
            self.best_gflops = gflops
        elif self.remain_step_num > 0:
            self.remain_step_num -= 1
        elif self.struggle_step_num > 0:
            self.struggle_step_num -= 1
        else:
            return False
        return not self._out_of_time()


def integer_range(lo: int, hi: int, step: int):
    """register_integer_independ_param_to_enumerater semantics: lo, lo+step, ... while <= hi."""
    v = lo
    while v <= hi:
        yield v
        v += step


def _ceil32(v: int) -> int:
    return (v + 31) // 32 * 32


@dataclasses.dataclass
class Candidate:
    name: str
    nodes: list  # compressed-view node lines without the "sub <id>" prefix
    template: str
    launches: list  # [(threads, row_reduce)]

    def lines(self, sub) -> str:
        return "\n".join(f"sub {sub} {n}" for n in self.nodes + [f"template {self.template}"])


@dataclasses.dataclass
class Trial:
    dense: str
    sub: int
    name: str
    launch: tuple
    ms: float
    gflops: float
    padding_rate: float


def compressed_candidates(mn: int, mx: int, avg: float, is_sorted: bool, quick: bool = True) -> list[Candidate]:
    """Strategies that apply to a sub-matrix with row nnz in [mn, mx] (mean avg). `quick` keeps one
    or two node-parameter points per strategy and a short launch sweep."""
    out: list[Candidate] = []
    T3 = [128, 256] if quick else list(integer_range(32, 256, 32))
    if mn >= 128:
        # strategy 8: BLB_COL_DIV(c) -> long-row template; c = 128 .. min(4096, ceil32(max)) x2
        cs, c = [], 128
        while c <= min(4096, _ceil32(mx)):
            cs.append(c)
            c *= 2
        for c in (cs[-2:] if quick else cs):
            out.append(Candidate(f"S8_K7_c{c}", [f"blb_col_fixed {c}"], "K7", [(t, 1) for t in sorted({min(1024, max(32, c // 16)), min(1024, max(64, c // 8)), min(1024, max(64, c // 4))})]))
    if mx <= 512:
        out.append(Candidate("S5_K3", ["row_padding 32 1", "tlb_row"], "K3", [(t, 1) for t in T3]))
        for mm in ([128, 256] if quick else [64, 128, 192, 256]):
            out.append(Candidate(f"S1_K2_m{mm}", [f"row_padding {mm} 1", f"blb_row_evenly {mm}", "tlb_row"], "K2",
                                 [(t, 1) for t in (128, 256)]))
    if not is_sorted:
        # strategy 9: TLB_NNZ_DIV(s) -> CSR5-like templates, s = 2 .. min(avg, 32). Rows of any
        # length qualify (a long row simply spans many warps), so a skewed matrix can run as ONE
        # kernel with no row sort: y is then written in row order instead of scattered.
        hi = int(max(2, min(avg, 32)))
        ss = sorted({2, max(2, hi // 2), hi}) if quick else sorted(set(integer_range(2, hi, max(1, (hi - 2) // 3 or 1))))
        if mx > 512:
            ss = sorted(set(ss) | {8, 16})
        for s in ss:
            out.append(Candidate(f"S9_K9_s{s}", [f"tlb_nnz {s}"], "K9", [(t, 1) for t in (128, 256)]))
            out.append(Candidate(f"S9_K10_s{s}", [f"tlb_nnz {s}"], "K10", [(t, 1) for t in (128, 256)]))
    if mn >= 30 and mx <= 512:
        # strategy 4: WLB_COL_DIV(c) -> warp per row chunk; c from 32 up past the longest row
        step = max(32, _ceil32(max(1, (mx - mn) // 3)))
        cs = list(integer_range(32, _ceil32(mx) + step, step))
        for c in (cs[:1] + cs[-1:] if quick else cs):
            out.append(Candidate(f"S4_K4_c{c}", [f"wlb_col_fixed {c}"], "K4", [(t, 1) for t in ((128, 256) if quick else integer_range(32, 512, 64))]))
    if mn >= 32 and mx <= 1024:
        cs = list(integer_range(32, min(128, _ceil32(math.ceil(mx / 2))), 32)) or [32]
        for mm in ([4] if quick else [2, 4]):
            for c in (cs[-1:] if quick else cs):
                out.append(Candidate(f"S6_K8_m{mm}_c{c}", [f"row_padding {mm} 1", f"blb_row_evenly {mm}", f"wlb_col_fixed {c}"], "K8",
                                     [(t, r) for t in (128, 256) for r in (1, 4)]))
        for bb in ([512] if quick else [128, 512, 896]):
            for c in (cs[-1:] if quick else cs):
                out.append(Candidate(f"S7_K8_b{bb}_c{c}", [f"blb_row_nnz {bb}", f"wlb_col_fixed {c}"], "K8", [(t, r) for t in (128, 256) for r in (1, 4)]))
    if mx <= 1024:
        cs = list(integer_range(1, min(16, max(1, math.ceil(mx / 2))), 3))
        for mm in ([64] if quick else [32, 64]):
            for c in (cs[:2] if quick else cs):
                out.append(Candidate(f"S2_K6_m{mm}_c{c}", [f"row_padding {mm} 1", f"blb_row_evenly {mm}", f"tlb_col_fixed {c}"], "K6",
                                     [(t, r) for t in (128, 256) for r in (1, 4)]))
        if not quick:
            for bb in (128, 512, 896):
                for c in cs:
                    out.append(Candidate(f"S3_K6_b{bb}_c{c}", [f"blb_row_nnz {bb}", f"tlb_col_fixed {c}"], "K6", [(t, r) for t in (128, 256) for r in (1, 4, 16)]))
    return out


def derive_tblock(template: str, n_tlb: int, n_wlb: int, n_blb: int, threads: int) -> int:
    """Launch shapes the reference derives instead of searching (default_auto_tuner.cc:465-498,
    688-693): one CTA per BLB for the CTA-per-BLB templates, ceil(units / threads) otherwise."""
    if template in ("K2", "K6", "K7", "K8", "K1", "K5"):
        n = n_blb
    elif template == "K4":
        n = (32 * n_wlb + threads - 1) // threads
    else:  # K3, K9, K10: one thread per TLB
        n = (n_tlb + threads - 1) // threads
    return int(max(1, min(n, MAX_TBLOCK_NUM)))


def set_launch(fmt: Format, group: capi.PlanGroup, sub: int, threads: int, reduce: int):
    info = fmt.sub_info(sub)
    t = TEMPLATE_OF_ID[info.template_type]
    if t == "EMPTY":
        return
    group.set_launch(sub, derive_tblock(t, info.n_tlb, info.n_wlb, info.n_blb, threads), threads, reduce)


def dense_strategies(quick: bool = True) -> list[str]:
    """G1, G2, G3 of the reference (dense-view graphs before COMPRESS)."""
    out = ["dense compress", "dense rowdiv_exp 32 4096 4\ndense compress"]
    g3 = [(128, 8)] if quick else [(mn, r) for mn in (512, 128, 32) for r in (4, 8, 16)]
    for mn, r in g3:
        out.append(f"dense sort 1\ndense rowdiv_exp {mn} 4096 {r}\ndense compress")
    return out


def search_sub(ctx, cm: Matrix, sub: int, n_subs: int, is_sorted: bool, quick, warmup, reps, log, dense, trials, strategy=None):
    """Best (candidate, launch) for one sub-matrix of a compressed matrix. `strategy` (SearchStrategy)
    ends the sweep early once trials stop improving; at least one candidate is always timed."""
    rows, nnz, mn, mx = cm.sub_rows(sub)
    cands = compressed_candidates(mn, mx, nnz / max(1, rows), is_sorted, quick)
    best = None
    stop = False
    others = "\n".join(f"sub {j} template EMPTY" for j in range(n_subs) if j != sub)
    for cand in cands:
        spec = cand.lines(sub) + ("\n" + others if others else "")
        try:
            fmt = cm.execute(spec)
        except capi.AspError as e:
            if log:
                log(f"  sub {sub} {cand.name}: graph rejected ({e})")
            continue
        rate = fmt.padding_rate(sub)
        if rate > PADDING_RATE_UP_BOUND:
            fmt.close()
            continue
        try:
            group = fmt.upload(ctx)
        except capi.AspError as e:
            if log:
                log(f"  sub {sub} {cand.name}: upload rejected ({e})")
            fmt.close()
            continue
        for (th, red) in cand.launches:
            try:
                set_launch(fmt, group, sub, th, red)
                ms, gf = group.time(warmup=warmup, reps=reps)
            except capi.AspError as e:
                if log:
                    log(f"  sub {sub} {cand.name} {th, red}: failed ({e})")
                continue
            trials.append(Trial(dense, sub, cand.name, (th, red), ms, gf, rate))
            if log:
                log(f"  sub {sub} [{rows} rows, nnz/row {mn}..{mx}] {cand.name} threads={th} reduce={red}: {ms * 1e3:.1f} us")
            if best is None or ms < best[2]:
                best = (cand, (th, red), ms)
            if strategy is not None and not strategy.continue_search(gf):
                stop = True
                break
        group.close()
        fmt.close()
        if stop:
            if log:
                log(f"  sub {sub}: search budget used up after {cand.name}")
            break
    return best


def search(ctx: capi.Context, m: CsrMatrix, quick: bool = True, warmup: int = 2, reps: int = 10, log=None,
           dense_list: list[str] | None = None, max_subs: int = 5, struggle_step_num: int | None = None, time_limit_s: float | None = None):
    """Full search. Returns (Format, PlanGroup, trials, description of the winning graph). With
    `struggle_step_num` and / or `time_limit_s` every sub-matrix sweep runs under the reference's stop
    rule (SearchStrategy); by default every candidate is timed."""
    hm = Matrix.from_csr(m)
    trials: list[Trial] = []
    winner = None  # (ms, dense, [(cand, launch)])
    for dense in (dense_list if dense_list is not None else dense_strategies(quick)):
        cm = hm.dense(dense)
        n = cm.n_subs
        if n > max_subs or (n == 1 and "rowdiv" in dense):
            # the reference abandons row divisions that give too many strips or no split at all
            cm.close()
            continue
        if log:
            log(f"dense view: {dense.replace(chr(10), ' | ')} -> {n} sub-matrices")
        picks = []
        for sub in range(n):
            strat = None
            if struggle_step_num is not None or time_limit_s is not None:
                strat = SearchStrategy(struggle_step_num if struggle_step_num is not None else 10, time_limit_s if time_limit_s is not None else float("inf"))
            b = search_sub(ctx, cm, sub, n, "sort" in dense, quick, warmup, reps, log, dense, trials, strat)
            if b is None:
                picks = None
                break
            picks.append(b)
        if picks is not None:
            # time the whole matrix with the per-strip winners
            spec = "\n".join(c.lines(i) for i, (c, _, _) in enumerate(picks))
            fmt = cm.execute(spec)
            group = fmt.upload(ctx)
            for i, (_, (th, red), _) in enumerate(picks):
                set_launch(fmt, group, i, th, red)
            ms, gf = group.time(warmup=warmup, reps=max(reps, 20))
            if log:
                log(f"  whole matrix: {ms * 1e3:.1f} us  {gf:.1f} GFLOP/s")
            if winner is None or ms < winner[0]:
                if winner is not None:
                    winner[4].close()
                    winner[3].close()
                winner = (ms, dense, picks, fmt, group)
            else:
                group.close()
                fmt.close()
        cm.close()
    hm.close()
    if winner is None:
        raise RuntimeError("no graph could be built and timed for this matrix")
    ms, dense, picks, fmt, group = winner
    desc = {"dense": dense.replace("\n", " | "),
            "subs": [{"graph": c.name, "nodes": c.nodes, "template": c.template, "threads": l[0], "row_reduce": l[1]} for c, l, _ in picks]}
    return fmt, group, trials, desc


def build(ctx: capi.Context, m: CsrMatrix, desc: dict):
    """Lower and upload exactly the graph a previous search() described (no timing)."""
    hm = Matrix.from_csr(m)
    cm = hm.dense(desc["dense"].replace(" | ", "\n"))
    if cm.n_subs != len(desc["subs"]):
        raise ValueError(f"graph describes {len(desc['subs'])} sub-matrices, the dense view gives {cm.n_subs}")
    spec = "\n".join(Candidate(s["graph"], s["nodes"], s["template"], []).lines(i) for i, s in enumerate(desc["subs"]))
    fmt = cm.execute(spec)
    group = fmt.upload(ctx)
    for i, s in enumerate(desc["subs"]):
        set_launch(fmt, group, i, s["threads"], s["row_reduce"])
    cm.close()
    hm.close()
    return fmt, group
