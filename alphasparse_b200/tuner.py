"""The search over Operator Graphs and launch parameters, as a thin layer over the C++ loop.

The loop itself (csrc/host/search.cpp, entry points asp_search / asp_search_gpu) follows the
reference's tuner:
  * dense-view strategies (whilte_list_path_impl.cc:4230, 4330, 4579): G1 compress only; G2 exponential
    row division; G3 coarse sort (step 1) + exponential row division with several (min, rate);
  * per sub-matrix, whitelist strategies gated on its row-nnz statistics
    (find_best_path_of_compressed_sub_matrix, whilte_list_path_impl.cc:3411-3960), each a
    compressed-view graph skeleton with a small node-parameter grid and one template;
  * per template, a launch-parameter sweep (default_auto_tuner.cc:449-2030) with integer ranges in
    the param_enumerater.cc sense (`lo, lo+step, ... <= hi`);
  * points whose padded / true nnz exceeds PADDING_RATE_UP_BOUND are skipped;
  * optionally the stop rule of search_strategy.cc per sub-matrix sweep.
Every trial is an in-process lowering + upload + CUDA-event timing through the C ABI instead of an
nvcc compile and an ~8 s run of a generated program; sub-matrices not under test carry the EMPTY
template, as in the reference's part_execute_code_builder.
"""
from __future__ import annotations

import ctypes as C
import dataclasses

from . import capi, graph
from .graph import Format, Matrix
from .matrices import CsrMatrix

PADDING_RATE_UP_BOUND = 4.0  # global_config.json of the reference
MAX_TBLOCK_NUM = 2**31 - 1  # the reference's 65535 grid cap is obsolete on sm_100
TEMPLATE_OF_ID = {v: k for k, v in capi.TEMPLATE.items()}


def integer_range(lo: int, hi: int, step: int):
    """register_integer_independ_param_to_enumerater semantics: lo, lo+step, ... while <= hi."""
    v = lo
    while v <= hi:
        yield v
        v += step


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
    padding_rate: float


def compressed_candidates(mn: int, mx: int, avg: float, is_sorted: bool, quick: bool = True) -> list[Candidate]:
    """Strategies that apply to a sub-matrix with row nnz in [mn, mx] (mean avg): what the C++ loop
    sweeps (asp_search_candidates). `quick` keeps one or two node-parameter points per strategy and
    a short launch sweep."""
    text = graph._lib().asp_search_candidates(int(mn), int(mx), float(avg), int(bool(is_sorted)), int(quick)).decode()
    out = []
    for line in text.splitlines():
        name, templ, nodes, launches = [f.strip() for f in line.split(";")]
        out.append(Candidate(name, nodes.split("|") if nodes else [], templ, [tuple(int(v) for v in l.split(":")) for l in launches.split(",") if l]))
    return out


def derive_tblock(template: str, n_tlb: int, n_wlb: int, n_blb: int, threads: int) -> int:
    """Launch shapes the reference derives instead of searching (default_auto_tuner.cc:465-498,
    688-693): one CTA per BLB for the CTA-per-BLB templates, ceil(units / threads) otherwise."""
    return int(graph._lib().asp_search_derive_tblock(capi.TEMPLATE[template], int(n_tlb), int(n_wlb), int(n_blb), int(threads)))


def set_launch(fmt: Format, group: capi.PlanGroup, sub: int, threads: int, reduce: int):
    info = fmt.sub_info(sub)
    t = TEMPLATE_OF_ID[info.template_type]
    if t == "EMPTY":
        return
    group.set_launch(sub, derive_tblock(t, info.n_tlb, info.n_wlb, info.n_blb, threads), threads, reduce)


def _options(quick, warmup, reps, max_subs, struggle_step_num, time_limit_s, log, prune_gbs=0.0, prune_min_bytes=0, strategies=None, checkpoint=None):
    opt = graph.SearchOptions()
    opt.quick = int(quick)  # 1 quick, 0 the reference's space plus extensions, 2 the reference's space exactly
    opt.warmup, opt.reps, opt.max_subs = int(warmup), int(reps), int(max_subs)
    opt.struggle_step_num = -1 if struggle_step_num is None else int(struggle_step_num)
    opt.time_limit_s = 0.0 if time_limit_s is None else float(time_limit_s)
    opt.padding_rate_up_bound = PADDING_RATE_UP_BOUND
    opt.prune_gbs, opt.prune_min_bytes = float(prune_gbs), int(prune_min_bytes)
    opt.strategy_mask = sum(1 << int(k) for k in strategies) if strategies else 0
    opt.checkpoint_path = checkpoint.encode() if checkpoint else None
    cb = graph.LOG_FN(lambda user, line: log(line.decode())) if log else graph.LOG_FN()
    opt.log_fn = cb
    return opt, cb  # the callback object must outlive the call


def _result(res_handle):
    """(description of the winning graph, trials, ms of the winner) from an asp_search_result, which is destroyed."""
    L = graph._lib()
    try:
        subs = []
        for i in range(L.asp_search_result_num_subs(res_handle)):
            pre = f"sub {i} "
            body = [ln[len(pre):] for ln in L.asp_search_result_sub_spec(res_handle, i).decode().splitlines()]
            th, rd = C.c_int64(), C.c_int64()
            graph._check(L.asp_search_result_sub_launch(res_handle, i, C.byref(th), C.byref(rd)))
            subs.append({"graph": L.asp_search_result_sub_name(res_handle, i).decode(), "nodes": body[:-1], "template": body[-1].split()[1],
                         "threads": int(th.value), "row_reduce": int(rd.value)})
        desc = {"dense": L.asp_search_result_dense(res_handle).decode().replace("\n", " | "), "subs": subs}
        trials = []
        for i in range(L.asp_search_result_num_trials(res_handle)):
            dense, sub, name, th, rd, ms, rate = [f.strip() for f in L.asp_search_result_trial(res_handle, i).decode().split(";")]
            trials.append(Trial(dense, int(sub.split()[1]), name, (int(th), int(rd)), float(ms), float(rate)))
        return desc, trials, float(L.asp_search_result_ms(res_handle))
    finally:
        L.asp_search_result_destroy(res_handle)


def search(ctx: capi.Context, m: CsrMatrix, quick: bool = True, warmup: int = 2, reps: int = 10, log=None, max_subs: int = 5,
           struggle_step_num: int | None = None, time_limit_s: float | None = None, prune_gbs: float = 0.0, checkpoint: str | None = None):
    """Full search on the GPU of `ctx` (asp_search_gpu). Returns (Format, PlanGroup, trials,
    description of the winning graph). With `struggle_step_num` and / or `time_limit_s` every
    sub-matrix sweep runs under the reference's stop rule; by default every candidate is timed.
    `prune_gbs` > 0 (an upper bound of the memory bandwidth in GB/s) skips candidates whose format
    cannot be read in the best time found so far."""
    hm = Matrix.from_csr(m)
    opt, keep = _options(quick, warmup, reps, max_subs, struggle_step_num, time_limit_s, log, prune_gbs, checkpoint=checkpoint)
    res = C.c_void_p()
    graph._check(graph._lib().asp_search_gpu(ctx.handle, hm._h, C.byref(opt), C.byref(res)))
    del keep
    desc, trials, _ = _result(res)
    hm.close()
    fmt, group = build(ctx, m, desc)
    return fmt, group, trials, desc


def search_with_timer(m: CsrMatrix, time_fn, quick: bool = True, warmup: int = 2, reps: int = 10, log=None, max_subs: int = 5,
                      struggle_step_num: int | None = None, time_limit_s: float | None = None, prune_gbs: float = 0.0, prune_min_bytes: int = 0, strategies=None, checkpoint: str | None = None):
    """asp_search with a caller-supplied timer `time_fn(fmt: Format, tblock, threads, reduce) -> ms or
    None` (None: the point cannot run). No GPU involved: used to test the loop against a model.
    Returns (description, trials, ms of the winner)."""
    hm = Matrix.from_csr(m)
    opt, keep = _options(quick, warmup, reps, max_subs, struggle_step_num, time_limit_s, log, prune_gbs, prune_min_bytes, strategies, checkpoint)

    def cb(user, fmt_handle, tb, th, rd, w, r, ms_out):
        view = Format.borrowed(fmt_handle)
        n = view.n_subs
        ms = time_fn(view, [tb[i] for i in range(n)], [th[i] for i in range(n)], [rd[i] for i in range(n)])
        if ms is None:
            return 1
        ms_out[0] = float(ms)
        return 0

    cfn = graph.TIME_FN(cb)
    res = C.c_void_p()
    graph._check(graph._lib().asp_search(hm._h, C.byref(opt), cfn, None, C.byref(res)))
    del keep
    out = _result(res)
    hm.close()
    return out


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


def build_row_chunks(ctx: capi.Context, m: CsrMatrix, desc: dict, n_chunks: int, align: int = 1):
    """The matrix cut into `n_chunks` row chunks of about equal size (boundaries at multiples of `align`), each lowered
    and uploaded on its own with the graph `desc` and global column indices: what asp_spmv_host_pipelined and the
    sharded loop take. Returns [(Format, PlanGroup, first row, end row, 1 + the largest column the chunk reads)]."""
    import numpy as np

    step = -(-m.n_rows // n_chunks)
    step = -(-step // align) * align
    out = []
    lo = 0
    while lo < m.n_rows:
        hi = min(m.n_rows, lo + step)
        sub = m.row_slice(lo, hi)
        if sub.nnz == 0:
            raise ValueError(f"rows [{lo}, {hi}) have no non-zeros: cut the chunks differently")
        fmt, group = build(ctx, sub, desc)
        out.append((fmt, group, lo, hi, int(np.max(sub.indices)) + 1))
        lo = hi
    return out


def write_trials_jsonl(path: str, m: CsrMatrix, trials, peak_gbs: float | None = None, append: bool = False) -> int:
    """One JSON object per timed point of a search (the reference prints to stdout and keeps ML rows in a CSV,
    machine_learning_data_set_collector.cc): dense-view graph, sub-matrix, candidate, launch, milliseconds, padding
    rate, and the derived GFLOP/s, algorithmic GB/s and, with `peak_gbs`, the roofline fraction. Returns the number
    of lines written."""
    import json

    b_alg = m.algorithmic_bytes()
    n = 0
    with open(path, "a" if append else "w") as fh:
        for t in trials:
            rec = {"dense": t.dense, "sub": t.sub, "graph": t.name, "threads": t.launch[0], "row_reduce": t.launch[1], "ms": t.ms,
                   "padding_rate": t.padding_rate, "rows": m.n_rows, "nnz": m.nnz, "dtype": str(m.values.dtype)}
            if t.ms > 0:
                rec["gflops"] = 2.0 * m.nnz / (t.ms * 1e-3) * 1e-9
                rec["algorithmic_GBs"] = b_alg / (t.ms * 1e-3) * 1e-9
                if peak_gbs:
                    rec["roofline_frac"] = rec["algorithmic_GBs"] / peak_gbs
            fh.write(json.dumps(rec) + "\n")
            n += 1
    return n
