"""Benchmark of the SpMV hot path: y = A x over the machine-designed formats.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c5|c1|c2|c3|c4|c4s] [--impl reference]

Default workload (every N, N = 1 included): the sharded graph configuration, R-MAT scale 26
(67,108,864 rows, ~1.06e9 non-zeros, fp32) generated on the GPUs, cost-balanced row blocks, x
replicated, ONE STEP = 100 repeated SpMVs (x <- A x). Strong scaling: the matrix is the same at every
N. The loop runs on P A P^T, the vertices renumbered by column count (--relabel): a step takes x0 in the
matrix's own numbering, permutes it in, iterates, and permutes the result out. With N > 1 every rank
cuts its block into row chunks and stores each finished chunk once through an NVLink multicast address
(NVSwitch replicates it) on a second stream, under the next chunk's kernel; one bounded-wait barrier
kernel per SpMV orders the ranks (--exchange: the other forms that were measured); the loop is enqueued
by one native call (asp_dist_spmv_iter, --loop). At N = 1 the line also carries `configs`: the
single-GPU configurations (c1..c4) replayed with the graphs the search picked for them, each with its
own time, roofline fraction and parity (c2 and c4 also with the host-to-host calls, plain and pipelined).

--workload c1|c2|c3|c4|c4s runs one single-GPU configuration as the main line (a step is one SpMV);
the graph is searched on the GPU (asp_search_gpu) unless --graph / --spec fixes it.

--impl reference times the CPU restatement of the reference's SpMV (oracle/csr_spmv.c, OpenMP over all
host cores) on the SAME matrix (for c5: the same scale-26 R-MAT, generated on the GPU and copied to the
host), one SpMV pass per step: the reference has no host SpMV of its own and its GPU path needs nvcc at
run time plus a per-matrix generated program.

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from alphasparse_b200 import matrices  # noqa: E402

WORKLOADS = {
    "c1": ("uniform random 4096^2 fp32, Poisson(16) per row, seed 0", lambda: matrices.uniform_random(4096, 16, 0)),
    "c2": ("5-point Laplacian 2048x2048 fp64, seed 1", lambda: matrices.laplacian_2d(2048, 1)),
    "c3": ("power-law 8388608^2 fp32, Zipf(2.1) rows capped at 500000, seed 2", lambda: matrices.power_law(8_388_608, 2.1, 500_000, 2)),
    "c4": ("3x3-block FEM-like fp64, 1048576 block rows x 27 blocks, seed 3", lambda: matrices.block_fem(1_048_576, 27, 4096, 3)),
    "c4s": ("3x3-block FEM-like fp64, 1048576 block rows x 9 blocks, seed 3", lambda: matrices.block_fem(1_048_576, 9, 4096, 3)),
}

# Two more matrices, only for profiling the kernel families that none of the five configurations ends up on
# (warp / CTA per row chunk, the shared-memory row reduce): medium rows and long rows, columns uniformly random.
def _rows_between(lo, hi, n_rows, n_cols, seed):
    rng = np.random.default_rng(seed)
    return matrices.from_row_lengths(rng.integers(lo, hi + 1, size=n_rows), n_cols, seed=seed)


WORKLOADS["pmid"] = ("profiling matrix: 1,000,000 rows of 40..120 non-zeros, fp32, random columns", lambda: _rows_between(40, 120, 1_000_000, 1_000_000, 21))
WORKLOADS["plong"] = ("profiling matrix: 60,000 rows of 1000..3000 non-zeros, fp32, random columns", lambda: _rows_between(1000, 3000, 60_000, 1_000_000, 22))

# The graphs the GPU search (`bench.py --workload cK`) picked for the single-GPU configurations; the default
# run replays them after its own timed region instead of searching again.
COMMITTED_GRAPHS = {
    "c1": {"dense": "dense compress", "subs": [{"graph": "S2_K6_m64_c4", "nodes": ["row_padding 64 1", "blb_row_evenly 64", "tlb_col_fixed 4"], "template": "K6", "threads": 128, "row_reduce": 1}]},
    # c2: the diagonal-value operator of this build (DIA storage: no column index per non-zero); the best graph over the
    # reference's own operators beside it
    "c2": {"dense": "dense compress", "subs": [{"graph": "S0_D1", "nodes": ["diag_value 64"], "template": "D1", "threads": 128, "row_reduce": 1}]},
    "c2_reference_operators": {"dense": "dense compress", "subs": [{"graph": "S5_K3", "nodes": ["row_padding 32 1", "tlb_row"], "template": "K3", "threads": 128, "row_reduce": 1}]},
    "c3": {"dense": "dense compress", "subs": [{"graph": "S9_K9_s16", "nodes": ["tlb_nnz 16"], "template": "K9", "threads": 128, "row_reduce": 2}]},
    # c4: the block-value operator of this build (one block-column index per 3 x 3 block); the best graph over the
    # reference's own operators is kept beside it, and the default run reports both
    "c4": {"dense": "dense compress", "subs": [{"graph": "S0_B1_3x3", "nodes": ["block_value 3 3"], "template": "B1", "threads": 128, "row_reduce": 1}]},
    "c4_reference_operators": {"dense": "dense compress", "subs": [{"graph": "S1_K2_m128", "nodes": ["row_padding 128 1", "blb_row_evenly 128", "tlb_row"], "template": "K2", "threads": 256, "row_reduce": 1}]},
}
COMMITTED_GRAPHS["c4s"] = COMMITTED_GRAPHS["c4"]
WORKLOADS["c4_reference_operators"] = WORKLOADS["c4"]
WORKLOADS["c2_reference_operators"] = WORKLOADS["c2"]


def profiled_traffic(workload: str, graph_desc) -> float | None:
    """dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the dominant kernel, from the table in
    profiles/dram_traffic.md (rows `| workload | graph | bytes | ...`); None when this graph has no capture."""
    subs = graph_desc.get("subs", []) if isinstance(graph_desc, dict) else []
    if len(subs) != 1:
        return None
    p = os.path.join(ROOT, "profiles", "dram_traffic.md")
    if not os.path.exists(p):
        return None
    workload = workload.split("_")[0]  # "c4_reference_operators" is c4 with another graph
    for line in open(p):
        f = [c.strip() for c in line.strip().strip("|").split("|")]
        if len(f) >= 3 and f[0] == workload and f[1] == subs[0].get("graph"):
            try:
                return float(f[2])
            except ValueError:
                return None
    return None


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    def __init__(self, device: int):
        super().__init__(daemon=True)
        self.device = device
        self.stop_flag = threading.Event()
        self.samples = []
        self.reasons = set()
        self.max_mhz = None

    def run(self):
        q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.device}", f"--query-gpu={q}", "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip().splitlines()
                if out:
                    f = [s.strip() for s in out[0].split(",")]
                    self.samples.append(float(f[0]))
                    self.max_mhz = float(f[1])
                    for n, v in zip(names, f[2:]):
                        if v.lower().startswith("active"):
                            self.reasons.add(n)
            except Exception:
                pass
            self.stop_flag.wait(0.1)

    def summary(self):
        return {"sm_mhz": float(np.median(self.samples)) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def use_all_host_cores(share: int = 1):
    """torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU legs are meant to use every host core this
    process may run on (the OpenMP runtime reads the variable when the first OpenMP library loads). `share`:
    number of local ranks that build their formats at the same time and split the cores."""
    os.environ["OMP_NUM_THREADS"] = str(max(1, len(os.sched_getaffinity(0)) // max(1, share)))


def oracle():
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import refdump

    return refdump


def cpu_baseline(m, x, budget_s: float = 12.0, reps_min: int = 2, reps_max: int = 200):
    """The CPU restatement of the reference's SpMV, timed on all host cores over repeated passes of the same
    matrix until `budget_s` is used. Returns (GFLOP/s, threads, passes, median seconds)."""
    rd = oracle()
    threads = int(rd.oracle_lib().asp_oracle_max_threads())
    rd.csr_native(m, x)  # warm-up and page touch
    t0 = time.perf_counter()
    times = []
    while len(times) < reps_min or (time.perf_counter() - t0 < budget_s and len(times) < reps_max):
        s = time.perf_counter()
        rd.csr_native(m, x)
        times.append(time.perf_counter() - s)
    med = float(np.median(times))
    return 2.0 * m.nnz / med * 1e-9, threads, len(times), med


def check_against_oracle(m, x_host, y_host) -> float:
    """max_i |y_i - y_ref_i| / sum_j |a_ij||x_j| against the CPU oracle: the whole matrix up to 3e8 non-zeros, else
    three row windows (head, middle, tail) of about 2e7 non-zeros each."""
    rd = oracle()
    if m.nnz <= 300_000_000:
        windows = [(0, m.n_rows)]
    else:
        windows = []
        for frac in (0.0, 0.5, 1.0):
            target = int(frac * (m.nnz - 20_000_000))
            a = int(np.searchsorted(m.indptr, target, side="left"))
            b = int(np.searchsorted(m.indptr, target + 20_000_000, side="right")) - 1
            a = min(a, m.n_rows - 1)
            windows.append((a, max(min(b, m.n_rows), a + 1)))
    worst = 0.0
    for a, b in windows:
        sub = m.row_slice(a, b) if (a, b) != (0, m.n_rows) else m
        y_ref, scl = rd.csr_ref(sub, x_host)
        worst = max(worst, rd.rel_err(y_host[a:b], y_ref, scl))
    return worst


def c5_host_matrix(scale: int):
    """The sharded workload's matrix as one host CSR: generated on the GPU (as the native arm does) when there is
    one, else with the numpy generator at a scale the host builds in seconds (then the sample says so)."""
    try:
        import torch

        if torch.cuda.is_available():
            from alphasparse_b200 import matrices_gpu

            dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
            indptr, cols, vals = matrices_gpu.rmat_block(scale, 16, 4, 0, 1 << scale, dev)
            m = matrices_gpu.to_host_csr(indptr, cols, vals, 1 << scale)
            x = matrices_gpu.rmat_x(scale, 4, dev).cpu().numpy()
            del indptr, cols, vals
            torch.cuda.empty_cache()
            return m, x, scale
    except Exception as e:  # no usable GPU: fall through to the host generator
        print(f"[reference] GPU generation unavailable ({e!r}); using the host generator", file=sys.stderr)
    sc = min(scale, 20)
    m, x = matrices.rmat(sc, 16, seed=4)
    return m, x, sc


def run_reference(args, rank, world):
    if rank != 0:
        return
    use_all_host_cores()
    if args.workload == "c5":
        m, x, sc = c5_host_matrix(args.scale)
        desc = f"R-MAT scale {sc}, edge factor 16, a/b/c/d .57/.19/.19/.05, seed 4"
        sample = (f"each step is ONE SpMV pass over the whole scale-{sc} matrix ({m.nnz} non-zeros) out of the 100 a native step runs"
                  + ("" if sc == args.scale else f"; scale {sc} instead of {args.scale}: no GPU to generate the matrix on"))
    else:
        desc, gen = WORKLOADS[args.workload]
        m, x = gen()
        sample = f"each step is one full SpMV pass of the {args.workload} matrix"
    W, K = max(args.warmup, 1), max(args.steps, 1)
    rd = oracle()
    threads = int(rd.oracle_lib().asp_oracle_max_threads())
    t_w = time.perf_counter()
    rd.csr_native(m, x)
    first = time.perf_counter() - t_w
    # bounded: the whole run is meant to end within a few minutes
    if first * (W + K) > 240.0:
        W = 1
    for _ in range(W - 1):
        rd.csr_native(m, x)
    t0 = time.perf_counter()
    for _ in range(K):
        rd.csr_native(m, x)
    dt = (time.perf_counter() - t0) / K
    gf = 2.0 * m.nnz / dt * 1e-9
    es = m.values.dtype.itemsize
    b_alg = m.nnz * (es + 4) + 4 * (m.n_rows + 1) + es * (m.n_rows + m.n_cols)
    line = {
        "impl": "reference", "metric": "SpMV GFLOP/s", "value": gf, "unit": "GFLOP/s", "n_gpus": args.gpus, "steps": K, "warmup": max(args.warmup, 1),
        "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong" if args.workload == "c5" else "weak", "vs_baseline": None,
        "dtype": "f64" if es == 8 else "f32", "data": "synthetic",
        "config": {"workload": args.workload, "description": desc, "rows": m.n_rows, "nnz": m.nnz, "algorithmic_GBs": b_alg / dt * 1e-9},
        "cpu_baseline": {"value": gf, "unit": "GFLOP/s", "cores": threads, "kind": "port", "sample": sample + "; OpenMP row-parallel CSR loop, accumulation in the value type"},
        "e2e": {"value": gf, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def time_group(ctx, group, dx, dy, zero_y, stream, warmup: int, min_batch_s: float = 0.2, batches: int = 5):
    """Median over `batches` batches, each long enough (>= min_batch_s) that clock samples fall inside it, of
    the time per SpMV (CUDA events on the launching stream). Returns (ms per SpMV, reps per batch, all batch ms)."""
    import torch

    def step():
        group.spmv(dx.data_ptr(), dy.data_ptr(), zero_y)

    for _ in range(max(warmup, 3)):
        step()
    ctx.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(10):
        step()
    e1.record(stream)
    e1.synchronize()
    est = max(e0.elapsed_time(e1) / 10, 1e-3)
    reps = int(min(max(50, min_batch_s * 1e3 / est), 20000))
    out = []
    for _ in range(batches):
        e0.record(stream)
        for _ in range(reps):
            step()
        e1.record(stream)
        e1.synchronize()
        out.append(e0.elapsed_time(e1) / reps)
    return float(np.median(out)), reps, out


def run_single(ctx, name: str, graph_desc, peak: float, log=None, searched=None):
    """One single-GPU configuration: build the matrix, lower `graph_desc` (or search when None), time, check."""
    import torch

    from alphasparse_b200 import capi, tuner

    desc, gen = WORKLOADS[name]
    t0 = time.perf_counter()
    m, x = gen()
    gen_s = time.perf_counter() - t0
    t0 = time.perf_counter()
    trials = []
    if graph_desc is None:
        fmt, group, trials, graph_desc = tuner.search(ctx, m, quick=True, log=log)
    else:
        fmt, group = tuner.build(ctx, m, graph_desc)
    build_s = time.perf_counter() - t0
    val_t = torch.float64 if m.values.dtype == np.float64 else torch.float32
    dx = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    dy = torch.zeros(m.n_rows, dtype=val_t, device="cuda")
    stream = torch.cuda.ExternalStream(ctx.stream)
    zero_y = "auto" if int(m.row_lengths().min()) > 0 else True
    ms, reps, batches = time_group(ctx, group, dx, dy, zero_y, stream, warmup=5)
    ctx.synchronize()
    rd = oracle()
    y_ref, scale = rd.csr_ref(m, x)
    parity = rd.rel_err(dy.cpu().numpy(), y_ref, scale)
    b_alg = m.algorithmic_bytes()
    achieved = b_alg / (ms * 1e-3) * 1e-9
    out = {"description": desc, "rows": m.n_rows, "nnz": m.nnz, "dtype": "f64" if m.values.dtype == np.float64 else "f32", "graph": graph_desc,
           "ms_per_spmv": ms, "gflops": 2.0 * m.nnz / (ms * 1e-3) * 1e-9, "achieved_GBs": achieved, "frac": achieved / peak, "algorithmic_bytes": b_alg,
           "traffic": profiled_traffic(name, graph_desc), "parity_max_rel_err": parity, "reps_per_batch": reps, "batches_ms": [round(b, 5) for b in batches],
           "padding_rate": round(max(fmt.padding_rate(i) for i in range(fmt.n_subs)), 4), "format_MB": round(group.format_bytes() / 1e6, 1),
           "generate_s": round(gen_s, 1), "build_s": round(build_s, 1), "trials": len(trials)}
    if name.split("_")[0] in ("c2", "c4") and "_reference_" not in name:
        try:
            out["host_to_host"] = host_to_host(ctx, m, x, group, graph_desc, y_ref, scale, HOST_CHUNKS)
        except Exception as e:  # an extra: never takes the configuration's line down
            out["host_to_host"] = {"error": repr(e)[:200]}
    keep = {"m": m, "x": x, "fmt": fmt, "group": group, "dx": dx, "dy": dy, "stream": stream, "zero_y": zero_y}
    return out, keep


HOST_CHUNKS = 4  # measured: 4 chunks 0.96 ms, 8 chunks 0.98, 16 chunks 1.14 (c2; per-chunk copies of 2 MB are latency-bound)


def host_to_host(ctx, m, x, group, graph_desc, y_ref, scale, n_chunks: int = 16):
    """One SpMV with x and y in pinned HOST memory, through the plain call (copy in, kernel, copy out in series:
    asp_spmv_host) and through the pipelined one (row chunks, x as a growing prefix, y leaving chunk by chunk:
    asp_spmv_host_pipelined); milliseconds per call, median of 7."""
    import torch

    from alphasparse_b200 import capi, tuner

    rd = oracle()
    hx = torch.from_numpy(np.ascontiguousarray(x)).pin_memory()
    hy = torch.empty(m.n_rows, dtype=hx.dtype).pin_memory()

    def med(fn):
        ts = []
        for _ in range(9):
            t0 = time.perf_counter()
            fn()
            ts.append((time.perf_counter() - t0) * 1e3)
        return float(np.median(ts[2:]))

    L = capi.lib()
    import ctypes as C

    plain = med(lambda: capi.check(L.asp_spmv_host(ctx.handle, group._plans, group.n, C.c_void_p(hx.data_ptr()), C.c_void_p(hy.data_ptr()))))
    err_plain = rd.rel_err(hy.numpy(), y_ref, scale)
    chunks = tuner.build_row_chunks(ctx, m, graph_desc, n_chunks, align=96)
    try:
        arg = [(g, lo, hi, ch) for _, g, lo, hi, ch in chunks]
        hy.fill_(0)
        piped = med(lambda: capi.spmv_host_pipelined(ctx, arg, hx.data_ptr(), hy.data_ptr()))
        err_piped = rd.rel_err(hy.numpy(), y_ref, scale)
    finally:
        for f, g, *_ in chunks:
            g.close()
            f.close()
    es = hx.element_size()
    return {"ms_plain_call": plain, "ms_pipelined_call": piped, "row_chunks": len(chunks), "parity_plain": err_plain, "parity_pipelined": err_piped,
            "h2d_bytes": int(m.n_cols * es), "d2h_bytes": int(m.n_rows * es),
            "note": "x and y in pinned host memory; one direction of PCIe moves x or y in bytes / bandwidth, the plain call pays both in series"}


def release(keep):
    import torch

    torch.cuda.synchronize()
    keep["group"].close()
    keep["fmt"].close()
    keep.clear()
    torch.cuda.empty_cache()


def run_c5(args, rank, world, local_rank, dist):
    """Sharded R-MAT, repeated SpMV (alphasparse_b200/bench_rmat.py). One step = `iters` SpMVs."""
    import torch

    from alphasparse_b200 import bench_rmat, capi

    log = (lambda s: print(f"[rank {rank}] {s}", file=sys.stderr)) if args.verbose else None
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()  # stopped right after the timed region: its samples cover set-up (idle) and the timed steps
    t_start = time.perf_counter()
    r = bench_rmat.run(args, rank, world, local_rank, dist, log, check_fn=None if args.profile_launches else check_against_oracle)
    sampler.stop_flag.set()
    if r.get("profile_only"):
        if rank == 0:
            n_, nnz_ = r["rows"], r["nnz"]
            print(json.dumps({"profile_launches": args.profile_launches, "workload": "c5", "scale": args.scale, "nnz": nnz_, "rows": n_,
                              "algorithmic_bytes": nnz_ * 8 + 4 * (n_ + 1) + 8 * n_, "format_bytes": r["format_bytes"], "graph": r["graph"]}))
        return
    n, nnz, iters = r["rows"], r["nnz"], r["iters"]
    K, W = max(args.steps, 1), max(args.warmup, 3)
    b_alg = nnz * 8 + 4 * (n + 1) + 4 * (n + n)
    achieved = b_alg * iters / (r["ms_per_step"] * 1e-3) * 1e-9
    peak, peak_kind = measured_peak_gbs()
    # clock samples of the timed region only: the last timed_wall_s seconds before the sampler stopped
    # (0.1 s apart; the compute-only pass that follows the timed region is also under load)
    in_region = sampler.samples[-max(3, int(r["timed_wall_s"] / 0.13)) :] if sampler.samples else []
    clocks = sampler.summary()
    if in_region:
        clocks["sm_mhz"] = float(np.median(in_region))
        clocks["samples_in_timed_region"] = len(in_region)
    line = None
    if rank == 0:
        line = {
            "metric": "SpMV GFLOP/s", "value": r["gflops"], "unit": "GFLOP/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "c5", "description": f"R-MAT scale {args.scale}, edge factor 16, a/b/c/d .57/.19/.19/.05, seed 4, {iters} repeated SpMVs per step (x <- A x)",
                       "rows": n, "nnz": nnz, "rows_rank0": r["rows_local"], "nnz_rank0": r["nnz_local"], "graph": r["graph"],
                       "l2": "inputs larger than L2", "build_s": round(r["search_s"], 1), "generate_s": round(r["gen_s"], 1),
                       "ms_per_spmv": r["ms_per_spmv"], "ms_per_step_median": r["ms_per_step_median"], "ms_compute_per_spmv_max_over_ranks": r["ms_compute_per_spmv_max"],
                       "row_chunks_per_rank": r["chunks"], "balance": args.balance, "relabel": r["relabel"], "staged_row_sums": r["staged"],
                       "exchange": "none (1 GPU)" if world == 1 else {"publish": "rows leave the SpMV kernel through the NVLink multicast address (multimem.st), end rows of the warps by a small kernel after it",
                                                                       "multicast": "multicast store pass per row chunk on a second stream, overlapped with the next chunk's kernel"}.get(r["exchange_used"], r["exchange_used"]),
                       "barrier": r["barrier"], "loop": r["loop"], "exchange_fallback": r["fallback_reason"],
                       "values": "x grows by about 8x per SpMV and overflows fp32 after ~40 of the 100: the later SpMVs multiply inf / NaN (same memory traffic); parity is checked on the first SpMV"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak * world, "unit": "GB/s", "frac": achieved / (peak * world), "traffic": profiled_traffic("c5", r["graph"]) if (world == 1 and args.scale == 26 and args.relabel == "indegree") else None,
                         "peak_kind": peak_kind, "algorithmic_bytes": b_alg, "launch": f"{iters} SpMV launches per step; peak = {world} x the measured copy bandwidth",
                         "note": "the gathers of x are bound by cache-line look-ups per SM (one per clock), not by DRAM: see profiles/"},
            "gpu_launches": int(K * iters * r["launches_per_spmv"]),
            "clocks": clocks, "parity_max_rel_err": r["parity"],
        }
    # end to end (all ranks take part): x0 from pinned host memory in, final x out, every step
    sh, iterate = r["sharded"], r["iterate"]
    hx = r["x0"].cpu().pin_memory()
    hy = torch.empty_like(hx).pin_memory()
    dev_x = torch.empty_like(r["x0"])
    stream = torch.cuda.ExternalStream(r["ctx"].stream)
    Ke = max(1, min(K, 3))
    torch.cuda.synchronize()
    if dist:
        dist.barrier()
    t0 = time.perf_counter()
    with torch.cuda.stream(stream):
        for _ in range(Ke):
            dev_x.copy_(hx, non_blocking=True)
            xf = iterate(dev_x, iters)
            hy.copy_(xf, non_blocking=True)
            stream.synchronize()
    e2e_s = (time.perf_counter() - t0) / Ke
    sh.check_barrier_status()
    replicas_agree = None
    if dist:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
        # every rank must hold the same final x, bit for bit
        # (compared as bit patterns: an overflowed x turns into NaN, and NaN != NaN)
        bits = xf.view(torch.int32).to(torch.int64)
        chk = torch.stack([bits.sum(), (bits * (torch.arange(bits.numel(), device=bits.device) % 8191 + 1)).sum()])
        lo, hi = chk.clone(), chk.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        replicas_agree = bool(torch.equal(lo, hi))
        del bits, chk
    if rank == 0:
        line["e2e"] = {"value": 2.0 * nnz * iters / e2e_s * 1e-9, "unit": "GFLOP/s", "h2d_bytes_per_step": int(4 * n), "d2h_bytes_per_step": int(4 * n),
                       "ms_per_step": e2e_s * 1e3, "steps": Ke}
        line["replicas_agree"] = replicas_agree
        if world == 1 and not args.no_cpu_baseline:
            gf, threads, passes, med = cpu_baseline(r["m_local"], hx.numpy(), budget_s=10.0, reps_min=2, reps_max=5)
            line["cpu_baseline"] = {"value": gf, "unit": "GFLOP/s", "cores": threads, "kind": "port",
                                    "sample": f"{passes} SpMV passes over the whole matrix as the GPU loop holds it ({r['relabel']}; {nnz} nnz, median {med * 1e3:.0f} ms each) out of the {iters} of a step; OpenMP row-parallel CSR loop"}
    # Tear down in dependency order: torch frees pinned blocks by recording an event on the stream
    # they were last used on, and that stream belongs to the context object.
    torch.cuda.synchronize()
    ctx = r["ctx"]
    del hx, hy, dev_x, xf, stream, sh, iterate
    for g in r["group"]:
        g.close()
    for k in ("sharded", "x0", "group", "fmt", "m_local", "bufs", "iterate", "labels"):
        r.pop(k, None)
    import gc

    gc.collect()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    if rank == 0 and world == 1 and not args.no_configs:
        # the single-GPU configurations, replayed with their committed graphs (not part of the timed region above)
        line["configs"] = {}
        for name in args.configs.split(","):
            try:
                out, keep = run_single(ctx, name, COMMITTED_GRAPHS[name], peak, log)
                release(keep)
            except Exception as e:  # a sub-configuration never takes the main line down
                out = {"error": repr(e)[:300]}
            line["configs"][name] = out
            if time.perf_counter() - t_start > args.configs_budget_s:
                line["configs"]["skipped"] = f"time budget of {args.configs_budget_s:.0f} s used"
                break
    if rank == 0:
        line["wall_s"] = round(time.perf_counter() - t_start, 1)
        print(json.dumps(line), flush=True)
    r.pop("ctx", None)
    del ctx
    if dist:
        dist.barrier()
        dist.destroy_process_group()


def run_one_config(args, rank, world, local_rank, dist):
    """--workload c1|c2|c3|c4|c4s as the main line (single GPU: with N > 1 every rank runs its own replica)."""
    import torch

    from alphasparse_b200 import capi, tuner

    W, K = max(args.warmup, 3), max(args.steps, 1)
    log = (lambda s: print(f"[rank {rank}] {s}", file=sys.stderr)) if args.verbose else None
    peak, peak_kind = measured_peak_gbs()
    ctx = capi.Context(local_rank)
    graph_desc = None
    if args.graph:
        graph_desc = json.load(open(args.graph))["config"]["graph"] if os.path.exists(args.graph) else json.loads(args.graph)
    elif args.committed:
        graph_desc = COMMITTED_GRAPHS[args.workload]
    t_s = time.perf_counter()
    if args.spec:
        # one fixed graph (profiling runs): candidate name from the whitelist table, dense view from --dense
        from alphasparse_b200.graph import Matrix

        desc, gen = WORKLOADS[args.workload]
        m, x = gen()
        hm = Matrix.from_csr(m)
        cm = hm.dense(args.dense.replace("|", "\n"))
        if cm.n_subs != 1:
            raise SystemExit("--spec needs a dense view with one sub-matrix")
        rows_, nnz_, mn_, mx_ = cm.sub_rows(0)
        cand = [c for c in tuner.compressed_candidates(mn_, mx_, nnz_ / rows_, "sort" in args.dense, quick=False) if c.name == args.spec]
        if not cand:
            raise SystemExit(f"no candidate named {args.spec} applies to this matrix")
        th, red = (args.threads or cand[0].launches[0][0]), cand[0].launches[0][1]
        graph_desc = {"dense": args.dense.replace("|", " | "), "subs": [{"graph": cand[0].name, "nodes": cand[0].nodes, "template": cand[0].template, "threads": th, "row_reduce": red}]}
        cm.close()
        hm.close()
        del m, x
    if args.profile_launches and args.profile_specs:
        # several graphs over one matrix, a few launches each (one process for one ncu capture of several kernel families)
        from alphasparse_b200.graph import Matrix

        desc_, gen_ = WORKLOADS[args.workload]
        m_, x_ = gen_()
        hm = Matrix.from_csr(m_)
        cm = hm.dense("dense compress")
        rows_, nnz_, mn_, mx_ = cm.sub_rows(0)
        table = {c.name: c for c in tuner.compressed_candidates(mn_, mx_, nnz_ / rows_, False, quick=False)}
        dx_ = torch.from_numpy(np.ascontiguousarray(x_)).cuda()
        dy_ = torch.zeros(m_.n_rows, dtype=dx_.dtype, device="cuda")
        done, built = {}, []
        for name in args.profile_specs.split(","):
            # "<candidate>[@threads[:row_reduce]]"; the launches of all graphs come first (what a capture counts), the timings after
            name, _, launch = name.partition("@")
            cand = table[name]
            fmt_ = cm.execute(cand.lines(0))
            group_ = fmt_.upload(ctx)
            th, red = cand.launches[0]
            if launch:
                th, red = int(launch.split(":")[0]), (int(launch.split(":")[1]) if ":" in launch else red)
            tuner.set_launch(fmt_, group_, 0, th, red)
            for _ in range(args.profile_launches):
                group_.spmv(dx_.data_ptr(), dy_.data_ptr(), True)
            ctx.synchronize()
            built.append((name, th, red, fmt_, group_))
        for name, th, red, fmt_, group_ in built:
            ms, gf = group_.time(2, 10, True)
            done[name] = {"threads": th, "row_reduce": red, "launch": group_.get_launch(0), "format_bytes": group_.format_bytes(), "padding_rate": round(fmt_.padding_rate(0), 4), "ms": ms, "gflops": gf}
            group_.close()
            fmt_.close()
        print(json.dumps({"profile_launches": args.profile_launches, "workload": args.workload, "nnz": m_.nnz, "rows": m_.n_rows,
                          "algorithmic_bytes": m_.algorithmic_bytes(), "graphs": done}))
        cm.close()
        hm.close()
        return
    if args.profile_launches:
        desc_, gen_ = WORKLOADS[args.workload]
        m_, x_ = gen_()
        fmt_, group_ = tuner.build(ctx, m_, graph_desc) if graph_desc is not None else tuner.search(ctx, m_, quick=True)[:2]
        dx_ = torch.from_numpy(np.ascontiguousarray(x_)).cuda()
        dy_ = torch.zeros(m_.n_rows, dtype=dx_.dtype, device="cuda")
        for _ in range(args.profile_launches):
            group_.spmv(dx_.data_ptr(), dy_.data_ptr(), "auto" if int(m_.row_lengths().min()) > 0 else True)
        ctx.synchronize()
        print(json.dumps({"profile_launches": args.profile_launches, "workload": args.workload, "nnz": m_.nnz, "rows": m_.n_rows,
                          "algorithmic_bytes": m_.algorithmic_bytes(), "format_bytes": group_.format_bytes()}))
        group_.close()
        fmt_.close()
        return
    sampler = ClockSampler(local_rank)
    out, keep = run_single(ctx, args.workload, graph_desc, peak, log)
    search_s = time.perf_counter() - t_s
    m, x, group, dx, dy, stream, zero_y = (keep[k] for k in ("m", "x", "group", "dx", "dy", "stream", "zero_y"))
    if args.stage:
        for i in range(group.n):
            group.set_tuning(i, 0, 1)

    def step():
        group.spmv(dx.data_ptr(), dy.data_ptr(), zero_y)

    # the contract's bracket: W warm-up steps, then exactly K steps between two events, max over ranks
    for _ in range(W):
        step()
    ctx.synchronize()
    if dist:
        dist.barrier()
    if rank == 0:
        sampler.start()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(K):
        step()
    e1.record(stream)
    e1.synchronize()
    ms_total = e0.elapsed_time(e1)
    # and the median of 5 batches of >= 0.2 s each, during which the clocks are sampled
    ms_med, reps, batches = time_group(ctx, group, dx, dy, zero_y, stream, warmup=0)
    sampler.stop_flag.set()
    if dist:
        t = torch.tensor([ms_total], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / K

    # end to end through the host-buffer entry point: pinned x in, y out, every step
    val_t = torch.float64 if m.values.dtype == np.float64 else torch.float32
    hx = torch.from_numpy(np.ascontiguousarray(x)).pin_memory()
    hy = torch.empty(m.n_rows, dtype=val_t).pin_memory()
    plans = group._plans
    Ke = max(3, min(K, 30))
    for _ in range(2):
        capi.check(capi.lib().asp_spmv_host(ctx.handle, plans, group.n, C.c_void_p(hx.data_ptr()), C.c_void_p(hy.data_ptr())))
    if dist:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(Ke):
        capi.check(capi.lib().asp_spmv_host(ctx.handle, plans, group.n, C.c_void_p(hx.data_ptr()), C.c_void_p(hy.data_ptr())))
    e2e_s = (time.perf_counter() - t0) / Ke
    if dist:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())

    # launch-bound case (c1: the matrix lives in L2 and a kernel runs for a few microseconds): the same
    # SpMV replayed from a CUDA graph of 100 launches, so that host launch latency is out of the number
    graph_us = None
    if args.workload == "c1" and world == 1:
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(stream):
                with torch.cuda.graph(g, stream=stream):
                    for _ in range(100):
                        step()
                for _ in range(3):
                    g.replay()
                ge0, ge1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                ge0.record(stream)
                for _ in range(20):
                    g.replay()
                ge1.record(stream)
                ge1.synchronize()
            graph_us = ge0.elapsed_time(ge1) / 20 / 100 * 1e3
            del g
        except Exception as e:  # diagnostic extra, never fatal
            graph_us = f"unavailable: {e!r}"[:120]

    rd = oracle()
    y_ref, scale = rd.csr_ref(m, x)
    parity = rd.rel_err(hy.numpy(), y_ref, scale) if rank == 0 else None
    nnz_total = m.nnz * world
    b_alg = m.algorithmic_bytes()
    achieved = b_alg / (ms_step * 1e-3) * 1e-9
    if rank == 0:
        es = m.values.dtype.itemsize
        line = {
            "metric": "SpMV GFLOP/s", "value": 2.0 * nnz_total / (ms_step * 1e-3) * 1e-9, "unit": "GFLOP/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f64" if es == 8 else "f32", "data": "synthetic",
            "config": {"workload": args.workload, "description": out["description"] + ("" if world == 1 else f"; {world} independent replicas, one per GPU (replicas only: no data-path collective)"),
                       "rows": m.n_rows, "nnz": m.nnz, "graph": out["graph"], "l2": "inputs larger than L2 (format arrays %.0f MB)" % out["format_MB"],
                       "search_s": round(search_s, 2), "trials": out["trials"], "padding_rate": out["padding_rate"],
                       "ms_per_spmv_median_of_batches": ms_med, "reps_per_batch": reps, "batches_ms": [round(b, 5) for b in batches],
                       **({"us_per_spmv_from_a_cuda_graph_of_100": graph_us} if graph_us is not None else {}),
                       **({"host_to_host": out["host_to_host"]} if "host_to_host" in out else {})},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": profiled_traffic(args.workload, out["graph"]), "peak_kind": peak_kind, "algorithmic_bytes": b_alg,
                         "frac_median_of_batches": b_alg / (ms_med * 1e-3) * 1e-9 / peak,
                         "format_bytes": int(group.format_bytes() + es * (m.n_cols + m.n_rows))},
            "e2e": {"value": 2.0 * nnz_total / e2e_s * 1e-9, "unit": "GFLOP/s", "h2d_bytes_per_step": int(es * m.n_cols),
                    "d2h_bytes_per_step": int(es * m.n_rows), "ms_per_step": e2e_s * 1e3},
            "gpu_launches": int(K * group.launches()),
            "clocks": sampler.summary(),
            "parity_max_rel_err": parity,
        }
        if not args.no_cpu_baseline and world == 1:
            gf, threads, passes, med = cpu_baseline(m, x)
            line["cpu_baseline"] = {"value": gf, "unit": "GFLOP/s", "cores": threads, "kind": "port",
                                    "sample": f"{passes} full SpMV passes of this matrix (median {med * 1e3:.2f} ms), OpenMP row-parallel CSR loop"}
        print(json.dumps(line))
    del hx, hy
    release(keep)
    if dist:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="timed steps (default: 5 for c5, where a step is 100 SpMVs; 200 otherwise)")
    ap.add_argument("--warmup", type=int, default=None, help="untimed warm-up steps (default 3; at least 3 are always run)")
    ap.add_argument("--workload", default="c5", choices=sorted(k for k in WORKLOADS if "_" not in k) + ["c5"])
    ap.add_argument("--scale", type=int, default=26, help="c5: R-MAT scale (2^scale rows)")
    ap.add_argument("--iters", type=int, default=100, help="c5: repeated SpMVs per step (y -> x)")
    ap.add_argument("--chunks", type=int, default=0, help="c5: row chunks per rank (0: with the multicast store pass one per 1/(2N) of all rows the rank owns, at most 8; 1 with the publishing kernels; 2 with the NCCL forms)")
    ap.add_argument("--exchange", default="multicast", choices=["multicast", "publish", "allgather", "a2a"],
                    help="c5: how a rank's slice of the next x reaches the others: from inside the SpMV kernel (publish), by a multicast store pass per "
                         "chunk, or by NCCL (both multicast modes fall back to allgather where symmetric memory has no multicast address)")
    ap.add_argument("--relabel", default="indegree", choices=["indegree", "none"], help="c5: renumber the vertices by column count, hottest first, and run the loop on "
                    "P A P^T (x permuted on the way in, the result on the way out, inside every step): the hot part of x becomes contiguous")
    ap.add_argument("--host-chunks", type=int, default=0, help="c2 / c4: row chunks of the pipelined host-to-host call (0: default)")
    ap.add_argument("--loop", default="native", choices=["native", "python"], help="c5: who enqueues the repeated SpMVs: the native loop behind the C ABI "
                    "(asp_dist_spmv_iter; multicast exchange and single GPU) or the Python one (every exchange form)")
    ap.add_argument("--balance", default="auto", help="c5: what the row blocks of the ranks have equal amounts of: nnz, bytes (a row weighs one non-zero), "
                    "a number w (a row with non-zeros weighs w non-zeros), or auto (w = 3 + 1.5 log2(N / 2): 3 at 2 GPUs, 4.5 at 4, 6 at 8: the more ranks, the "
                    "larger the share of the exchange that the rank with the sparse tail carries, and the more slack it needs; measured: 8 GPUs 0.55 ms per SpMV with 6 against 0.65 with 4, "
                    "4 GPUs 1.03 with 5 against 1.08 with 8: the rank that owns the sparse tail also has the large exchange and must not be the slowest)")
    ap.add_argument("--tlb", type=int, default=0, help="c5: non-zeros per thread of the CSR5-like format (default 32)")
    ap.add_argument("--sort", default="auto", choices=["auto", "yes", "no"], help="c5: put the rows without non-zeros last (a one-bin coarse sort) so that the format drops them (auto = yes); "
                    "no = every row is stored, unpermuted, which lets the publishing kernels send 16-byte multicast stores (measured slower)")
    ap.add_argument("--cap-log2", type=int, default=0, help="CSR5-like plans: log2 of the rows per warp that go through shared memory (0: chosen at plan creation)")
    ap.add_argument("--generic-csr5", action="store_true", help="CSR5-like plans: the kernel that takes the TLB size at run time instead of the specialised one (comparison runs)")
    ap.add_argument("--stage", action="store_true", help="CSR5-like plans: row sums of a warp through shared memory, contiguous write-out")
    ap.add_argument("--search", action="store_true", help="c5: run the quick search instead of the default one-kernel graph")
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--full-search", action="store_true", help="sweep the full node-parameter and launch grids (slow)")
    ap.add_argument("--dense", default="dense compress", help="with --spec: dense-view nodes, '|'-separated")
    ap.add_argument("--spec", default=None, help="run exactly this compressed-view graph (name from the candidate list)")
    ap.add_argument("--threads", type=int, default=0, help="with --spec: thread_num_in_block")
    ap.add_argument("--graph", default=None, help="skip the search: a bench JSON line file (its config.graph is used) or the graph JSON itself")
    ap.add_argument("--committed", action="store_true", help="single-GPU workloads: replay the committed graph instead of searching")
    ap.add_argument("--configs", default="c1,c2,c2_reference_operators,c3,c4,c4_reference_operators", help="c5 at N = 1: single-GPU configurations to attach to the line")
    ap.add_argument("--no-configs", action="store_true")
    ap.add_argument("--configs-budget-s", type=float, default=600.0, help="no further sub-configuration is started once the run has taken this long")
    ap.add_argument("--profile-launches", type=int, default=0, help="for ncu captures: build the plan, run this many SpMVs and exit (no timing, one short JSON line)")
    ap.add_argument("--profile-specs", default=None, help="with --profile-launches: comma-separated graph names (candidate table) to run one after the other over the workload's matrix")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args()
    if args.host_chunks > 0:
        global HOST_CHUNKS
        HOST_CHUNKS = args.host_chunks
    if args.steps is None:
        args.steps = 5 if args.workload == "c5" else 200
    if args.warmup is None:
        args.warmup = 3

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    # the CPU legs (oracle checks, cpu_baseline) and the OpenMP host operators; the ranks of a node share its cores
    use_all_host_cores(int(os.environ.get("LOCAL_WORLD_SIZE", str(world))))

    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_

        dist = dist_
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    if args.workload == "c5":
        run_c5(args, rank, world, local_rank, dist)
    else:
        run_one_config(args, rank, world, local_rank, dist)


if __name__ == "__main__":
    main()
