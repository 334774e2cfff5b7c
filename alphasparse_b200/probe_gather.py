"""Ceiling probe for the x gathers of SpMV: how many random 4-byte (or 8-byte) reads per second of a
vector that fits L2 does one GPU sustain when nothing else is asked of it?

    python -m alphasparse_b200.probe_gather [--n 8388608] [--gathers 46000000] [--dtype f32]

Two measurements: torch.index_select into a preallocated output (4 B of index, one 32-byte sector of
x and 4 B of output per gather), with random and with sorted indices, and the library's gather-only
kernel (asp_probe_gather: eight gathers per thread in flight, nothing stored) swept over launch
shapes. The best figure bounds every SpMV kernel on a matrix with uniformly random columns, whatever
its format: each non-zero costs one such gather, and the L1 hands the L2 about one sector request
per clock and SM.
"""
from __future__ import annotations

import argparse
import json

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--n", type=int, default=8_388_608)
    ap.add_argument("--gathers", type=int, default=46_000_000)
    ap.add_argument("--dtype", default="f32", choices=["f32", "f64"])
    ap.add_argument("--reps", type=int, default=20)
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    dt = torch.float32 if args.dtype == "f32" else torch.float64
    g = torch.Generator(device=dev)
    g.manual_seed(2)
    x = torch.rand(args.n, generator=g, device=dev, dtype=dt)
    idx = torch.randint(0, args.n, (args.gathers,), generator=g, device=dev, dtype=torch.int64).to(torch.int32)
    out = torch.empty(args.gathers, device=dev, dtype=dt)
    idx_sorted = torch.sort(idx).values  # the same gathers with perfect locality, for contrast
    res = {}
    for name, ind in (("random", idx), ("sorted", idx_sorted)):
        for _ in range(3):
            torch.index_select(x, 0, ind, out=out)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.reps):
            torch.index_select(x, 0, ind, out=out)
        e1.record()
        e1.synchronize()
        us = e0.elapsed_time(e1) / args.reps * 1e3
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        res[name] = {"us": us, "gathers_per_s": args.gathers / (us * 1e-6), "gathers_per_clock_per_sm_at_1965MHz": args.gathers / (us * 1e-6) / sms / 1.965e9}
    # the library's own gather-only kernel (f32), swept over launch shapes
    best = None
    if args.dtype == "f32":
        import ctypes as C

        from . import capi

        L = capi.lib()
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        idx_u = idx.contiguous()
        one = torch.zeros(1, device=dev, dtype=torch.float32)
        torch.cuda.synchronize()
        for threads in (128, 256, 512):
            for per_sm in (4, 8, 16, 32):
                ms = C.c_float()
                capi.check(L.asp_probe_gather(idx_u.data_ptr(), x.data_ptr(), one.data_ptr(), args.gathers, threads, sms * per_sm, args.reps,
                                              torch.cuda.current_stream().cuda_stream, C.byref(ms)))
                rate = args.gathers / (ms.value * 1e-3)
                if best is None or rate > best["gathers_per_s"]:
                    best = {"us": ms.value * 1e3, "gathers_per_s": rate, "gathers_per_clock_per_sm_at_1965MHz": rate / sms / 1.965e9, "threads": threads, "ctas_per_sm": per_sm}
    print(json.dumps({"probe": "gather", "n": args.n, "gathers": args.gathers, "dtype": args.dtype, "torch_index_select": res, "gather_only_kernel_best": best}))


if __name__ == "__main__":
    main()
