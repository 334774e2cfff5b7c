"""Ceiling probe for the x gathers of SpMV: how many random 4-byte (or 8-byte) reads per second of a
vector that fits L2 does one GPU sustain when nothing else is asked of it?

    python -m alphasparse_b200.probe_gather [--n 8388608] [--gathers 46000000] [--dtype f32]

The indices are read coalesced and the gathered values are only summed (torch.index_select followed
by a reduction is avoided: the gather itself is timed with a preallocated output, so the kernel
moves 4 B of index, one 32-byte sector of x and 4 B of output per gather). The figure bounds every
SpMV kernel on a matrix with uniformly random columns, whatever its format: each non-zero costs one
such gather, and the L1 hands the L2 about one sector request per clock and SM.
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
    print(json.dumps({"probe": "gather", "n": args.n, "gathers": args.gathers, "dtype": args.dtype, **res}))


if __name__ == "__main__":
    main()
