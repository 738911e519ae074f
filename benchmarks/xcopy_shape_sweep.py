#!/usr/bin/env python
"""Tuning sweep of the bulk-copy kernel's pipeline shape (tile bytes x stages x stores in flight x walk order x CTAs) on one
process: a local HBM→HBM copy, and with --peer a push from GPU 0 into GPU 1 over NVLink. Device-timed with CUDA events, seeded
data, byte-compared once per shape, next to the copy engine on the same buffers. GB = 1e9 B.

    python benchmarks/xcopy_shape_sweep.py [--mib 1024] [--iters 10] [--peer] [--out FILE.json]
"""
from __future__ import annotations

import argparse
import itertools
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import torch

    import memfabric_hybrid_b200 as mf

    ap = argparse.ArgumentParser()
    ap.add_argument("--mib", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--peer", action="store_true")
    ap.add_argument("--out", default="")
    args = ap.parse_args()

    n = args.mib << 20
    torch.cuda.set_device(0)
    src = torch.empty(n, dtype=torch.uint8, device="cuda:0")
    dst = torch.zeros(n, dtype=torch.uint8, device="cuda:1" if args.peer else "cuda:0")
    if args.peer:
        dst.copy_(src)  # makes torch enable peer access
        torch.cuda.synchronize(1)
    s = torch.cuda.current_stream().cuda_stream
    mf.native.fill_pattern(src.data_ptr(), n, 7, s)
    torch.cuda.synchronize()
    sms = torch.cuda.get_device_properties(0).multi_processor_count

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / args.iters

    def same():
        return bool(torch.equal(src, dst.to("cuda:0") if args.peer else dst))

    rows = []
    ce_us = timed(lambda: mf.native.copy_engine(dst.data_ptr(), src.data_ptr(), n, s))
    base_us = timed(lambda: mf.native.xcopy(dst.data_ptr(), src.data_ptr(), n, 0, s))
    for tile_kib, stages, inflight, blocked, per_sm in itertools.product((16, 32, 64), (3, 4, 6, 8), (1, 2, 3), (0, 1), (1, 2)):
        tile = tile_kib << 10
        smem = tile * stages + 128
        if inflight >= stages or smem > 220 << 10 or (per_sm == 2 and smem > 110 << 10):
            continue
        dst.zero_()
        if args.peer:
            torch.cuda.synchronize(1)  # the clearing ran on the other GPU's stream: it must be over before the copy starts
        rc = mf.native.xcopy_shaped(dst.data_ptr(), src.data_ptr(), n, tile, stages, inflight, blocked, sms * per_sm, s)
        torch.cuda.synchronize()
        if rc != 0 or not same():
            rows.append({"tile_kib": tile_kib, "stages": stages, "inflight": inflight, "blocked": blocked, "ctas": sms * per_sm, "error": rc})
            continue
        us = timed(lambda: mf.native.xcopy_shaped(dst.data_ptr(), src.data_ptr(), n, tile, stages, inflight, blocked, sms * per_sm, s))
        rows.append({"tile_kib": tile_kib, "stages": stages, "inflight": inflight, "blocked": blocked, "ctas": sms * per_sm, "us": round(us, 2),
                     "GBps": round(n / us / 1e3, 1)})
    good = sorted((r for r in rows if "us" in r), key=lambda r: r["us"])
    out = {"bytes": n, "peer": args.peer, "copy_engine_us": round(ce_us, 2), "copy_engine_GBps": round(n / ce_us / 1e3, 1),
           "default_shape_us": round(base_us, 2), "default_shape_GBps": round(n / base_us / 1e3, 1), "best": good[:12],
           "worst": good[-3:], "all": good, "errors": [r for r in rows if "error" in r], "shapes_tried": len(rows)}
    text = json.dumps(out, indent=1)
    print(text)
    if args.out:
        with open(args.out, "w") as f:
            f.write(text)


if __name__ == "__main__":
    main()
