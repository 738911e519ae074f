#!/usr/bin/env python
"""Mid-size copies (64 KiB - 16 MiB), where neither bandwidth nor launch latency alone decides: the load/store kernel, the
bulk-copy kernel with small tiles and the copy engine side by side, local or (--peer) GPU 0 → GPU 1 in one process.
Back-to-back copies on one stream, device-timed with CUDA events; microseconds per copy.

    python benchmarks/xcopy_mid_sweep.py [--peer] [--iters 50] [--out FILE.json]
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import torch

    import memfabric_hybrid_b200 as mf

    ap = argparse.ArgumentParser()
    ap.add_argument("--peer", action="store_true")
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    top = 16 << 20
    torch.cuda.set_device(0)
    src = torch.empty(top, dtype=torch.uint8, device="cuda:0")
    dst = torch.zeros(top, dtype=torch.uint8, device="cuda:1" if args.peer else "cuda:0")
    if args.peer:
        dst.copy_(src)
        torch.cuda.synchronize(1)
    s = torch.cuda.current_stream().cuda_stream
    mf.native.fill_pattern(src.data_ptr(), top, 3, s)
    torch.cuda.synchronize()
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    n = mf.native

    def timed(fn):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return round(e0.elapsed_time(e1) * 1e3 / args.iters, 2)

    rows = []
    d, a = dst.data_ptr(), src.data_ptr()
    for kib in (64, 128, 256, 512, 1024, 2048, 4096, 8192, 16384):
        nb = kib << 10
        row = {"kib": kib, "copy_engine_us": timed(lambda: n.copy_engine(d, a, nb, s)), "auto_us": timed(lambda: n.xcopy(d, a, nb, 0, s)),
               "ldst_us": timed(lambda: n.xcopy(d, a, nb, -1, s))}
        for tile_kib, stages, inflight in ((8, 4, 1), (16, 4, 1), (16, 8, 3), (32, 4, 2)):
            tiles = max(1, nb // (tile_kib << 10))
            per_sm = 2 if (tile_kib << 10) * stages + 128 <= (110 << 10) else 1
            ctas = min(tiles, sms * per_sm)
            row[f"bulk_{tile_kib}k_{stages}s_{inflight}f_us"] = timed(lambda: n.xcopy_shaped(d, a, nb, tile_kib << 10, stages, inflight, 0, ctas, s))
        dst.zero_()
        if args.peer:
            torch.cuda.synchronize(1)
        n.xcopy(d, a, nb, 0, s)
        torch.cuda.synchronize()
        row["ok"] = bool(torch.equal(src[:nb], dst[:nb].to("cuda:0")))
        rows.append(row)
        print(json.dumps(row), flush=True)
    if args.out:
        with open(args.out, "w") as f:
            json.dump({"peer": args.peer, "rows": rows}, f, indent=1)


if __name__ == "__main__":
    main()
