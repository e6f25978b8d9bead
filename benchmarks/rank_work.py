"""Per-rank work of a P-rank step on ONE GPU: compress of one rank's gradient and the fused
decode + update of P payloads, with the kernels' own stage times.

A P-rank step makes every rank compress a gradient of batch/P rows and decode P payloads; this
reproduces that load without P GPUs (the payloads are P local buffers, nothing waits on a peer):

    python benchmarks/rank_work.py --ranks 8            # 62,500 rows per rank of the 50M-feature problem
    python benchmarks/rank_work.py --ranks 8 --adam
    python benchmarks/rank_work.py --ranks 1

Prints one JSON line: median CUDA-event times of the two launches (they include the launch latency of
an idle GPU), the stage times from the kernels' `globaltimer` stamps (compress: summary, split query,
bucketize + count, scatter + sketch insert, key code, narrow + publish; decode: prepare, decode, apply as seen by block 0)
and how long after block 0 the last decode block finished.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import numpy as np
    import torch
    from sketchml_b200.data import SyntheticSpec
    from sketchml_b200.ops import generate_gpu
    from sketchml_b200.ops.codec import GpuCompressor, GpuDecoder
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", type=int, default=8)
    ap.add_argument("--global-batch", type=int, default=500_000)
    ap.add_argument("--dim", type=int, default=50_000_000)
    ap.add_argument("--nnz-per-row", type=int, default=30)
    ap.add_argument("--adam", action="store_true")
    ap.add_argument("--plain-adam-state", action="store_true",
                    help="two plain moment arrays instead of the engine's packed {m, v, sum, -} quads")
    ap.add_argument("--iters", type=int, default=8)
    args = ap.parse_args()
    P, dim = args.ranks, args.dim
    per = args.global_batch // P
    spec = SyntheticSpec(per * P, dim, args.nnz_per_row, 1.1, "binary", "logistic", 0.01, 0.0, 17)
    csr, _ = generate_gpu(spec, 0, per * P, "cuda")
    g = torch.Generator(device="cuda").manual_seed(1)
    keys, vals = [], []
    for r in range(P):
        lo, hi = int(csr.rowptr[r * per]), int(csr.rowptr[(r + 1) * per])
        k = torch.unique(csr.cols[lo:hi]).int()
        keys.append(k)
        vals.append((torch.randn(k.numel(), generator=g, device="cuda") * 1e-3).float())
    nmax = max(k.numel() for k in keys)
    comp = GpuCompressor(dim, nmax, 256, 8, 3, 0.2, seed=17)
    dec = GpuDecoder(dim, nmax * P, max_groups=8)
    bufs = [torch.zeros(comp.capacity, dtype=torch.uint8, device="cuda") for _ in range(P)]
    w = torch.zeros(dim, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    m = v = None
    if args.adam:
        if args.plain_adam_state:
            m, v = torch.zeros(dim, device="cuda"), torch.zeros(dim, device="cuda")
        else:
            quad = torch.zeros((dim, 4), device="cuda")
            m, v = quad[:, 0], quad[:, 1]
    tc, td = [], []
    for it in range(args.iters):
        for r in range(P):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            comp.compress_local(keys[r], vals[r], step=it, rank=r, world=P, out=bufs[r])
            b.record()
            torch.cuda.synchronize()
            if it >= 3:
                tc.append(a.elapsed_time(b))
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        dec.decode_update([x.data_ptr() for x in bufs], [None] * P, comp.capacity, it, status, w, 0.05, m, v, 1.0)
        b.record()
        torch.cuda.synchronize()
        if it >= 3:
            td.append(a.elapsed_time(b))
    if int(status.item()):
        raise SystemExit(f"kernel status {int(status.item()):#x}")
    last = (args.iters - 1) & 1
    cs = comp.workspace[:256].cpu().numpy().view(np.int64)[8:15]
    dall = dec.workspace[:256].cpu().numpy().view(np.int64)
    ds = dall[8 + 4 * last:12 + 4 * last]
    print(json.dumps({
        "ranks": P, "optimizer": "adam" if args.adam else "sgd", "nnz_per_rank": int(keys[0].numel()),
        "compress_launch_ms": float(np.median(tc)), "decode_launch_ms": float(np.median(td)),
        "compress_stages_us": [float(cs[i + 1] - cs[i]) / 1e3 for i in range(6)],
        "decode_stages_us": [float(ds[i + 1] - ds[i]) / 1e3 for i in range(3)],
        "decode_last_block_after_block0_us": float(dall[16 + last] - ds[3]) / 1e3 if dall[16 + last] else None}))


if __name__ == "__main__":
    main()
