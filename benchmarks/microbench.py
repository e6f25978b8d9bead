"""Compression / collective microbenchmark.

A synthetic sparse fp32 gradient of dimension `--dim` (default 100M) with a non-zero fraction
of 1 % and 10 %, sorted uniform-random keys and Laplace(0, 1e-3) values is exchanged among the
ranks of one node in three ways:

  fused      compress kernel -> peer stores into every rank's slot -> decode + aggregate kernel
  nccl_dense NCCL all-reduce of the dense fp32 gradient
  nccl_kv    NCCL all-gather of the raw (key, value) pairs + local scatter-add

and reports, per (density, bucket count): device time (CUDA events, max over ranks), effective
GB/s of gradient exchanged (8 bytes per non-zero per rank, the fp32 key+value size), payload
bytes, compression ratio against 8 and 12 bytes per non-zero, relative L2 error of the decoded
mean against the exact mean, and the achieved fraction of the roofline (slower of HBM bytes at
the measured copy bandwidth and payload bytes over NVLink at the measured link bandwidth).

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/microbench.py
    python benchmarks/microbench.py --dim 20000000          # one GPU

Prints one JSON line per case on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def make_gradient(dim, nnz, seed, device):
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    # sorted distinct uniform keys: draw with a margin, unique, cut to nnz
    k = torch.randint(0, dim, (int(nnz * 1.15) + 64,), generator=g, device=device, dtype=torch.int64)
    k = torch.unique(k)
    if k.numel() > nnz:
        sel = torch.randperm(k.numel(), generator=g, device=device)[:nnz]
        k = k[sel].sort().values
    u = (torch.rand(k.numel(), generator=g, device=device) - 0.5).clamp(-0.4999999, 0.4999999)
    v = -1e-3 * torch.sign(u) * torch.log1p(-2 * u.abs())      # Laplace(0, 1e-3)
    v = torch.where(v.abs() < 1e-8, torch.full_like(v, 1e-6), v)
    return k.to(torch.int32).contiguous(), v.float().contiguous()


def timed(fn, barrier, warmup, iters, flush):
    import torch
    for _ in range(warmup):
        fn()
    barrier()
    ts = []
    for _ in range(iters):
        flush.fill_(1)
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--dim", type=int, default=100_000_000)
    p.add_argument("--densities", default="0.01,0.1")
    p.add_argument("--bins", default="64,128,256")
    p.add_argument("--rows", type=int, default=3)
    p.add_argument("--col-ratio", type=float, default=0.2)
    p.add_argument("--groups", type=int, default=8)
    p.add_argument("--iters", type=int, default=7)
    p.add_argument("--warmup", type=int, default=3)
    args = p.parse_args(argv)

    import torch
    import torch.distributed as dist
    from sketchml_b200.ops import GpuCompressor, GpuDecoder, lib as L
    from sketchml_b200.ops.codec import read_status
    from sketchml_b200.parallel import make_comm
    from sketchml_b200.parallel.exchange import PeerExchange
    from sketchml_b200.utils.roofline import NVLINK_GBS_MEASURED, load_peaks

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    comm = make_comm("auto", device=dev)
    peaks = load_peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def maxr(x):
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    dim = args.dim
    for dens in [float(x) for x in args.densities.split(",")]:
        nnz = int(dim * dens)
        keys, vals = make_gradient(dim, nnz, 1000 + rank, dev)
        n = keys.numel()
        meta = torch.tensor([n, 1, 0, 0], dtype=torch.int64, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        # exact mean over ranks (reference for the error)
        exact = torch.zeros(dim, dtype=torch.float32, device=dev)
        exact.index_add_(0, keys.long(), vals / world)
        if world > 1:
            dist.all_reduce(exact)
        # ---- baselines ----
        dense = torch.zeros(dim, dtype=torch.float32, device=dev)

        def nccl_dense():
            dense.zero_()
            dense.index_add_(0, keys.long(), vals)
            if world > 1:
                dist.all_reduce(dense)

        kk = torch.zeros((world, n + 1024), dtype=torch.int32, device=dev)
        vv = torch.zeros((world, n + 1024), dtype=torch.float32, device=dev)
        kpad = torch.zeros(n + 1024, dtype=torch.int32, device=dev)
        vpad = torch.zeros(n + 1024, dtype=torch.float32, device=dev)
        kpad[:n], vpad[:n] = keys, vals
        counts = torch.full((world,), n, dtype=torch.int64, device=dev)
        acc = torch.zeros(dim, dtype=torch.float32, device=dev)

        def nccl_kv():
            acc.zero_()
            if world > 1:
                dist.all_gather_into_tensor(kk.view(-1), kpad)
                dist.all_gather_into_tensor(vv.view(-1), vpad)
            else:
                kk[0], vv[0] = kpad, vpad
            L.check(L.lib().skml_scatter_kv(L.ptr(acc), L.ptr(kk), L.ptr(vv), L.ptr(counts), n + 1024, world, L.stream()),
                    "scatter_kv")

        t_dense = maxr(timed(nccl_dense, barrier, args.warmup, args.iters, flush))
        t_kv = maxr(timed(nccl_kv, barrier, args.warmup, args.iters, flush))
        for q in [int(x) for x in args.bins.split(",")]:
            comp = GpuCompressor(dim, n, q, args.groups, args.rows, args.col_ratio, seed=7, device=dev)
            dec = GpuDecoder(dim, n * world + 1024, device=dev)
            xchg = PeerExchange(comm, comp.capacity, dev)
            out = torch.zeros(dim, dtype=torch.float32, device=dev)
            step = [0]

            def fused():
                s = step[0]
                sp, sf = xchg.send_ptrs(s)
                rp, rf = xchg.recv_ptrs(s)
                comp.compress(keys, vals, meta, s, rank, world, sp[rank], xchg.slot_capacity, sp, sf, status)
                dec.decode_update(rp, rf, xchg.slot_capacity, s, status, out_sum=out)
                step[0] += 1

            t_fused = maxr(timed(fused, barrier, args.warmup, args.iters, flush))
            out.zero_()   # the decode adds into `out`: one clean pass for the error figure
            barrier()
            fused()
            barrier()
            st = read_status(status)
            if st:
                raise RuntimeError(f"kernel status 0x{st:x}")
            head = xchg.local_slot(step[0] - 1, rank)[:256].cpu().numpy()
            import numpy as np
            pbytes = int(np.frombuffer(head.tobytes(), dtype=np.uint64, count=1, offset=144)[0])
            err = float(torch.linalg.vector_norm(out - exact) / torch.linalg.vector_norm(exact))
            # roofline: compress reads keys+values (8 B/nnz) and writes the payload; decode reads world
            # payloads and does one 32-byte-sector read-modify-write per key
            hbm = 8 * n + pbytes + world * pbytes + world * n * 64
            link = (world - 1) * pbytes
            t_roof = max(hbm / (peaks["hbm_gbs"] * 1e9), link / (NVLINK_GBS_MEASURED * 1e9))
            xchg.close()
            if rank == 0:
                print(json.dumps({
                    "bench": "compress_exchange", "n_gpus": world, "dim": dim, "nnz_per_rank": n, "density": dens,
                    "bins": q, "groups": args.groups, "rows": args.rows, "col_ratio": args.col_ratio,
                    "fused_ms": t_fused, "nccl_dense_ms": t_dense, "nccl_kv_ms": t_kv,
                    "fused_gradient_GBs": 8e-9 * n * world / (t_fused * 1e-3),
                    "nccl_kv_gradient_GBs": 8e-9 * n * world / (t_kv * 1e-3),
                    "payload_bytes": pbytes, "ratio_vs_8B": 8 * n / pbytes, "ratio_vs_12B": 12 * n / pbytes,
                    "rel_l2_error": err, "speedup_vs_dense": t_dense / t_fused, "speedup_vs_kv": t_kv / t_fused,
                    "roofline_ms": t_roof * 1e3, "roofline_fraction": t_roof * 1e3 / t_fused,
                    "roofline_denominator": f"{peaks['hbm_gbs']} GB/s HBM ({peaks['source']}), {NVLINK_GBS_MEASURED} GB/s link (measured)",
                }), flush=True)
            del comp, dec, xchg, out
        del dense, kk, vv, acc, exact
    comm.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
