"""Random-access ceilings of one GPU, as denominators for the gather / scatter bound kernels.

The gradient, compaction and decode kernels touch one 32-byte sector per non-zero at data
dependent addresses; the STREAM-style copy bandwidth is not their bound. This script measures,
with plain PyTorch ops, how many independent 4-byte gathers and 4-byte atomic adds per second
the device sustains on tables larger than L2 (uniform indices) and prints one JSON line.

    python benchmarks/random_access.py [--table-mb 400] [--n 16000000]
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import torch
    from sketchml_b200.utils.timing import cuda_time_ms
    p = argparse.ArgumentParser()
    p.add_argument("--table-mb", type=int, default=400)
    p.add_argument("--n", type=int, default=16_000_000)
    a = p.parse_args()
    dev = torch.device("cuda")
    elems = a.table_mb * (1 << 20) // 4
    table = torch.zeros(elems, dtype=torch.float32, device=dev)
    idx = torch.randint(0, elems, (a.n,), device=dev, dtype=torch.int64)
    val = torch.ones(a.n, dtype=torch.float32, device=dev)
    out = torch.empty(a.n, dtype=torch.float32, device=dev)
    t_g = cuda_time_ms(lambda: torch.index_select(table, 0, idx, out=out), iters=7)
    t_s = cuda_time_ms(lambda: table.index_add_(0, idx, val), iters=7)
    big = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    big2 = torch.empty_like(big)
    t_c = cuda_time_ms(lambda: big2.copy_(big), iters=7)
    print(json.dumps({"table_mb": a.table_mb, "n": a.n, "gather_ms": t_g, "gathers_per_s": a.n / t_g * 1e3,
                      "atomic_add_ms": t_s, "atomic_adds_per_s": a.n / t_s * 1e3,
                      "gather_sector_GBs": 32e-9 * a.n / t_g * 1e3, "atomic_sector_GBs": 64e-9 * a.n / t_s * 1e3,
                      "copy_GBs": 2 * big.numel() / t_c * 1e-6}))


if __name__ == "__main__":
    main()
