"""Loss-vs-time comparison of the compressed exchange against the uncompressed baselines.

Trains the same synthetic problem for the same number of epochs with
  * the fused sketch exchange (`--compressor Sketch`),
  * the NCCL dense all-reduce baseline (`None`),
  * the NCCL raw key/value all-gather baseline (`Float`),
and prints one JSON line per arm: training / validation loss per epoch, cumulative device time
per epoch, time to reach the target validation loss (the uncompressed run's final loss plus
`--slack`), and the relative gap of the final training loss to the uncompressed run.

    python benchmarks/convergence.py                       # one GPU
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/convergence.py
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def run_arm(args, compressor, algo):
    import torch
    from sketchml_b200.config import MLConf
    from sketchml_b200.trainer import Trainer
    kw = dict(algo=algo, format="synthetic", feature_num=args.dim, syn_rows=args.rows, syn_nnz_per_row=args.nnz_per_row,
              syn_zipf_s=args.zipf, syn_wstar_density=args.wstar_density, epoch_num=args.epochs,
              batch_sample_ratio=args.batch_fraction, learn_rate=args.lr, learn_decay=0.0, l2_reg=args.l2,
              valid_ratio=0.05, compressor=compressor, quant_bin_num=args.bins, sketch_group_num=args.groups,
              sketch_row_num=args.sketch_rows, sketch_col_ratio=args.col_ratio, optimizer=args.optimizer,
              device="cuda", seed=3, extras={"heartbeat": False})
    if algo == "linreg":
        kw.update(syn_values="normal", syn_noise=0.1)
    elif algo == "svm":
        kw.update(syn_values="uniform_l2", syn_noise=0.1)
    t = Trainer(MLConf(**kw))
    t.timer.enabled = False
    t.load_data()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    h = t.train()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    out = {"compressor": compressor, "algo": algo, "world": t.comm.world, "train_loss": h["train_loss"],
           "valid_loss": h["valid_loss"], "time_ms": h["time_ms"], "wall_s": wall, "accuracy": h["accuracy"]}
    if hasattr(t.engine, "payload_stats"):
        nnz, nbytes = t.engine.payload_stats(t.step - 1)
        out["payload_bytes_per_nnz"] = nbytes / max(nnz, 1)
    rank = t.comm.rank
    t.close()
    return out, rank


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--rows", type=int, default=4_000_000)
    p.add_argument("--dim", type=int, default=4_000_000)
    p.add_argument("--nnz-per-row", type=int, default=30)
    p.add_argument("--zipf", type=float, default=1.1)
    p.add_argument("--wstar-density", type=float, default=0.01)
    p.add_argument("--epochs", type=int, default=5)
    p.add_argument("--batch-fraction", type=float, default=0.01)
    p.add_argument("--lr", type=float, default=0.5)
    p.add_argument("--l2", type=float, default=1e-6)
    p.add_argument("--bins", type=int, default=256)
    p.add_argument("--groups", type=int, default=8)
    p.add_argument("--sketch-rows", type=int, default=3)
    p.add_argument("--col-ratio", type=float, default=0.2)
    p.add_argument("--optimizer", default="sgd")
    p.add_argument("--algo", default="lr")
    p.add_argument("--slack", type=float, default=0.01)
    p.add_argument("--arms", default="None,Float,Sketch")
    args = p.parse_args()
    results = {}
    rank = 0
    for arm in args.arms.split(","):
        results[arm], rank = run_arm(args, arm, args.algo)
    if rank == 0:
        base = results.get("None") or next(iter(results.values()))
        target = base["valid_loss"][-1] * (1.0 + args.slack)
        for arm, r in results.items():
            reach = next((t for l, t in zip(r["valid_loss"], r["time_ms"]) if l <= target), None)
            r["target_valid_loss"] = target
            r["time_to_target_ms"] = reach
            r["final_train_gap_vs_uncompressed"] = abs(r["train_loss"][-1] - base["train_loss"][-1]) / abs(base["train_loss"][-1])
            print(json.dumps(r))
    import torch.distributed as dist
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
