"""Time-to-target-loss and final-loss gap of the sketch exchange against the uncompressed raw
key/value exchange, over a sweep of sketch settings (groups x rows x column ratio) and both
optimizers (SGD; lazy Adam, the reference's optimizer: ml/objective/Adam.scala:27-77).

The reference logs train loss, validation loss and cumulative time per epoch at the end of a run
(ml/algorithm/GeneralizedLinearModel.scala:98-101); this prints the same three series per arm plus
  * `gap`: relative gap of the final training loss to the uncompressed run at equal epochs
    (the 1 % bound is judged on this),
  * `time_to_target_ms`: device-inclusive wall time until the validation loss reaches the
    uncompressed run's final validation loss plus `--slack`,
  * `payload_bytes_per_nnz`: what the setting costs on the wire.

    python benchmarks/time_to_loss.py                                  # one GPU
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/time_to_loss.py
"""
from __future__ import annotations

import argparse
import copy
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from convergence import run_arm  # noqa: E402


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--rows", type=int, default=4_000_000)
    p.add_argument("--dim", type=int, default=4_000_000)
    p.add_argument("--nnz-per-row", type=int, default=30)
    p.add_argument("--zipf", type=float, default=1.1)
    p.add_argument("--wstar-density", type=float, default=0.01)
    p.add_argument("--epochs", type=int, default=5)
    p.add_argument("--batch-fraction", type=float, default=0.01)
    p.add_argument("--l2", type=float, default=1e-6)
    p.add_argument("--bins", type=int, default=256)
    p.add_argument("--algo", default="lr")
    p.add_argument("--slack", type=float, default=0.01)
    p.add_argument("--optimizers", default="sgd,adam")
    p.add_argument("--lr-sgd", type=float, default=0.5)
    p.add_argument("--lr-adam", type=float, default=0.01)
    p.add_argument("--settings", default="8x3x0.2,8x2x0.3,8x3x0.5,16x3x0.2,16x3x0.5,32x3x0.2,32x3x0.5",
                   help="comma-separated groups x rows x column-ratio triples")
    args = p.parse_args()
    for opt in args.optimizers.split(","):
        a = copy.copy(args)
        a.optimizer, a.lr = opt, (args.lr_adam if opt == "adam" else args.lr_sgd)
        a.groups, a.sketch_rows, a.col_ratio = 8, 3, 0.2
        base, rank = run_arm(a, "Float", args.algo)
        target = base["valid_loss"][-1] * (1.0 + args.slack)
        rows = [("uncompressed (raw key/value all-gather)", base)]
        for s in args.settings.split(","):
            g, r, c = s.split("x")
            a.groups, a.sketch_rows, a.col_ratio = int(g), int(r), float(c)
            res, _ = run_arm(a, "Sketch", args.algo)
            rows.append((f"sketch {g} groups, {r} rows x {c}", res))
        if rank == 0:
            for name, r in rows:
                reach = next((t for l, t in zip(r["valid_loss"], r["time_ms"]) if l <= target), None)
                print(json.dumps({
                    "optimizer": opt, "arm": name, "world": r["world"], "epochs": args.epochs,
                    "final_train_loss": r["train_loss"][-1], "final_valid_loss": r["valid_loss"][-1],
                    "gap": abs(r["train_loss"][-1] - base["train_loss"][-1]) / abs(base["train_loss"][-1]),
                    "valid_gap": abs(r["valid_loss"][-1] - base["valid_loss"][-1]) / abs(base["valid_loss"][-1]),
                    "target_valid_loss": target, "time_to_target_ms": reach, "total_ms": r["time_ms"][-1],
                    "payload_bytes_per_nnz": r.get("payload_bytes_per_nnz"),
                    "train_loss": r["train_loss"], "valid_loss": r["valid_loss"], "time_ms": r["time_ms"]}))
    import torch.distributed as dist
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
