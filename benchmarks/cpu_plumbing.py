"""CPU plumbing run: L2 logistic regression over torch-gloo ranks with fp64 gradients,
checked against an uncompressed run.

Configuration (defaults): 100k rows x 100k features, 20 nnz/row, binary values, Zipf(1.1) columns
without replacement per row, labels Bernoulli(sigmoid(x.w*)) with w* ~ N(0,1) on 10 % of the
features, lr 0.1, lambda 1e-4, 10 epochs, batch fraction 0.1, 128 quantile buckets,
MinMaxSketch of 3 rows x 1/5 of nnz columns, delta-binary keys.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/cpu_plumbing.py

Rank 0 prints one JSON line with the per-epoch losses of both runs, samples/s, payload bytes and
compression ratios.
"""
import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    import torch
    from sketchml_b200.config import MLConf
    from sketchml_b200.parallel import make_comm
    from sketchml_b200.trainer import Trainer
    p = argparse.ArgumentParser()
    p.add_argument("--rows", type=int, default=100_000)
    p.add_argument("--dim", type=int, default=100_000)
    p.add_argument("--epochs", type=int, default=10)
    p.add_argument("--optimizer", default="sgd")
    a = p.parse_args()
    torch.set_num_threads(max(1, (os.cpu_count() or 2) // int(os.environ.get("WORLD_SIZE", "1"))))
    comm = make_comm("gloo")
    out = {}
    for comp in ("None", "Sketch"):
        conf = MLConf(algo="lr", format="synthetic", feature_num=a.dim, syn_rows=a.rows, syn_nnz_per_row=20, syn_zipf_s=1.1,
                      syn_wstar_density=0.1, epoch_num=a.epochs, batch_sample_ratio=0.1, learn_rate=0.1, l2_reg=1e-4,
                      valid_ratio=0.1, compressor=comp, quant_bin_num=128, sketch_row_num=3, sketch_col_ratio=0.2,
                      key_encoder="delta_binary", optimizer=a.optimizer, dtype="float64", device="cpu", seed=11,
                      extras={"heartbeat": False})
        t = Trainer(conf, comm=comm)
        t.load_data()
        t0 = time.perf_counter()
        h = t.train()
        dt = time.perf_counter() - t0
        ex = t.metrics.of("exchange")
        out[comp] = {"train_loss": h["train_loss"], "valid_loss": h["valid_loss"], "seconds": dt,
                     "samples_per_s": a.rows * 0.9 * 0.1 * 10 * a.epochs / dt / 1.0,
                     "payload_bytes": ex[-1]["payload_bytes"] if ex else None, "nnz": ex[-1]["nnz"] if ex else None,
                     "ratio_vs_8B": ex[-1]["ratio_vs_8B"] if ex else None, "ratio_vs_12B": ex[-1]["ratio_vs_12B"] if ex else None,
                     "weights_abs_sum": float(t.model.weights.abs().sum())}
        t.close()
    if comm.rank == 0:
        gap = abs(out["Sketch"]["train_loss"][-1] - out["None"]["train_loss"][-1]) / out["None"]["train_loss"][-1]
        print(json.dumps({"bench": "cpu_plumbing", "world": comm.world, "rows": a.rows, "dim": a.dim, "optimizer": a.optimizer,
                          "final_train_gap": gap, **out}))
    comm.close()


if __name__ == "__main__":
    main()
