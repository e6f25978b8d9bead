"""Headline benchmark: samples/s of L2 logistic regression with sketch-compressed gradient
exchange on the configuration "50M rows x 50M features, 30 nnz/row, binary values,
Zipf(1.1) columns, batch fraction 0.01, lr 0.05, 256 quantile buckets", rows sharded
evenly over the GPUs of one node (total work per step is fixed: strong scaling).

    python bench.py --gpus N --steps K --warmup W          # this framework
    python bench.py --impl reference ...                    # the reference (a JVM/Spark program)

Prints one JSON line on rank 0. `value` is device-timed (CUDA events, max over ranks) with
the shard resident on the GPU; `e2e.value` runs the same steps through
``Trainer.train_streamed`` with every step's batch copied from pinned host memory and its
loss read back.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

CONFIG_NAME = "L2-LR 50M rows x 50M features, 30 nnz/row, Zipf(1.1), batch 0.01, lr 0.05, q=256"


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--rows", type=int, default=50_000_000)
    p.add_argument("--dim", type=int, default=50_000_000)
    p.add_argument("--nnz-per-row", type=int, default=30)
    p.add_argument("--batch-fraction", type=float, default=0.01)
    p.add_argument("--compressor", default="Sketch", choices=["Sketch", "None", "Float"])
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--unfused", action="store_true")
    p.add_argument("--pipeline-depth", type=int, default=0, choices=[0, 1])
    return p.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons of this rank's GPU during the timed region
    (NVML reads every few milliseconds from a thread; nothing is set or reset)."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.index, self.sm, self.bits, self.mx, self.power = index, [], 0, None, []
        self._stop = threading.Event()
        self.th = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = int(vis.split(",")[self.index]) if vis and vis.replace(",", "").isdigit() else self.index
            self.h = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.mx = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None
            return
        self.th = threading.Thread(target=self._poll, daemon=True)
        self.th.start()

    def _poll(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
                self.bits |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                self.power.append(nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
            except Exception:
                pass
            time.sleep(0.002)

    def stop(self) -> dict:
        if self.th is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable"]}
        self._stop.set()
        self.th.join(timeout=1)
        reasons = sorted(n for b, n in self.REASONS.items() if self.bits & b)
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.mx, "reasons": reasons,
                "samples": len(self.sm), "power_w_max": max(self.power) if self.power else None}


def reference_arm(args):
    # pip answers "Directory is not installable. Neither 'setup.py' nor 'pyproject.toml' found" for the
    # reference tree: it is a Maven project of Java and Scala sources for Spark 2.2, and this image has
    # no JDK, Maven, Scala or Spark.
    print(json.dumps({"impl": "reference", "unavailable":
                      "the reference is a Java/Scala Spark application (Maven build); no JDK, Maven, Scala or Spark "
                      "in this image and it is not pip-installable"}))
    return 0


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)
    import torch
    import torch.distributed as dist
    from sketchml_b200.config import MLConf
    from sketchml_b200.data import HostBatchFeeder, PinnedBatch, SyntheticSpec, shard_rows
    from sketchml_b200.data.dataset import CSRMatrix
    from sketchml_b200.ops import generate_gpu, lib as L
    from sketchml_b200.trainer import Trainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    conf = MLConf(algo="lr", format="synthetic", feature_num=args.dim, worker_num=world, valid_ratio=0.0,
                  epoch_num=1, batch_sample_ratio=args.batch_fraction, learn_rate=0.05, learn_decay=0.9, l2_reg=1e-4,
                  compressor=args.compressor, quant_bin_num=256, sketch_group_num=8, sketch_row_num=3,
                  sketch_col_ratio=0.2, optimizer="sgd", device="cuda", seed=17, syn_rows=args.rows,
                  pipeline_depth=args.pipeline_depth,
                  syn_nnz_per_row=args.nnz_per_row, syn_zipf_s=1.1, syn_wstar_density=0.01,
                  extras={"fused": not args.unfused, "heartbeat": False})
    trainer = Trainer(conf)
    trainer.timer.enabled = False
    comm = trainer.comm
    lo, hi = shard_rows(args.rows, rank, world)
    spec = SyntheticSpec(args.rows, args.dim, args.nnz_per_row, 1.1, "binary", "logistic", 0.01, 0.0, 17)
    t_gen = time.perf_counter()
    csr, _ = generate_gpu(spec, lo, hi - lo, dev)
    torch.cuda.synchronize()
    t_gen = time.perf_counter() - t_gen
    eng = trainer.engine
    from sketchml_b200.data import DataSet
    trainer.train_data = DataSet(CSRMatrix(csr.rowptr[:1], csr.cols[:0], None, csr.labels[:0], args.dim))
    eng.attach_device_csr(csr)
    global_batch = eng.batch_rows * world

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def run_steps(n):
        for _ in range(n):
            trainer.train_one_iteration(0, 0)

    run_steps(args.warmup)
    barrier()
    eng.check()
    sampler = ClockSampler(local)
    sampler.start()
    l0 = L.LAUNCHES[0]
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    a.record()
    t_issue = time.perf_counter()
    run_steps(args.steps)
    t_issue = time.perf_counter() - t_issue  # host time to enqueue the steps (the device runs behind)
    b.record()
    barrier()
    ms = a.elapsed_time(b)
    launches = L.LAUNCHES[0] - l0
    clocks = sampler.stop()
    eng.check()
    nnz, pbytes = eng.payload_stats(trainer.step - 1)
    stages = eng.stage_times_us()
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    value = global_batch * args.steps / (ms / 1e3)
    losses = eng.loss_ring[: min(eng.batch_index, eng.loss_ring.shape[0])].cpu()

    e2e = None
    if not args.no_e2e:
        e2e = run_e2e(args, trainer, csr, dev, world, barrier)

    if rank == 0:
        out = {
            "metric": "training throughput (samples/s), compressed-gradient data-parallel SGD",
            "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "fp32", "data": "synthetic (device-generated, random planted model)",
            "config": {"model": CONFIG_NAME if (args.rows, args.dim) == (50_000_000, 50_000_000) else
                       f"L2-LR {args.rows} rows x {args.dim} features (reduced, not the named config)",
                       "global_batch": global_batch, "seq_len": args.nnz_per_row, "parallelism": f"dp{world}",
                       "compressor": args.compressor, "sketch": "q=256, 8 groups, 3 rows x 0.2 cols, delta-binary keys",
                       "l2_policy": "inputs larger than L2: every step reads a fresh batch slice plus 200 MB of "
                                    "weights and 400 MB of accumulators",
                       "fused": not args.unfused, "pipeline_depth": args.pipeline_depth},
            "clocks": clocks, "gpu_launches": launches,
            "payload": {"nnz_per_rank": nnz, "bytes_per_rank": pbytes,
                        "ratio_vs_8B_per_nnz": 8.0 * nnz / max(pbytes, 1), "ratio_vs_12B_per_nnz": 12.0 * nnz / max(pbytes, 1)},
            "loss_first_last": [float(losses[0, 1] / max(float(losses[0, 0]), 1)),
                                float(losses[-1, 1] / max(float(losses[-1, 0]), 1))] if len(losses) else None,
            "datagen_s": t_gen, "stage_us_last_step_rank0": stages,
            "host_issue_ms_per_step_rank0": 1e3 * t_issue / args.steps,
        }
        if e2e is not None:
            out["e2e"] = e2e
        print(json.dumps(out))
    trainer.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def run_e2e(args, trainer, csr, dev, world, barrier):
    """Same steps through Trainer.train_streamed: batches come from pinned host memory."""
    import torch
    import torch.distributed as dist
    from sketchml_b200.data import HostBatchFeeder, PinnedBatch
    from sketchml_b200.data.dataset import CSRMatrix
    eng = trainer.engine
    B = eng.batch_rows
    k = args.nnz_per_row
    # a ring of pinned host batches, cycled: every step still copies its batch host->device; eight
    # batches (far more than L2 holds) keep the host-side preparation of the ring short
    nb = min(args.steps + args.warmup, max(2, csr.rows // max(B, 1)), 8)
    batches = []
    for i in range(nb):
        lo = (i * B) % max(csr.rows - B + 1, 1)
        m = CSRMatrix(csr.rowptr[lo:lo + B + 1].cpu(), csr.cols[lo * k:(lo + B) * k].cpu(), None,
                      csr.labels[lo:lo + B].cpu(), args.dim)
        batches.append(PinnedBatch(m, local_ids=True))
    feeder = HostBatchFeeder(batches, dev)
    trainer.train_streamed(feeder, args.warmup, first=0)
    barrier()
    loss_host = torch.zeros((args.steps, 4), dtype=torch.float64).pin_memory()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    a.record()
    trainer.train_streamed(feeder, args.steps, first=args.warmup, loss_host=loss_host)
    b.record()
    barrier()
    ms = a.elapsed_time(b)
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    eng.check()
    return {"value": B * world * args.steps / (ms / 1e3), "unit": "samples/s", "ms_per_step": ms / args.steps,
            "h2d_bytes_per_step": batches[0].h2d_bytes(), "d2h_bytes_per_step": 32,
            "input_transport": batches[0].transport(),
            "last_loss": float(loss_host[-1, 1] / max(float(loss_host[-1, 0]), 1.0))}


if __name__ == "__main__":
    sys.exit(main())
