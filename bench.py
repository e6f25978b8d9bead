"""Headline benchmark: training throughput (samples/s) of data-parallel minibatch SGD on a sparse
generalized linear model with sketch-compressed gradient exchange, rows sharded evenly over the
GPUs of one node (the total work per step is fixed: strong scaling).

    python bench.py --gpus N --steps K --warmup W                  # this framework, headline configuration
    python bench.py --config svm200m | linreg10m ...               # the other two training configurations
    python bench.py --impl reference ...                            # the reference (a JVM/Spark program)

Prints one JSON line on rank 0.

* ``value``: the fused sketch exchange with the shard resident on the GPU, device-timed (CUDA events,
  max over ranks, median over segments of exactly K steps each; the spread is in ``segments``).
  The one-time preparation it relies on is reported beside it: ``index_build_s`` / ``index_bytes``
  (the transposed batch index) and ``value_without_index`` (the same steps with no prepared index).
* ``vs_baseline``: ``value`` over the throughput of this framework's own uncompressed arm that ships
  raw (key, value) pairs through an NCCL all-gather, measured in the same invocation on the same data;
  the NCCL dense all-reduce arm is in ``baselines`` too. The reference itself publishes no numbers.
* ``e2e``: the same steps through ``Trainer.train_streamed`` with every step's batch copied from pinned
  host memory in plain CSR form (no host-side preparation of any kind) and its loss read back;
  ``e2e.prepacked`` is the variant whose batches were packed into the compact local-id transport form
  when the data set was loaded, with the host time that packing took per batch.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

# The training configurations: data shape, model, step size. Noise values are standard deviations.
CONFIGS = {
    "lr50m": dict(name="L2-LR 50M rows x 50M features, 30 nnz/row, Zipf(1.1), batch 0.01, lr 0.05, q=256",
                  algo="lr", rows=50_000_000, dim=50_000_000, k=30, zipf=1.1, values="binary", task="logistic",
                  wdens=0.01, noise=0.0, batch=0.01, lr=0.05, l2=1e-4, q=256),
    "svm200m": dict(name="Linear SVM 200M rows x 100M features, 30 nnz/row, unit-L2 rows, Zipf(1.2), batch 0.005, "
                         "lambda 1e-5, q=64",
                    algo="svm", rows=200_000_000, dim=100_000_000, k=30, zipf=1.2, values="uniform_l2", task="svm",
                    wdens=0.005, noise=0.1, batch=0.005, lr=0.05, l2=1e-5, q=64),
    "linreg10m": dict(name="Least squares 10M rows x 1M features, 200 nnz/row, N(0,1) values, uniform columns, "
                           "batch 0.05, lr 0.01, q=256 (dense-kind gradients)",
                      algo="linreg", rows=10_000_000, dim=1_000_000, k=200, zipf=0.0, values="normal", task="regression",
                      wdens=1.0, noise=0.316, batch=0.05, lr=0.01, l2=1e-4, q=256),
}


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--config", default="lr50m", choices=list(CONFIGS))
    p.add_argument("--rows", type=int, default=0, help="override the configuration's row count (reduced run)")
    p.add_argument("--dim", type=int, default=0)
    p.add_argument("--nnz-per-row", type=int, default=0)
    p.add_argument("--batch-fraction", type=float, default=0.0)
    p.add_argument("--compressor", default="Sketch", choices=["Sketch", "None", "Float"],
                   help="the arm reported as `value` (the baselines are measured in every run anyway)")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-baselines", action="store_true")
    p.add_argument("--unfused", action="store_true")
    p.add_argument("--pipeline-depth", type=int, default=0, choices=[0, 1])
    p.add_argument("--index-form", default="columns", choices=["tiled", "columns"],
                   help="prepared batch index: plain per-column lists, or row-tiled (coefficient tiles in shared memory, no "
                        "atomics; slower on the named configurations)")
    p.add_argument("--exchange-sms", type=int, default=0,
                   help="SMs given to the cooperative compress / decode kernels (0 = all); with --pipeline-depth 1 the "
                        "rest runs the next batch's gradient")
    p.add_argument("--min-seconds", type=float, default=0.5, help="timed segments are repeated until this much time is covered")
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


class Bench:
    def __init__(self, args):
        import torch
        self.torch = torch
        self.args = args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus and self.world > 1:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={self.world}")
        self.dev = torch.device("cuda", self.local)
        torch.cuda.set_device(self.dev)
        c = dict(CONFIGS[args.config])
        self.reduced = False
        for key, val in (("rows", args.rows), ("dim", args.dim), ("k", args.nnz_per_row), ("batch", args.batch_fraction)):
            if val:
                self.reduced = self.reduced or c[key] != val
                c[key] = val
        self.c = c
        self.comm = None
        self.csr = None

    # -- plumbing --------------------------------------------------------------------------------
    def barrier(self):
        import torch.distributed as dist
        if self.world > 1:
            dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, xs):
        import torch.distributed as dist
        t = self.torch.tensor(list(xs), dtype=self.torch.float64, device=self.dev)
        if self.world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.cpu().tolist()

    def conf(self, compressor, **extras):
        from sketchml_b200.config import MLConf
        c, a = self.c, self.args
        ex = {"fused": not a.unfused, "heartbeat": False}
        if a.exchange_sms:
            ex["exchange_sms"] = a.exchange_sms
        ex["tiled_index"] = a.index_form == "tiled"
        ex.update(extras)
        return MLConf(algo=c["algo"], format="synthetic", feature_num=c["dim"], worker_num=self.world, valid_ratio=0.0,
                      epoch_num=1, batch_sample_ratio=c["batch"], learn_rate=c["lr"], learn_decay=0.9, l2_reg=c["l2"],
                      compressor=compressor, quant_bin_num=c["q"], sketch_group_num=8, sketch_row_num=3,
                      sketch_col_ratio=0.2, optimizer="sgd", device="cuda", seed=17, syn_rows=c["rows"],
                      pipeline_depth=a.pipeline_depth, syn_nnz_per_row=c["k"], syn_zipf_s=c["zipf"],
                      syn_values=c["values"], syn_wstar_density=c["wdens"], syn_noise=c["noise"], extras=ex)

    def make_trainer(self, compressor, **extras):
        from sketchml_b200.data import DataSet
        from sketchml_b200.data.dataset import CSRMatrix
        from sketchml_b200.trainer import Trainer
        t = Trainer(self.conf(compressor, **extras), comm=self.comm)
        self.comm = t.comm
        t.timer.enabled = False
        csr = self.csr
        t.train_data = DataSet(CSRMatrix(csr.rowptr[:1], csr.cols[:0], None, csr.labels[:0], self.c["dim"]))
        t.engine.attach_device_csr(csr)
        return t

    def generate(self):
        from sketchml_b200.data import SyntheticSpec, shard_rows
        from sketchml_b200.ops import generate_gpu
        c = self.c
        lo, hi = shard_rows(c["rows"], self.rank, self.world)
        spec = SyntheticSpec(c["rows"], c["dim"], c["k"], c["zipf"], c["values"], c["task"], c["wdens"], c["noise"], 17)
        t0 = time.perf_counter()
        self.csr, _ = generate_gpu(spec, lo, hi - lo, self.dev)
        self.torch.cuda.synchronize()
        return time.perf_counter() - t0

    # -- timing ----------------------------------------------------------------------------------
    def time_arm(self, trainer, steps, warmup, min_seconds, max_segments=200, sampler=None):
        """Warm-up, then segments of exactly `steps` steps, each bracketed by barrier + synchronize and
        timed with CUDA events; every segment's time is the maximum over ranks."""
        torch = self.torch
        from sketchml_b200.ops import lib as L
        for _ in range(warmup):
            trainer.train_one_iteration(0, 0)
        self.barrier()
        trainer.engine.check()
        if sampler is not None:
            sampler.start()
        times, launches, issue = [], None, None
        n_seg = 1
        s = 0
        while s < n_seg:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            l0 = L.LAUNCHES[0]
            self.barrier()
            a.record()
            t_issue = time.perf_counter()
            for _ in range(steps):
                trainer.train_one_iteration(0, 0)
            t_issue = time.perf_counter() - t_issue
            b.record()
            self.barrier()
            times.append(a.elapsed_time(b))
            if s == 0:
                launches, issue = L.LAUNCHES[0] - l0, t_issue
                first = self.max_over_ranks([times[0]])[0]   # every rank derives the same segment count
                n_seg = int(min(max_segments, max(3, math.ceil(min_seconds * 1e3 / max(first, 1e-3)))))
            s += 1
        clocks = sampler.stop() if sampler is not None else None
        trainer.engine.check()
        times = self.max_over_ranks(times)
        return {"ms_per_step": statistics.median(times) / steps, "segment_ms": times, "launches": launches,
                "host_issue_ms_per_step": 1e3 * issue / steps, "clocks": clocks}

    def run_e2e(self, trainer, steps, warmup, local_ids):
        """Steps through Trainer.train_streamed: batches come from pinned host memory. With
        `local_ids` the batches are packed into the compact transport form first (timed separately)."""
        torch = self.torch
        from sketchml_b200.data import HostBatchFeeder, PinnedBatch
        from sketchml_b200.data.dataset import CSRMatrix
        csr, eng = self.csr, trainer.engine
        B, k = eng.batch_rows, self.c["k"]
        ring = int(min(steps + warmup, max(2, csr.rows // max(B, 1)), 4 if local_ids else 12))
        batches, pack_s = [], 0.0
        for i in range(ring):
            lo = (i * B) % max(csr.rows - B + 1, 1)
            m = CSRMatrix(csr.rowptr[lo:lo + B + 1].cpu(), csr.cols[lo * k:(lo + B) * k].cpu(),
                          None if csr.values is None else csr.values[lo * k:(lo + B) * k].cpu(),
                          csr.labels[lo:lo + B].cpu(), self.c["dim"])
            t0 = time.perf_counter()
            batches.append(PinnedBatch(m, local_ids=local_ids))
            pack_s += time.perf_counter() - t0
        feeder = HostBatchFeeder(batches, self.dev)
        trainer.train_streamed(feeder, warmup, first=0)
        self.barrier()
        loss_host = torch.zeros((steps, 4), dtype=torch.float64).pin_memory()
        times = []
        for seg in range(3):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.barrier()
            a.record()
            trainer.train_streamed(feeder, steps, first=warmup + seg * steps, loss_host=loss_host)
            b.record()
            self.barrier()
            times.append(a.elapsed_time(b))
        times = self.max_over_ranks(times)
        eng.check()
        ms = statistics.median(times)
        out = {"value": B * self.world * steps / (ms / 1e3), "unit": "samples/s", "ms_per_step": ms / steps,
               "segment_ms": times, "h2d_bytes_per_step": batches[0].h2d_bytes(), "d2h_bytes_per_step": 32,
               "input_transport": batches[0].transport(),
               "last_loss": float(loss_host[-1, 1] / max(float(loss_host[-1, 0]), 1.0))}
        if local_ids:
            out["host_pack_ms_per_batch"] = 1e3 * pack_s / ring
            out["note"] = "batches packed on the host before the clock started (data-set load time); not the headline e2e"
        else:
            out["host_work_per_batch"] = "none: the pinned CSR arrays are copied as they are"
        return out


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)
    import torch
    import torch.distributed as dist
    bn = Bench(args)
    c, world, rank = bn.c, bn.world, bn.rank
    from sketchml_b200.parallel import make_comm
    bn.comm = make_comm("auto", device=bn.dev)   # one process group for all arms of this invocation
    t_gen = bn.generate()

    arm = args.compressor
    product = bn.make_trainer(arm)
    eng = product.engine
    global_batch = eng.batch_rows * world
    index_s, index_bytes = getattr(eng, "index_build_s", 0.0), getattr(eng, "index_bytes", 0)
    has_index = getattr(eng, "tindex", None) is not None
    res = bn.time_arm(product, args.steps, args.warmup, args.min_seconds, sampler=ClockSampler(bn.local))
    ms_step = res["ms_per_step"]
    value = global_batch / (ms_step / 1e3)
    nnz, pbytes = eng.payload_stats(product.step - 1)
    stages = eng.stage_times_us()
    losses = eng.loss_ring[: min(eng.batch_index, eng.loss_ring.shape[0])].cpu()
    index_s = bn.max_over_ranks([index_s])[0]

    e2e = None
    if not args.no_e2e and arm == "Sketch":
        e2e = bn.run_e2e(product, args.steps, args.warmup, local_ids=False)
        if c["values"] == "binary":
            e2e["prepacked"] = bn.run_e2e(product, args.steps, args.warmup, local_ids=True)
    product.close()
    del product, eng
    torch.cuda.empty_cache()

    extra = {}
    if has_index:
        t = bn.make_trainer(arm, transposed_index=False)
        r = bn.time_arm(t, args.steps, args.warmup, min(args.min_seconds, 0.2), max_segments=20)
        t.close()
        del t
        torch.cuda.empty_cache()
        ms_plain = r["ms_per_step"]
        batches_per_epoch = max(1, int(round(1.0 / c["batch"])))
        gain_s = (ms_plain - ms_step) * 1e-3 * batches_per_epoch
        extra = {"value_without_index": global_batch / (ms_plain / 1e3), "ms_per_step_without_index": ms_plain,
                 "index_pays_off_after_epochs": (index_s / gain_s) if gain_s > 0 else None}
    baselines = {}
    if not args.no_baselines:
        for name, comp in (("nccl_kv_allgather", "Float"), ("nccl_dense_allreduce", "None")):
            if comp == arm:
                continue
            t = bn.make_trainer(comp)
            r = bn.time_arm(t, args.steps, args.warmup, min(args.min_seconds, 0.2), max_segments=20)
            baselines[name] = {"value": global_batch / (r["ms_per_step"] / 1e3), "ms_per_step": r["ms_per_step"],
                               "mode": t.engine.mode}
            t.close()
            del t
            torch.cuda.empty_cache()
    kv = baselines.get("nccl_kv_allgather")

    if rank == 0:
        seg = res["segment_ms"]
        out = {
            "metric": "training throughput (samples/s), compressed-gradient data-parallel SGD",
            "value": value, "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": (value / kv["value"]) if kv else None,
            "baseline_is": "this framework's uncompressed arm (NCCL all-gather of raw key/value pairs), same invocation, "
                           "same data; the reference publishes no numbers" if kv else None,
            "dtype": "fp32", "data": "synthetic (device-generated, random planted model)",
            "config": {"model": c["name"] if not bn.reduced else
                       f"{c['algo']} {c['rows']} rows x {c['dim']} features, {c['k']} nnz/row (reduced, not the named configuration)",
                       "global_batch": global_batch, "seq_len": c["k"], "parallelism": f"dp{world}",
                       "compressor": arm, "sketch": f"q={c['q']}, 8 groups, 3 rows x 0.2 cols, delta-binary keys",
                       "l2_policy": "inputs larger than L2: every step reads a fresh batch slice (and its prepared "
                                    "column index when `index_bytes` > 0) plus random words of the weight array, "
                                    "together several times the 126 MB of L2",
                       "fused": not args.unfused, "pipeline_depth": args.pipeline_depth,
                       "exchange_sms": args.exchange_sms or "all"},
            "segments": {"count": len(seg), "steps_each": args.steps, "ms_min": min(seg), "ms_median": statistics.median(seg),
                         "ms_max": max(seg)},
            "clocks": res["clocks"], "gpu_launches": res["launches"],
            "compress_cluster_blocks": int(__import__("sketchml_b200.ops.lib", fromlist=["lib"]).lib().skml_compress_cluster_size()),
            "index_build_s": index_s, "index_bytes": index_bytes, **extra,
            "baselines": baselines,
            "payload": {"nnz_per_rank": nnz, "bytes_per_rank": pbytes,
                        "ratio_vs_8B_per_nnz": 8.0 * nnz / max(pbytes, 1), "ratio_vs_12B_per_nnz": 12.0 * nnz / max(pbytes, 1)},
            "loss_first_last": [float(losses[0, 1] / max(float(losses[0, 0]), 1)),
                                float(losses[-1, 1] / max(float(losses[-1, 0]), 1))] if len(losses) else None,
            "datagen_s": t_gen, "stage_us_last_step_rank0": stages,
            "host_issue_ms_per_step_rank0": res["host_issue_ms_per_step"],
        }
        if e2e is not None:
            out["e2e"] = e2e
        print(json.dumps(out))
    if world > 1 and dist.is_initialized():
        dist.barrier()
    bn.comm.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
