"""The training driver: load -> epochs of (gradient, compressed exchange, update) -> validate.

Reference: ml/algorithm/GeneralizedLinearModel.scala:45-177 (``loadData``, ``train``,
``trainOneEpoch``, ``trainOneIteration``, ``computeGradient``, ``aggregateAndUpdate``,
``validate``) and ml/util/ValidationUtil.scala:12-41. The reference gathers the workers'
compressed gradients at the Spark driver, sums them, compresses the sum a second time and
broadcasts it. Here every rank receives every rank's payload and decodes all of them in
rank order (one lossy step); ``conf.recompress_sum`` restores the second lossy step on the
host engine for parity experiments.

Two engines implement the per-step work behind the same driver:
``HostEngine`` (torch + the C++ oracle + gloo; any machine) and
``sketchml_b200.engine_gpu.GpuEngine`` (sm_100a kernels + peer-memory exchange).
"""
from __future__ import annotations

import math
import os
import pickle
import time
from typing import List, Optional

import numpy as np
import torch

from . import config as C
from .config import MLConf
from .data import CSRMatrix, DataSet, SyntheticSpec, generate_cpu, load_data, shard_rows, split_train_valid
from .gradient import kinds as G
from .models import build_model
from .parallel import FaultInjector, Heartbeat, LocalComm, PayloadError, make_comm, validate_payload
from .utils import (MetricsLogger, PhaseTimer, export_model, get_logger, load_checkpoint, rank_sum_auc, save_checkpoint,
                    weights_hash)

logger = get_logger()


def validation_counts(pre: torch.Tensor, y: torch.Tensor, loss) -> List[float]:
    """(sum loss, TP, TN, FP, FN, n) as in ValidationUtil.scala:21-32."""
    z = pre * y
    pos = pre > 0
    tp = int(((z > 0) & pos).sum())
    tn = int(((z > 0) & ~pos).sum())
    fp = int(((z < 0) & pos).sum())
    fn = int(((z < 0) & ~pos).sum())
    return [float(loss.loss(pre, y).sum()), tp, tn, fp, fn, int(y.numel())]


class HostEngine:
    """Per-step numerics on the host: torch tensors, oracle compressors, byte exchange
    through the host collective layer."""

    name = "host"

    def __init__(self, trainer: "Trainer"):
        self.t = trainer
        self.gradient: G.Gradient = G.ZeroGradient
        self.last_payload_bytes = 0
        self.last_raw_nnz = 0
        self.last_eval = None

    def compute_gradient(self):
        m = self.t.model
        grad, bs, obj, reg = m.optimizer.mini_batch_gradient_descent(m.weights, self.t.train_data, m.loss)
        self.gradient = grad
        return bs, obj, reg

    def _encode(self, g: G.Gradient, step: int, loss_partials) -> bytes:
        conf, comm = self.t.conf, self.t.comm
        comp = G.compress(g, conf, step, comm.rank, comm.world, loss_partials=loss_partials)
        if conf.extras.get("eval_compression") and g.kind is not G.Kind.ZeroGradient:
            self.last_eval = G.evaluate_compression(g, comp)
        if comp.kind is G.Kind.Sketch:
            return b"S" + comp.payload
        return b"P" + pickle.dumps((step, comm.rank, comp))

    def _decode(self, blob: bytes, step: int, src: int) -> G.Gradient:
        if not blob:
            raise PayloadError(f"rank {src} published nothing for step {step}")
        if blob[:1] == b"S":
            validate_payload(blob[1:], expect_step=step, expect_rank=src, expect_dim=self.t.conf.feature_num)
            return G.SketchGradient(None, self.t.conf, payload=blob[1:])
        s, r, comp = pickle.loads(blob[1:])
        if s != step or r != src:
            raise PayloadError(f"stale or misplaced message from rank {src}: step {s}, rank {r}")
        return comp

    def aggregate_and_update(self, step: int, loss_partials):
        t = self.t
        conf, comm = t.conf, t.comm
        g = self.gradient
        self.last_raw_nnz = g.count_nnz() if g.kind is not G.Kind.ZeroGradient else 0
        with t.timer.phase("compress"):
            blob = self._encode(g, step, loss_partials)
        out = t.injector.outgoing(step, blob) if t.injector else blob
        self.last_payload_bytes = len(blob) - 1
        with t.timer.phase("exchange"):
            blobs = comm.all_gather_bytes(out if out is not None else b"")
        with t.timer.phase("decode_sum"):
            grads = [self._decode(b, step, r) for r, b in enumerate(blobs)]
            total = G.sum_gradients(conf.feature_num, grads)
            if conf.recompress_sum and total.kind is not G.Kind.ZeroGradient:
                total = G.compress(total, conf, step, 0, comm.world)
            total.times_by(1.0 / comm.world)
        with t.timer.phase("update"):
            t.model.optimizer.update(total, t.model.weights)

    def validate(self):
        t = self.t
        if t.valid_data is None or t.valid_data.size == 0:
            return [0.0, 0, 0, 0, 0, 0]
        b = t.valid_data.matrix.to("cpu")
        pre = t.model.loss.predict(t.model.weights.double().cpu(), b)
        if t.conf.extras.get("auc"):
            self.last_auc = rank_sum_auc(pre, b.labels)
        return validation_counts(pre, b.labels.double(), t.model.loss)

    def sync(self):
        pass

    def cursor(self) -> int:
        return self.t.train_data.read_index if self.t.train_data else 0

    def set_cursor(self, c: int) -> None:
        self.t.train_data.read_index = c


class Trainer:
    def __init__(self, conf: MLConf, comm=None, injector: Optional[FaultInjector] = None, engine: str = "auto"):
        self.conf = conf
        want_cuda = conf.device == "cuda" or (conf.device == "auto" and torch.cuda.is_available())
        self.device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if want_cuda else torch.device("cpu")
        if want_cuda:
            torch.cuda.set_device(self.device)
        self.comm = comm if comm is not None else make_comm("auto", device=self.device)
        if conf.worker_num != self.comm.world:
            conf.worker_num = self.comm.world  # workers are the ranks of this job
        self.injector = injector
        self.timer = PhaseTimer(use_cuda=want_cuda)
        self.metrics = MetricsLogger(conf.metrics_path or None, self.comm.rank)
        self.heartbeat = Heartbeat(self.comm, timeout_s=float(conf.extras.get("heartbeat_timeout_s", 30.0))) \
            if self.comm.world > 1 and conf.extras.get("heartbeat", True) else None
        self.model = build_model(conf, self.device if want_cuda else "cpu")
        self.train_data: Optional[DataSet] = None
        self.valid_data: Optional[DataSet] = None
        self.w_star = None
        self.step = 0
        self.start_epoch = 0
        self.history = {"train_loss": [], "valid_loss": [], "time_ms": [], "accuracy": []}
        if engine == "auto":
            engine = "gpu" if want_cuda else "host"
        if engine == "gpu":
            from .engine_gpu import GpuEngine
            self.engine = GpuEngine(self)
        else:
            self.engine = HostEngine(self)

    # ------------------------------------------------------------------ data
    def load_data(self, matrix: Optional[CSRMatrix] = None, global_offset: int = 0) -> None:
        """GeneralizedLinearModel.scala:45-76."""
        t0 = time.perf_counter()
        conf, comm = self.conf, self.comm
        dtype = self.model.dtype
        if matrix is None:
            if conf.format == C.FORMAT_SYNTHETIC:
                lo, hi = shard_rows(conf.syn_rows, comm.rank, comm.world)
                spec = SyntheticSpec(conf.syn_rows, conf.feature_num, conf.syn_nnz_per_row, conf.syn_zipf_s,
                                     conf.syn_values, self.model.task, conf.syn_wstar_density, conf.syn_noise,
                                     conf.seed)
                if hasattr(self.engine, "generate"):
                    matrix, self.w_star = self.engine.generate(spec, lo, hi - lo)
                else:
                    matrix, self.w_star = generate_cpu(spec, lo, hi - lo, dtype)
                global_offset = lo
            else:
                matrix, global_offset, _ = load_data(conf.input, conf.format, conf.feature_num, comm.rank,
                                                     comm.world, conf.use_neg_y, dtype)
        train, valid = split_train_valid(matrix, conf.valid_ratio, conf.seed, global_offset)
        self.train_data, self.valid_data = DataSet(train), DataSet(valid)
        counts = comm.all_reduce_sum([train.rows, valid.rows])
        if hasattr(self.engine, "attach_data"):
            self.engine.attach_data()
        if conf.resume:
            self._resume(conf.resume)
        logger.info("Load data cost %.0f ms, %d train data, %d valid data",
                    (time.perf_counter() - t0) * 1e3, int(counts[0]), int(counts[1]))
        self.metrics.log("load", train_rows=int(counts[0]), valid_rows=int(counts[1]),
                         ms=(time.perf_counter() - t0) * 1e3)

    # ----------------------------------------------------------------- train
    def train(self) -> dict:
        """GeneralizedLinearModel.scala:80-102."""
        conf = self.conf
        logger.info("Start to train a %s model on %d worker(s) [%s engine]", self.model.get_name(),
                    self.comm.world, self.engine.name)
        t0 = time.perf_counter()
        batch_num = conf.batch_num
        for epoch in range(self.start_epoch, conf.epoch_num):
            loss = self.train_one_epoch(epoch, batch_num)
            v = self.validate(epoch)
            self.history["train_loss"].append(loss)
            self.history["valid_loss"].append(v["valid_loss"])
            self.history["accuracy"].append(v["precision"])
            self.history["time_ms"].append((time.perf_counter() - t0) * 1e3)
            if conf.checkpoint_every and conf.checkpoint_dir and (epoch + 1) % conf.checkpoint_every == 0:
                self.checkpoint(os.path.join(conf.checkpoint_dir, f"epoch_{epoch + 1:04d}.ckpt"), epoch + 1)
        logger.info("Train loss: [%s]", ", ".join(f"{x:.6f}" for x in self.history["train_loss"]))
        logger.info("Valid loss: [%s]", ", ".join(f"{x:.6f}" for x in self.history["valid_loss"]))
        logger.info("Time: [%s]", ", ".join(f"{x:.0f}" for x in self.history["time_ms"]))
        if conf.export_path and self.comm.rank == 0:
            self.engine.sync()
            export_model(conf.export_path, self.model.weights, self.model.get_name())
        self.metrics.log("phases", **{k: v["total_ms"] for k, v in self.timer.summary().items()})
        return self.history

    def train_one_epoch(self, epoch: int, batch_num: int) -> float:
        t0 = time.perf_counter()
        rows0 = self.rows_seen = getattr(self, "rows_seen", 0)
        losses = []
        for batch in range(batch_num):
            losses.append(self.train_one_iteration(epoch, batch))
        losses = self.engine.resolve_losses(losses) if hasattr(self.engine, "resolve_losses") else losses
        loss = float(np.mean(losses)) if losses else float("nan")
        dt = time.perf_counter() - t0
        sps = (self.rows_seen - rows0) / dt if dt > 0 else 0.0
        logger.info("Epoch[%d] train cost %.0f ms, loss=%.6f, %.0f samples/s", epoch, dt * 1e3, loss, sps)
        self.metrics.log("epoch", epoch=epoch, train_loss=loss, ms=dt * 1e3, samples_per_s=sps)
        return loss

    def train_one_iteration(self, epoch: int, batch: int):
        if self.injector:
            self.injector.between_steps(self.step)
        if self.heartbeat:
            self.heartbeat.beat(self.step)
            self.heartbeat.check(self.step)
        try:
            batch_loss, partials = self.compute_gradient(epoch, batch)
            self.aggregate_and_update(epoch, batch, partials)
        except Exception as e:
            if self.heartbeat:
                self.heartbeat.mark_failed(f"{type(e).__name__}: {e}"[:200])
            raise
        self.step += 1
        return batch_loss

    def train_streamed(self, feeder, steps: int, first: int = 0, loss_host: Optional[torch.Tensor] = None):
        """Runs ``steps`` iterations on minibatches that live in pinned host memory: every step
        copies its batch host->device (overlapped with the previous step through the feeder's
        side stream) and copies the step's loss partials device->host into ``loss_host``
        (pinned, shape [steps, 4]). Returns ``loss_host``; synchronise before reading it."""
        eng = self.engine
        if not hasattr(eng, "attach_device_csr"):
            raise NotImplementedError("train_streamed feeds device staging buffers: it needs the GPU engine (device='cuda')")
        if loss_host is None:
            loss_host = torch.zeros((steps, 4), dtype=torch.float64).pin_memory()
        feeder.prefetch(first)
        for k in range(steps):
            i = first + k
            if k + 1 < steps:
                feeder.prefetch(i + 1)
            csr, rows = feeder.get(i)
            h, _, _ = eng.compute_gradient(csr=csr, segments=[(0, rows)], batch_rows=rows, done_event=feeder.free[i & 1])
            if not getattr(eng, "deferred_release", False):
                feeder.release(i)  # the gradient kernels are already in the stream
            eng.aggregate_and_update(self.step, None)  # otherwise they are launched here and record the event
            loss_host[k].copy_(eng.loss_ring[h.index % eng.loss_ring.shape[0]], non_blocking=True)
            self.step += 1
        return loss_host

    def compute_gradient(self, epoch: int, batch: int):
        """GeneralizedLinearModel.scala:125-141: batch loss = objLoss/batchSize + regLoss/workerNum."""
        with self.timer.phase("gradient"):
            bs, obj, reg = self.engine.compute_gradient()
        if isinstance(bs, (int, float)):
            tot = self.comm.all_reduce_sum([bs, obj, reg])
            self.rows_seen = getattr(self, "rows_seen", 0) + int(tot[0])
            batch_loss = tot[1] / max(tot[0], 1.0) + tot[2] / self.comm.world
            self.metrics.log("batch", epoch=epoch, batch=batch, batch_size=int(tot[0]), obj_loss=tot[1] / max(tot[0], 1.0),
                             reg_loss=tot[2] / self.comm.world, batch_loss=batch_loss)
            return batch_loss, [float(bs), float(obj), float(reg), 0.0]
        # device engines return handles; the loss is resolved at the end of the epoch
        self.rows_seen = getattr(self, "rows_seen", 0) + int(bs.rows) * self.comm.world
        return bs, None

    def aggregate_and_update(self, epoch: int, batch: int, partials) -> None:
        """GeneralizedLinearModel.scala:143-159."""
        self.engine.aggregate_and_update(self.step, partials)
        eng = self.engine
        if getattr(eng, "last_raw_nnz", 0) and getattr(eng, "last_payload_bytes", 0):
            self.metrics.log("exchange", step=self.step, nnz=eng.last_raw_nnz, payload_bytes=eng.last_payload_bytes,
                             ratio_vs_8B=8.0 * eng.last_raw_nnz / eng.last_payload_bytes,
                             ratio_vs_12B=12.0 * eng.last_raw_nnz / eng.last_payload_bytes,
                             **({"rel_l2": eng.last_eval["rel_l2"], "cosine": eng.last_eval["cosine"]}
                                if getattr(eng, "last_eval", None) else {}))

    def validate(self, epoch: int) -> dict:
        """GeneralizedLinearModel.scala:161-177."""
        t0 = time.perf_counter()
        with self.timer.phase("validate"):
            local = self.engine.validate()
        s = self.comm.all_reduce_sum(local)
        n = max(s[5], 1.0)
        out = {"valid_loss": s[0] / n, "precision": (s[1] + s[2]) / n,
               "true_recall": s[1] / max(s[1] + s[4], 1.0), "false_recall": s[2] / max(s[2] + s[3], 1.0),
               "valid_num": int(s[5])}
        if self.conf.extras.get("auc"):
            # as in the reference (ValidationUtil.scala:43-92) every worker ranks its own validation rows
            out["auc"] = float(getattr(self.engine, "last_auc", float("nan")))
        logger.info("Epoch[%d] validation cost %.0f ms, valid size=%d, loss=%.6f, precision=%.6f, "
                    "trueRecall=%.6f, falseRecall=%.6f", epoch, (time.perf_counter() - t0) * 1e3, out["valid_num"],
                    out["valid_loss"], out["precision"], out["true_recall"], out["false_recall"])
        self.metrics.log("validate", epoch=epoch, **out)
        return out

    # ----------------------------------------------------------- checkpoints
    def checkpoint(self, path: str, epoch: int) -> None:
        self.engine.sync()
        h = weights_hash(self.model.weights)
        h0 = self.comm.broadcast_object(h, 0)
        if h != h0:
            raise RuntimeError(f"replica drift: rank {self.comm.rank} weights differ from rank 0")
        if self.comm.rank == 0:
            save_checkpoint(path, model_state=self.model.state_dict(), conf=self.conf.to_dict(), step=self.step,
                            epoch=epoch, cursor=self.engine.cursor())
        self.comm.barrier()

    def _resume(self, path: str) -> None:
        blob = load_checkpoint(path)
        self.model.load_state_dict(blob["model"])
        self.step, self.start_epoch = int(blob["step"]), int(blob["epoch"])
        self.engine.set_cursor(int(blob["cursor"]))
        if hasattr(self.engine, "after_resume"):
            self.engine.after_resume()
        logger.info("Resumed from %s at epoch %d, step %d", path, self.start_epoch, self.step)

    def close(self) -> None:
        self.metrics.close()
        if hasattr(self.engine, "close"):
            self.engine.close()
