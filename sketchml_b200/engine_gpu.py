"""Device engine of the training driver: every per-step phase is a kernel launch on the
rank's B200 and nothing in the step synchronises with the host.

Step = gradient kernel (margin + coefficient + scatter) -> compaction -> fused compress +
publish into all peers' receive slots -> fused decode + aggregate + update. Loss partials
travel inside the payload headers and are summed by the decode kernel into a per-step ring
that the host reads once per epoch. The uncompressed NCCL baselines (``compressor=None``:
dense all-reduce; ``compressor=Float``: raw key/value all-gather) share the gradient and
compaction kernels.

Reference: ml/algorithm/GeneralizedLinearModel.scala:116-177 (the same phases, run as Spark
actions with a driver round-trip each).
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from . import config as C
from .data import SyntheticSpec
from .ops import lib as L
from .ops.codec import GpuCompressor, GpuDecoder, read_status
from .ops.datagen import generate_gpu
from .ops.glm import (DeviceCSR, GlmState, compact_gradient, glm_grad, glm_validate, update_dense, update_gathered,
                      update_sparse)
from .parallel.failure import check_status


class _BatchHandle:
    def __init__(self, rows: int, index: int):
        self.rows, self.index = rows, index


class GpuEngine:
    name = "gpu"

    def __init__(self, trainer):
        self.t = trainer
        self.conf = trainer.conf
        self.device = trainer.device
        L.lib()  # fail now if the CUDA library is missing
        self.csr: Optional[DeviceCSR] = None
        self.valid_csr: Optional[DeviceCSR] = None
        self.read_index = 0
        self.last_payload_bytes = 0
        self.last_raw_nnz = 0
        self.mode = {C.COMPRESSOR_SKETCH: "sketch", C.COMPRESSOR_NONE: "nccl_dense", C.COMPRESSOR_FLOAT: "nccl_kv",
                     C.COMPRESSOR_FIXED_POINT: "nccl_kv", C.COMPRESSOR_ZIP: "nccl_kv"}.get(self.conf.compressor)
        # FixedPoint / Zip: values are quantized on the device (ops/baseline_quant.py), keys travel raw
        self.value_quant = self.conf.compressor if self.conf.compressor in (C.COMPRESSOR_FIXED_POINT, C.COMPRESSOR_ZIP) else None
        if self.mode is None:
            raise ValueError(f"Unrecognizable gradient compressor: {self.conf.compressor}")
        if self.conf.dtype != "float32":
            raise ValueError("the GPU engine computes in float32")

    # ------------------------------------------------------------------ data
    def generate(self, spec: SyntheticSpec, lo: int, rows: int):
        csr, w = generate_gpu(spec, lo, rows, self.device)
        return csr.to_matrix(), w

    def attach_data(self) -> None:
        t, conf = self.t, self.conf
        self.csr = DeviceCSR(t.train_data.matrix, self.device)
        self.valid_csr = DeviceCSR(t.valid_data.matrix, self.device) if t.valid_data.size else None
        self._setup_buffers()

    def attach_device_csr(self, csr: DeviceCSR, valid: Optional[DeviceCSR] = None) -> None:
        """Used by benchmarks: adopt an existing device shard without a host round trip."""
        self.csr, self.valid_csr = csr, valid
        self._setup_buffers()

    def _setup_buffers(self) -> None:
        conf, comm = self.conf, self.t.comm
        dim = conf.feature_num
        self.batch_rows = int(self.csr.rows * conf.batch_sample_ratio)
        bound = min(dim, max(1, self.batch_rows * max(1, self.csr.max_row_nnz)))
        # every rank must size its slots alike: take the maximum over ranks
        if comm.world > 1:
            tt = torch.tensor([bound], dtype=torch.int64, device=self.device)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            bound = int(tt.item())
        self.n_max = bound
        allow_dense = bound > dim * 2 // 3
        if allow_dense and self.mode == "nccl_kv":
            self.mode = "nccl_dense"  # near-dense gradients: the raw key/value list is no smaller
        self.st = GlmState.create(dim, bound, self.device, allow_dense)
        self.loss_ring = torch.zeros((max(conf.batch_num, 1), 4), dtype=torch.float64, device=self.device)
        self.partials_template = torch.tensor([float(self.batch_rows), 0.0, 0.0, 0.0], dtype=torch.float64,
                                              device=self.device)
        self.batch_index = 0
        self._template_rows = self.batch_rows
        m = self.t.model
        self.reg_every_step = bool(conf.extras.get("reg_loss_every_step", dim <= (1 << 22)))
        self.adam = conf.optimizer == "adam"
        if self.adam and conf.extras.get("packed_adam_state", True):
            # both moments (and, in the fused decode kernel, the per-coordinate sum of the ranks' values) of a
            # coordinate in one 16-byte quad: a lazy Adam step touches one memory sector of state per
            # coordinate instead of three
            opt = m.optimizer
            quad = torch.zeros((dim, 4), dtype=torch.float32, device=self.device)
            quad[:, 0].copy_(opt.m)
            quad[:, 1].copy_(opt.v)
            self.adam_quad = quad
            opt.m, opt.v = quad[:, 0], quad[:, 1]
        # regularisation loss lambda * ||w||_2 of every batch: one launch of a norm kernel per step for the
        # baseline arms; the sketch arm's decode kernel keeps the sum of squares current as it updates, so
        # its steps pass over the model only once per epoch (to shed the rounding of the running sum)
        self.wsq = torch.zeros(1, dtype=torch.float64, device=self.device)
        self.norm_scratch = torch.zeros(int(L.lib().skml_weight_norm_scratch_bytes()) // 8, dtype=torch.float64,
                                        device=self.device)
        self._norm_seeded = False
        if self.mode == "sketch":
            # extras["exchange_sms"]: SMs the two cooperative kernels take (default: all). With pipeline_depth=1
            # the rest is left to the next batch's gradient kernels on their own stream.
            xsms = int(conf.extras.get("exchange_sms", 0) or 0)
            self.comp = GpuCompressor(dim, bound, conf.quant_bin_num, conf.sketch_group_num, conf.sketch_row_num,
                                      conf.sketch_col_ratio, conf.seed, self.device, grid=xsms,
                                      fused=bool(conf.extras.get("fused", True)), budget_s=conf.step_timeout_s,
                                      key_encoder=conf.key_encoder, cell_bits=0 if conf.cell_bits == 0 else -1,
                                      quantile_summary=str(conf.extras.get("quantile_summary", "sample")))
            self.dec = GpuDecoder(dim, bound * comm.world, self.device, fused=bool(conf.extras.get("fused", True)), grid=3 * xsms,
                                  budget_s=conf.step_timeout_s, max_groups=conf.sketch_group_num,
                                  table_capacity=self._table_scratch_bytes(conf, bound, comm.world))
            if self.reg_every_step and m.loss.is_l2_reg and conf.extras.get("track_norm", True):
                self.dec.track_norm(self.wsq, self.partials_template[2:3], m.loss.lam)
            from .parallel.exchange import PeerExchange
            self.xchg = PeerExchange(comm, self.comp.capacity, self.device)
            self._prepare_fast_step()
            self.depth = int(conf.pipeline_depth)
            if self.depth == 1:
                # gradient one step stale: batch t+1 is differentiated on its own stream while step t
                # is still being compressed, exchanged and applied; the sparse-gradient buffers are doubled
                self.sts = [self.st, GlmState.create(dim, bound, self.device, allow_dense)]
                self.stream_g = torch.cuda.Stream(device=self.device)
                self.ev_grad = [torch.cuda.Event(), torch.cuda.Event()]
                self.ev_applied = [torch.cuda.Event(), torch.cuda.Event()]
                for e in self.ev_applied:
                    e.record()
        elif self.mode == "nccl_kv":
            self.kv_keys = torch.zeros((comm.world, bound), dtype=torch.int32, device=self.device)
            self.kv_vals = torch.zeros((comm.world, bound), dtype=torch.float32, device=self.device)
            self.kv_counts = torch.zeros(comm.world, dtype=torch.int64, device=self.device)
            self.kv_acc = torch.zeros(dim, dtype=torch.float32, device=self.device)
            self.fp_codec = self.zip_codec = None
            if self.value_quant == C.COMPRESSOR_FIXED_POINT:
                from .ops.baseline_quant import FixedPointCodec
                self.fp_codec = FixedPointCodec(bound, conf.fixed_point_bit_num, comm.world, self.device)
            elif self.value_quant == C.COMPRESSOR_ZIP:
                from .ops.baseline_quant import ZipCodec
                self.zip_codec = ZipCodec(bound, conf.quant_bin_num, comm.world, self.device)
        else:
            self.dense_sum = torch.zeros(dim, dtype=torch.float32, device=self.device)
        # the prepared gradient path serves every arm alike (the uncompressed baselines too)
        self.depth = int(conf.pipeline_depth) if self.mode == "sketch" else 0
        self._build_transposed_index()

    def _prepare_fast_step(self) -> None:
        """Argument blocks of the single-call step (`skml_train_step`), one per slot parity."""
        import ctypes as CT
        m, st, comm, conf = self.t.model, self.st, self.t.comm, self.conf
        opt = m.optimizer
        am, av = (opt.m, opt.v) if self.adam else (None, None)
        self._ca, self._da = [], []
        for par in (0, 1):
            sp, sf = self.xchg.send_ptrs(par)
            rp, rf = self.xchg.recv_ptrs(par)
            self._ca.append(self.comp.make_args(st.keys, st.vals, st.meta, 0, comm.rank, comm.world, sp[comm.rank],
                                                self.xchg.slot_capacity, sp, sf, st.status, st.partials, None))
            self._da.append(self.dec.make_args(rp, rf, self.xchg.slot_capacity, 0, st.status, m.weights, 0.0, am, av,
                                               1.0, None))
        a = L.StepArgs()
        a.w, a.g, a.bitmap = L.ptr(m.weights), L.ptr(st.g), L.ptr(st.bitmap)
        a.loss_id, a.hot = m.loss.loss_id, int(min(conf.hot_columns, st.dim) // 32 * 32)
        a.partials, a.partials_template, a.status = L.ptr(st.partials), L.ptr(self.partials_template), L.ptr(st.status)
        a.budget_cycles = L.budget_cycles(conf.step_timeout_s)
        a.lam = m.loss.get_reg_param() if m.loss.is_l2_reg else 0.0
        a.block_counts, a.meta, a.keys, a.gvals = L.ptr(st.block_counts), L.ptr(st.meta), L.ptr(st.keys), L.ptr(st.vals)
        a.dense_vals, a.n_max, a.dim = L.ptr(st.dense_vals), st.n_max, st.dim
        self._sa = a
        self._step_fn = L.lib().skml_train_step
        self._byref = CT.byref
        import ctypes
        self._ca_ptr = [ctypes.pointer(x) for x in self._ca]
        self._da_ptr = [ctypes.pointer(x) for x in self._da]
        self._pending = None

    def _build_transposed_index(self) -> None:
        """Column-major index of every minibatch, when the batches are fixed row slices (shard size a
        multiple of the batch size) and the index fits beside the data."""
        from .ops.transposed import build_batch_index
        import time
        self.tindex = None
        self.index_build_s, self.index_bytes = 0.0, 0   # what the one-time preparation cost (reported by the benchmarks)
        conf, csr, B = self.conf, self.csr, self.batch_rows
        if not conf.extras.get("transposed_index", True) or self.depth != 0 or B <= 0 or csr.rows % B != 0:
            return
        need = csr.nnz * (8 if csr.values is not None else 4) * 1.1 + 16 * B * max(1, csr.max_row_nnz)
        free, _ = torch.cuda.mem_get_info(self.device)
        if need > 0.8 * free:
            return
        idx = []
        torch.cuda.synchronize(self.device)
        t0 = time.perf_counter()
        # extras["tiled_index"]: the row-tiled form (a row tile's coefficients in shared memory, no atomics at all,
        # strictly bit-reproducible). Off by default: measured on the headline batch it is slower (partial sums
        # 176 us + combine 92 us against 103 us), because the frequent columns, which hold most entries, already
        # gather near-sequential coefficients in the per-column form, and a 192 KB tile allows one block per SM.
        tiled = bool(conf.extras.get("tiled_index", False))
        for b in range(csr.rows // B):
            bi = build_batch_index(csr, b * B, (b + 1) * B, tiled=tiled)
            if bi.n_cols > self.st.dim * 2 // 3 or bi.n_cols > self.st.n_max:
                return  # near-dense gradients take the dense kind: keep the scatter path
            idx.append(bi)
        if tiled:
            # one scratch for the partial sums of all batches (a step uses one batch's index at a time)
            shared = torch.zeros(max([bi.tiled.n_pairs for bi in idx if bi.tiled is not None] + [1]), dtype=torch.float32,
                                 device=self.device)
            for bi in idx:
                if bi.tiled is not None:
                    bi.tiled.partial = shared
        torch.cuda.synchronize(self.device)
        self.index_build_s, self.index_bytes = time.perf_counter() - t0, sum(bi.nbytes() for bi in idx)
        self.tindex = idx
        self.coef = torch.zeros((B + 3) // 4 * 4, dtype=torch.float32, device=self.device)

    def _launch_fast_step(self, step: int, lr: float, adam_scale: float, ring_ptr: int) -> None:
        csr, segs, rows, done_event = self._pending
        self._pending = None
        a = self._sa
        a.grad_done_event = done_event.cuda_event if done_event is not None else None
        a.rowptr, a.cols, a.vals, a.labels = L.ptr(csr.rowptr), L.ptr(csr.cols), L.ptr(csr.values), L.ptr(csr.labels)
        a.nnz_padded, a.avg_nnz = csr.nnz_padded, float(csr.avg_nnz)
        for i in range(2):
            lo, hi = segs[i] if i < len(segs) else (0, 0)
            a.seg_lo[i], a.seg_cnt[i] = lo, hi - lo
        a.inv_batch = 1.0 / max(1, rows)
        bi = self._index_of(csr, segs)
        if bi is not None and bi.tiled is not None:
            tp = bi.tiled
            a.t_colptr, a.t_vals, a.t_ucols, a.t_cols = None, L.ptr(bi.svals), L.ptr(bi.ucols), bi.n_cols
            a.t_long_col, a.t_long = None, 0
            a.tt_tile_pair_ptr, a.tt_pair_ptr, a.tt_lrow = L.ptr(tp.tile_pair_ptr), L.ptr(tp.pair_ptr), L.ptr(tp.lrow)
            a.tt_pair_dst, a.tt_col_pair_ptr, a.tt_partial = L.ptr(tp.pair_dst), L.ptr(tp.col_pair_ptr), L.ptr(tp.partial)
            a.tt_tiles, a.tt_tile_rows, a.tt_rows = tp.n_tiles, tp.tile_rows, bi.rows
            a.t_meta, a.coef = L.ptr(bi.meta), L.ptr(self.coef)
        elif bi is not None:
            a.tt_pair_ptr = None
            a.t_colptr, a.t_rowidx, a.t_vals, a.t_ucols = L.ptr(bi.colptr), L.ptr(bi.rowidx), L.ptr(bi.svals), L.ptr(bi.ucols)
            a.t_bins, a.t_long_col, a.t_long_e0, a.t_long_e1 = (L.ptr(bi.bins), L.ptr(bi.long_col), L.ptr(bi.long_e0),
                                                                L.ptr(bi.long_e1))
            a.t_short, a.t_medium, a.t_long, a.t_cols = bi.n_short, bi.n_medium, bi.n_long, bi.n_cols
            a.t_meta, a.coef = L.ptr(bi.meta), L.ptr(self.coef)
        else:
            a.t_colptr = a.tt_pair_ptr = None
        lid = getattr(csr, "lid", None) if bi is None else None
        if lid is not None:
            ucols, n_cols, meta_ptr = lid
            if n_cols > self.st.n_max:
                raise ValueError(f"a local-id batch with {n_cols} distinct columns exceeds the engine's bound {self.st.n_max}")
            if getattr(self, "_wc", None) is None:
                self._wc = torch.zeros(self.st.n_max + 8, dtype=torch.float32, device=self.device)
                self._gc = torch.zeros(self.st.n_max + 8, dtype=torch.float32, device=self.device)
            a.l_ucols, a.l_meta, a.l_ncols, a.wc, a.gc = L.ptr(ucols), meta_ptr, n_cols, L.ptr(self._wc), L.ptr(self._gc)
            from types import SimpleNamespace
            bi = SimpleNamespace(n_cols=n_cols, ucols=ucols, local=True)  # what payload_stats / the shadow check need
        else:
            a.l_ucols = None
        self._last_index = bi
        par = step & 1
        a.compress = self._ca_ptr[par]
        a.decode = self._da_ptr[par]
        a.step, a.lr, a.adam_scale, a.loss_out = step, lr, adam_scale, ring_ptr
        L.check(self._step_fn(self._byref(a), L.stream()), "skml_train_step")
        if lid is not None:
            L.count_launches(len(segs) + 2 + 2)  # gather, gradient segment(s), finalize, compress, decode
        else:
            L.count_launches((3 if bi is not None else len(segs) + 3) + 1 +
                             (1 if self.st.dense_vals is not None and bi is None else 0) + 1)

    # ----------------------------------------------------------------- steps
    def _segments(self, count: int):
        segs, n, left = [], self.csr.rows, count
        while left > 0 and n > 0:
            take = min(left, n - self.read_index)
            segs.append((self.read_index, self.read_index + take))
            self.read_index = (self.read_index + take) % n
            left -= take
        return segs

    def compute_gradient(self, csr: Optional[DeviceCSR] = None, segments=None, batch_rows: Optional[int] = None,
                         done_event=None):
        """``done_event`` (a recorded torch.cuda.Event): where the gradient kernels are launched later, inside the
        single-call step, the event is recorded right after them and ``deferred_release`` is set, so that a
        feeder can reuse the batch's staging buffers no earlier than that."""
        m, st = self.t.model, self.st
        self.deferred_release = False
        csr = csr or self.csr
        rows = self.batch_rows if batch_rows is None else batch_rows
        segs = self._segments(rows) if segments is None else segments
        if self._fast_ok() and len(segs) <= 2:
            if rows != self._template_rows:
                self.partials_template[0] = float(rows)
                self._template_rows = rows
            self._refresh_reg_loss()
            self._pending = (csr, segs, rows, done_event)
            self.deferred_release = done_event is not None
            m.optimizer.advance()
            return _BatchHandle(rows, self.batch_index), None, None
        if getattr(csr, "lid", None) is not None:
            raise NotImplementedError("local-id batches need the fused sketch engine's single-call step")
        if rows != self._template_rows:
            self.partials_template[0] = float(rows)
            self._template_rows = rows
        self._refresh_reg_loss()
        lam = m.loss.get_reg_param() if m.loss.is_l2_reg else 0.0
        if getattr(self, "depth", 0) == 1 and self.mode == "sketch":
            par = self.batch_index & 1
            st = self.sts[par]
            with torch.cuda.stream(self.stream_g):
                # the buffers of this parity were last read by step t-2's compress kernel
                self.stream_g.wait_event(self.ev_applied[par])
                st.partials.copy_(self.partials_template)
                bi = self._index_of(csr, segs)
                if bi is not None:
                    from .ops.transposed import glm_grad_transposed
                    glm_grad_transposed(csr, bi, m.weights, self.coef, st.vals, st.partials, st.status, m.loss.loss_id, lam,
                                        self.conf.step_timeout_s)
                    st.keys[:bi.n_cols].copy_(bi.ucols)
                    st.meta.copy_(bi.meta)
                else:
                    glm_grad(csr, segs, m.weights, st, m.loss.loss_id, rows, self.conf.hot_columns, self.conf.step_timeout_s)
                    compact_gradient(st, m.weights, lam)
                self.ev_grad[par].record()
            m.optimizer.advance()
            return _BatchHandle(rows, self.batch_index), None, None
        st.partials.copy_(self.partials_template)
        bi = self._index_of(csr, segs)
        if bi is not None:
            # prepared batch: coefficients per row, then one gather-sum per distinct column; the keys are the index's
            from .ops.transposed import glm_grad_transposed
            glm_grad_transposed(csr, bi, m.weights, self.coef, st.vals, st.partials, st.status, m.loss.loss_id, lam,
                                self.conf.step_timeout_s)
            st.keys[:bi.n_cols].copy_(bi.ucols)
            st.meta.copy_(bi.meta)
        else:
            glm_grad(csr, segs, m.weights, st, m.loss.loss_id, rows, self.conf.hot_columns, self.conf.step_timeout_s)
            compact_gradient(st, m.weights, lam)
        m.optimizer.advance()
        h = _BatchHandle(rows, self.batch_index)
        return h, None, None

    def _refresh_reg_loss(self, force: bool = False) -> None:
        """Leaves lambda * ||w||_2 (un-squared, ml/objective/Loss.scala:48-53) of the current model in the
        loss template. Models above 4M coordinates skip the per-batch term (`resolve_losses` adds one
        value per epoch) unless ``extras["reg_loss_every_step"]`` asks for it."""
        m = self.t.model
        if not (self.reg_every_step and m.loss.is_l2_reg):
            return
        tracked = self.mode == "sketch" and self.dec.norm_track is not None
        if tracked and self._norm_seeded and not force and self.batch_index % max(self.conf.batch_num, 1):
            return  # the decode kernel of the previous step left the value
        L.check(L.lib().skml_weight_norm(L.ptr(m.weights), m.weights.numel(), float(m.loss.lam), L.ptr(self.wsq),
                                         L.ptr(self.partials_template[2:3]), L.ptr(self.norm_scratch), L.stream()),
                "skml_weight_norm")
        L.count_launches(1)
        self._norm_seeded = True

    @staticmethod
    def _table_scratch_bytes(conf, bound, world):
        """Scratch for the sketch tables of Huffman-coded payloads, expanded to two-byte bucket codes:
        rows x ceil(col_ratio x keys) cells per group, every rank's payload at once."""
        if conf.cell_bits != 0:
            return 0
        cells = conf.sketch_row_num * (conf.sketch_col_ratio * bound + 16 * conf.sketch_group_num)
        return int(2 * world * cells) + 4096

    def _index_of(self, csr, segs):
        """The prepared column index of the batch `segs` of the resident shard, if there is one."""
        if getattr(self, "tindex", None) is None or csr is not self.csr or len(segs) != 1:
            return None
        lo, hi = segs[0]
        if hi - lo != self.batch_rows or lo % self.batch_rows:
            return None
        return self.tindex[lo // self.batch_rows]

    def _fast_ok(self) -> bool:
        return (self.mode == "sketch" and getattr(self, "depth", 0) == 0 and bool(self.conf.extras.get("single_call_step", True)) and
                bool(self.conf.extras.get("fused", True)) and
                not (self.t.injector is not None and self.t.injector.skip_publish_steps))

    def _lr_and_scale(self):
        opt = self.t.model.optimizer
        if self.adam:
            opt.advance_betas()
            return opt.lr_0, opt.step_scale()
        return opt.learning_rate(), 1.0

    def aggregate_and_update(self, step: int, partials) -> None:
        m, st, comm = self.t.model, self.st, self.t.comm
        lr, adam_scale = self._lr_and_scale()
        opt = m.optimizer
        am, av = (opt.m, opt.v) if self.adam else (None, None)
        ring = self.loss_ring[self.batch_index % self.loss_ring.shape[0]]
        if self.mode == "sketch" and getattr(self, "_pending", None) is not None:
            self._launch_fast_step(step, lr, adam_scale, ring.data_ptr())
            if self.conf.extras.get("check_status_every_step", False):
                self.check()
            self._maybe_shadow(step, st, self._last_index)
        elif self.mode == "sketch":
            par = self.batch_index & 1
            if getattr(self, "depth", 0) == 1:
                st = self.sts[par]
                torch.cuda.current_stream().wait_event(self.ev_grad[par])
            send_p, send_f = self.xchg.send_ptrs(step)
            recv_p, recv_f = self.xchg.recv_ptrs(step)
            skip = self.t.injector is not None and step in self.t.injector.skip_publish_steps
            if not skip:
                self.comp.compress(st.keys, st.vals, st.meta, step, comm.rank, comm.world, send_p[comm.rank],
                                   self.xchg.slot_capacity, send_p, send_f, st.status, st.partials, st.dense_vals)
            self.dec.decode_update(recv_p, recv_f, self.xchg.slot_capacity, step, st.status, m.weights, lr, am, av,
                                   adam_scale, ring)
            if getattr(self, "depth", 0) == 1:
                self.ev_applied[par].record()
            if self.conf.extras.get("check_status_every_step", comm.world > 1 and bool(self.t.injector)):
                self.check()
            if not skip:
                self._maybe_shadow(step, st, None)
        if self.mode != "sketch" and self.value_quant:
            self._quantize_values(step)
        if self.mode == "nccl_kv" and (self.fp_codec is not None or self.zip_codec is not None):
            self._exchange_coded(step, lr, am, av, adam_scale, ring)
            self.batch_index += 1
            return
        if self.mode == "sketch":
            pass
        elif self.mode == "nccl_dense":
            # baseline: all-reduce of the dense fp32 gradient, then update of every coordinate
            self._densify()
            if comm.world > 1:
                dist.all_reduce(self.dense_sum)
                dist.all_reduce(st.partials)
            ring.copy_(st.partials)
            update_dense(m.weights, self.dense_sum, 1.0 / comm.world, lr, am, av, adam_scale, sparse_only=True)
        else:
            # baseline: all-gather of raw (key, value) pairs padded to the slot size, local sum
            if comm.world > 1:
                dist.all_gather_into_tensor(self.kv_keys.view(-1), st.keys)
                dist.all_gather_into_tensor(self.kv_vals.view(-1), st.vals)
                dist.all_gather_into_tensor(self.kv_counts, st.meta[:1])
                dist.all_reduce(st.partials)
                L.check(L.lib().skml_scatter_kv(L.ptr(self.kv_acc), L.ptr(self.kv_keys), L.ptr(self.kv_vals),
                                                L.ptr(self.kv_counts), self.n_max, comm.world, L.stream()), "scatter_kv")
                # update and clear on the gathered coordinates only: nothing here is proportional to dim
                update_gathered(m.weights, self.kv_acc, self.kv_keys, self.kv_counts, self.n_max, comm.world,
                                1.0 / comm.world, lr, am, av, adam_scale)
            else:
                update_sparse(m.weights, st.keys, st.vals, st.meta, self.n_max, 1.0, lr, am, av, adam_scale)
            ring.copy_(st.partials)
        self.batch_index += 1

    def _maybe_shadow(self, step: int, st, index) -> None:
        """Debug mode `extras={"shadow_every": k}`: every k-th step this rank's payload is recomputed
        by the CPU oracle from the same keys, values and split points and compared bit for bit
        (synchronises; raises `ShadowMismatch`)."""
        k = int(self.conf.extras.get("shadow_every", 0) or 0)
        if k <= 0 or step % k:
            return
        from .utils.shadow import check_payload
        self.sync()
        self.check()
        if index is not None:
            n, keys, kind = index.n_cols, index.ucols, 1
        else:
            n, keys, kind = int(st.meta[0]), st.keys, int(st.meta[1])
        if kind != 1 or n == 0:
            return
        conf = self.conf
        payload = self.comp.payload_bytes(self.xchg.local_slot(step, self.t.comm.rank))
        check_payload(payload, keys[:n].cpu().numpy(), st.vals[:n].cpu().numpy(), conf.feature_num, self.comp.last_splits(),
                      conf.sketch_group_num, conf.sketch_row_num, conf.sketch_col_ratio, self.comp.seed)
        self.shadow_checks = getattr(self, "shadow_checks", 0) + 1

    def _exchange_coded(self, step, lr, am, av, adam_scale, ring) -> None:
        """FixedPoint / Zip baselines: packed codes (plus the norm or the midpoint table) and raw keys are
        what crosses NVLink."""
        st, comm, m = self.st, self.t.comm, self.t.model
        fp, zp = self.fp_codec, self.zip_codec
        if fp is not None:
            fp.pack(st.vals, st.meta[:1], self._fp_seed(step))
            codes, side, all_codes, all_side = fp.codes, fp.norm, getattr(fp, "all_codes", None), getattr(fp, "all_norms", None)
        else:
            zp.pack(st.vals, st.meta[:1])
            codes, side, all_codes, all_side = zp.codes, zp.mids, getattr(zp, "all_codes", None), getattr(zp, "all_mids", None)
        codec = fp if fp is not None else zp
        if comm.world > 1:
            dist.all_gather_into_tensor(self.kv_keys.view(-1), st.keys)
            dist.all_gather_into_tensor(all_codes.view(-1), codes)
            dist.all_gather_into_tensor(self.kv_counts, st.meta[:1])
            dist.all_gather_into_tensor(all_side.view(-1), side)
            dist.all_reduce(st.partials)
            codec.unpack(self.kv_keys, all_codes, all_side, self.kv_counts, comm.world, acc=self.kv_acc)
            update_gathered(m.weights, self.kv_acc, self.kv_keys, self.kv_counts, self.n_max, comm.world,
                            1.0 / comm.world, lr, am, av, adam_scale)
        else:
            codec.unpack(st.keys, codes, side, st.meta[:1], 1, vals_out=st.vals)
            update_sparse(m.weights, st.keys, st.vals, st.meta, self.n_max, 1.0, lr, am, av, adam_scale)
        ring.copy_(st.partials)

    def _fp_seed(self, step: int) -> int:
        return self.conf.seed * 1315423911 + step * 8191 + self.t.comm.rank

    def _quantize_values(self, step: int) -> None:
        """Dense gradient kind (and the dense all-reduce arm) under a value quantizer: the values are
        replaced in place by what the quantizer would decode to."""
        from .ops.baseline_quant import ZipCodec, fixed_point_roundtrip
        st, conf = self.st, self.conf
        targets = []
        if getattr(self, "fp_codec", None) is None and getattr(self, "zip_codec", None) is None:
            targets.append((st.vals, st.meta[0]))   # sparse lists are otherwise coded by the pack kernels
        if st.dense_vals is not None:
            targets.append((st.dense_vals, torch.where(st.meta[1] == 2, st.meta[0] * 0 + st.dim, st.meta[0] * 0)))
        for vals, n in targets:
            if self.value_quant == C.COMPRESSOR_FIXED_POINT:
                fixed_point_roundtrip(vals, n, conf.fixed_point_bit_num,
                                      conf.seed * 1315423911 + step * 8191 + self.t.comm.rank)
            else:
                cache = self.__dict__.setdefault("_zip_roundtrip", {})
                zc = cache.get(vals.numel())
                if zc is None:
                    zc = cache[vals.numel()] = ZipCodec(vals.numel(), conf.quant_bin_num, 1, self.device)
                zc.roundtrip(vals, n.reshape(1))

    def _densify(self) -> None:
        st = self.st
        self.dense_sum.zero_()
        L.check(L.lib().skml_scatter_kv(L.ptr(self.dense_sum), L.ptr(st.keys), L.ptr(st.vals), L.ptr(st.meta), st.n_max,
                                        1, L.stream()), "scatter_kv")
        if st.dense_vals is not None:  # dense kind: the compaction wrote every coordinate instead of a list
            self.dense_sum.copy_(torch.where(st.meta[1] == 2, st.dense_vals, self.dense_sum))

    def after_resume(self) -> None:
        """The weights were replaced from outside (checkpoint): the running sum of squares is stale."""
        self._norm_seeded = False

    def check(self) -> None:
        """Reads the status word (synchronises) and raises on a kernel-reported error."""
        s = read_status(self.st.status)
        if not s and getattr(self, "depth", 0) == 1:
            s = read_status(self.sts[1].status)
        if s:
            if self.mode == "sketch":
                self.comp.reset()
                self.dec.reset()
                if getattr(self, "adam_quad", None) is not None:
                    self.adam_quad[:, 2].zero_()   # the per-coordinate sums of an interrupted lazy-Adam step
            check_status(s, f"at step {self.t.step} on rank {self.t.comm.rank}")

    def resolve_losses(self, handles) -> List[float]:
        """One device->host read per epoch: batch loss = sum obj / sum batch + reg / world."""
        self.check()
        m = self.t.model
        if not self.reg_every_step and m.loss.is_l2_reg:
            self.loss_ring[:, 2] = torch.linalg.vector_norm(m.weights).double() * m.loss.lam * self.t.comm.world
        ring = self.loss_ring.cpu()
        world = self.t.comm.world
        out = []
        for h in handles:
            r = ring[h.index % ring.shape[0]]
            out.append(float(r[1] / max(float(r[0]), 1.0) + r[2] / world))
        return out

    def validate(self):
        m = self.t.model
        if self.valid_csr is None or self.valid_csr.rows == 0:
            return [0.0, 0, 0, 0, 0, 0]
        margins = None
        if self.conf.extras.get("auc"):
            margins = torch.empty(self.valid_csr.rows, dtype=torch.float32, device=self.device)
        acc = glm_validate(self.valid_csr, m.weights, m.loss.loss_id, self.st.status, margins=margins,
                           budget_s=self.conf.step_timeout_s)
        if margins is not None:
            from .utils import rank_sum_auc
            self.last_auc = rank_sum_auc(margins, self.valid_csr.labels)
        return acc.cpu().tolist()

    def payload_stats(self, step: int):
        """(nnz, payload bytes) of this rank's last payload (synchronises)."""
        if self.mode != "sketch":
            n = int(self.st.meta[0])
            return n, 8 * n
        buf = self.xchg.local_slot(step, self.t.comm.rank)
        head = buf[:256].cpu().numpy()
        import numpy as np
        total = int(np.frombuffer(head.tobytes(), dtype=np.uint64, count=1, offset=144)[0])
        nnz = self._last_index.n_cols if getattr(self, "_last_index", None) is not None else int(self.st.meta[0])
        return nnz, total

    def stage_times_us(self):
        """Durations of the stages of this rank's last fused compress and decode launches, from the
        `globaltimer` stamps the kernels leave in their workspaces (synchronises). Compress:
        summary, split query, bucketize + count, scatter + sketch insert, key code, narrow + publish.
        Decode: prepare (including the wait for the peers' payloads), accumulate, claims."""
        if self.mode != "sketch":
            return None
        import numpy as np
        last = (self.t.step - 1) & 1  # the decode kernel keeps the stamps of even and odd steps apart
        c = self.comp.workspace[:256].cpu().numpy().view(np.int64)[8:15]
        kind = 1 if getattr(self, "_last_index", None) is not None else int(self.st.meta[1])  # index batches are sparse
        if kind != 1 or not all(0 <= int(c[i + 1] - c[i]) < 10**9 for i in range(6)):
            return None   # dense-kind or empty step: the sparse compress kernel left no stamps
        dall = self.dec.workspace[:256].cpu().numpy().view(np.int64)
        d, dprev = dall[8 + 4 * last:12 + 4 * last], dall[8 + 4 * (1 - last):12 + 4 * (1 - last)]
        return {"compress": [float(c[i + 1] - c[i]) / 1e3 for i in range(6)],
                "decode": [float(d[i + 1] - d[i]) / 1e3 for i in range(3)],
                # idle time between the end of the compress kernel's last stage and the start of the decode kernel
                "compress_to_decode_gap": float(d[0] - c[6]) / 1e3,
                # from the end of the previous step's decode kernel to the start of this step's compress kernel:
                # the gradient kernels and the launch gaps around them
                "prev_decode_to_compress": float(c[0] - dprev[3]) / 1e3 if dprev[3] else None,
                # how long after block 0 the last block of the decode kernel finished (SGD / plain-Adam modes)
                "decode_last_block_after_block0": float(dall[16 + last] - d[3]) / 1e3 if dall[16 + last] else None}

    def sync(self) -> None:
        torch.cuda.synchronize(self.device)

    def cursor(self) -> int:
        return self.read_index

    def set_cursor(self, c: int) -> None:
        self.read_index = c

    def close(self) -> None:
        if getattr(self, "xchg", None) is not None:
            self.sync()
            self.xchg.close()
