"""Python wrappers of the fused compress and decode+update kernels."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np
import torch

from . import lib as L

FLAG_BYTES = 256  # 2 parities x 16 ranks x 8 bytes


@dataclass
class ExchangeRegionView:
    """Addresses inside one rank's receive region: ``[256 B of arrival flags][2 parities x
    world slots]``. ``base`` is that region's address as seen from the calling process
    (a local allocation or a peer mapping)."""
    base: int
    world: int
    slot_capacity: int

    def slot(self, parity: int, src: int) -> int:
        return self.base + FLAG_BYTES + (parity * self.world + src) * self.slot_capacity

    def flag(self, parity: int, src: int) -> int:
        return self.base + (parity * L.MAX_PEERS + src) * 8

    @staticmethod
    def region_bytes(world: int, slot_capacity: int) -> int:
        return FLAG_BYTES + 2 * world * slot_capacity


def read_status(status: torch.Tensor, reset: bool = True) -> int:
    """Reads (synchronising) and optionally clears a kernel status word."""
    v = int(status.item()) & 0xFFFFFFFF
    if v and reset:
        status.zero_()
    return v


class GpuCompressor:
    """Owns the scratch memory of the fused compress kernel for gradients of up to
    ``n_max`` non-zeros (sparse kind) or ``dim`` coordinates (dense kind)."""

    def __init__(self, dim: int, n_max: int, bin_num: int = 256, group_num: int = 8, row_num: int = 2,
                 col_ratio: float = 0.3, seed: int = 0, device="cuda", fused: bool = True, grid: int = 0,
                 budget_s: float = 1.0, key_encoder: str = "delta_binary", cell_bits: int = -1,
                 quantile_summary: str = "sample"):
        if bin_num > L.GPU_MAX_BINS:
            raise ValueError(f"the GPU compressor supports at most {L.GPU_MAX_BINS} buckets")
        self.lib = L.lib()
        self.dim, self.n_max = int(dim), int(max(n_max, 1))
        self.bin_num, self.group_num, self.row_num, self.col_ratio = bin_num, group_num, row_num, float(col_ratio)
        self.seed, self.fused, self.grid, self.budget_s = seed, fused, grid, budget_s
        if key_encoder not in ("delta_binary", "delta_adaptive"):
            raise ValueError(f"Unrecognizable key encoder: {key_encoder}")
        self.key_encoder = 1 if key_encoder == "delta_adaptive" else 0
        if cell_bits not in (-1, 0, 8, 16):
            raise ValueError("cell_bits: -1 (8/16-bit codes by bucket count) or 0 (Huffman-coded tables)")
        self.cell_bits = 0 if cell_bits == 0 else -1
        if quantile_summary not in ("sample", "sketch"):
            raise ValueError("quantile_summary: 'sample' (split points from a shared 4096-value sample) or 'sketch' "
                             "(mergeable k = 128 summaries)")
        self.quantile_summary = 1 if quantile_summary == "sketch" else 0
        self.device = torch.device(device)
        ws_n = max(self.n_max, 1)
        self.ws_bytes = int(self.lib.skml_compress_workspace_bytes(ws_n, bin_num, group_num, row_num, self.col_ratio, 0))
        self.workspace = torch.zeros(self.ws_bytes, dtype=torch.uint8, device=self.device)
        # the dense kind (one code per coordinate) is only reachable when nnz can exceed 2/3 dim
        self.dense_possible = self.n_max * 3 > self.dim * 2
        self.capacity = int(self.lib.skml_payload_capacity(self.n_max, self.dim if self.dense_possible else 0, bin_num,
                                                           group_num, row_num, self.col_ratio))

    def reset(self) -> None:
        """Clears barrier words, counters and publication marks (needed only after a kernel reported an error)."""
        self.workspace.zero_()

    def _args(self, keys, vals, meta, step, rank, world, payload_ptr, slot_capacity, peer_payload, peer_flag,
              status, loss_partials, given) -> L.CompressArgs:
        a = L.CompressArgs()
        a.keys, a.vals, a.meta = L.ptr(keys), L.ptr(vals), L.ptr(meta)
        a.n_max, a.dim = self.n_max, self.dim
        a.bin_num, a.group_num, a.row_num, a.col_ratio = self.bin_num, self.group_num, self.row_num, self.col_ratio
        a.seed, a.step, a.rank, a.world = self.seed, step, rank, world
        a.loss_partials = L.ptr(loss_partials)
        a.payload, a.slot_capacity = payload_ptr, slot_capacity
        for r in range(world):
            a.peer_payload[r] = peer_payload[r]
            a.peer_flag[r] = peer_flag[r]
        a.workspace, a.workspace_bytes = L.ptr(self.workspace), self.ws_bytes
        a.status = L.ptr(status)
        a.budget_cycles = L.budget_cycles(self.budget_s)
        if given is not None:
            splits, mn, mx = given
            a.given_splits, a.n_given, a.given_min, a.given_max = L.ptr(splits), splits.numel(), float(mn), float(mx)
        a.fused, a.grid, a.key_encoder, a.cell_bits = int(self.fused), self.grid, self.key_encoder, self.cell_bits
        a.quantile_summary = self.quantile_summary
        return a

    def make_args(self, *a, **k) -> L.CompressArgs:
        return self._args(*a, **k)

    def compress(self, keys: Optional[torch.Tensor], vals: torch.Tensor, meta: torch.Tensor, step: int, rank: int,
                 world: int, payload_ptr: int, slot_capacity: int, peer_payload: Sequence[int],
                 peer_flag: Sequence[Optional[int]], status: torch.Tensor, loss_partials: Optional[torch.Tensor] = None,
                 dense_vals: Optional[torch.Tensor] = None, given=None) -> None:
        """Launches the sparse-kind kernel (acts iff meta[1] is 0 or 1) and, when ``dense_vals``
        is given, the dense-kind kernel (acts iff meta[1] == 2)."""
        a = self._args(keys, vals, meta, step, rank, world, payload_ptr, slot_capacity, peer_payload, peer_flag,
                       status, loss_partials, given)
        L.check(self.lib.skml_compress_sparse(C.byref(a), L.stream()), "skml_compress_sparse")
        L.count_launches(1 if self.fused else 8)
        if dense_vals is not None:
            a.vals = L.ptr(dense_vals)
            L.check(self.lib.skml_compress_dense(C.byref(a), L.stream()), "skml_compress_dense")
            L.count_launches(1 if self.fused else 4)

    def compress_local(self, keys: torch.Tensor, vals: torch.Tensor, step: int = 0, rank: int = 0, world: int = 1,
                       dense: bool = False, given=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Single-GPU convenience: compresses into a fresh (or given) byte buffer and returns it."""
        n = vals.numel()
        meta = torch.tensor([n, 2 if dense else (1 if n else 0), 0, 0], dtype=torch.int64, device=self.device)
        buf = out if out is not None else torch.zeros(self.capacity, dtype=torch.uint8, device=self.device)
        status = torch.zeros(1, dtype=torch.int32, device=self.device)
        ptrs = [None] * world
        ptrs[rank] = buf.data_ptr()
        flags = [None] * world
        if dense:
            a = self._args(None, vals, meta, step, rank, world, buf.data_ptr(), buf.numel(), ptrs, flags, status, None, given)
            L.check(self.lib.skml_compress_dense(C.byref(a), L.stream()), "skml_compress_dense")
        else:
            a = self._args(keys, vals, meta, step, rank, world, buf.data_ptr(), buf.numel(), ptrs, flags, status, None, given)
            L.check(self.lib.skml_compress_sparse(C.byref(a), L.stream()), "skml_compress_sparse")
        st = read_status(status)
        if st:
            self.reset()
            from ..parallel.failure import check_status
            check_status(st, "in the compress kernel")
        return buf

    def last_splits(self):
        """The distinct split points the last launch used (float32 numpy array, ascending): the
        q - 1 queried order statistics with duplicates dropped, read back from the workspace
        (synchronises). Not meaningful after a launch that was given its splits."""
        off = int(self.lib.skml_compress_splits_offset(self.n_max, self.bin_num, self.group_num, self.row_num,
                                                       self.col_ratio, self.grid))
        raw = self.workspace[off:off + 4 * (self.bin_num - 1)].cpu().numpy().view(np.uint32)
        bits = np.where(raw & np.uint32(0x80000000), raw & np.uint32(0x7FFFFFFF), ~raw).astype(np.uint32)
        v = bits.view(np.float32)
        keep = np.ones(len(v), dtype=bool)
        keep[1:] = v[1:] != v[:-1]
        return v[keep]

    @staticmethod
    def payload_bytes(buf: torch.Tensor) -> bytes:
        head = buf[:256].cpu().numpy().tobytes()
        total = int(np.frombuffer(head, dtype=np.uint64, count=1, offset=144)[0])
        return buf[:total].cpu().numpy().tobytes()


class GpuDecoder:
    """Owns the scratch memory of the fused decode + aggregate + update kernel."""

    def __init__(self, dim: int, key_capacity: int, device="cuda", fused: bool = True, grid: int = 0,
                 budget_s: float = 1.0, max_groups: int = 32, table_capacity: int = 0):
        """``table_capacity``: bytes of scratch for the sketch tables of payloads that carry them
        Huffman-coded (they are expanded to bucket codes before the keys are decoded); 0 = two bytes per
        decoded key."""
        self.lib = L.lib()
        self.max_groups = int(max_groups)
        self.dim, self.key_capacity = int(dim), int(max(key_capacity, 1))
        self.device = torch.device(device)
        self.fused, self.grid, self.budget_s = fused, grid, budget_s
        self.acc = torch.zeros(self.dim, dtype=torch.int64, device=self.device)
        self.key_scratch = torch.zeros(self.key_capacity, dtype=torch.int32, device=self.device)
        self.val_scratch = torch.zeros(self.key_capacity, dtype=torch.float32, device=self.device)
        self.workspace = torch.zeros(256, dtype=torch.uint8, device=self.device)
        self.table_capacity = int(table_capacity) if table_capacity > 0 else 2 * self.key_capacity + 4096
        self.table_scratch = torch.zeros(self.table_capacity, dtype=torch.uint8, device=self.device)
        self.norm_track = None  # (sum of w^2, where lambda * ||w|| goes, lambda): see track_norm

    def track_norm(self, sumsq: torch.Tensor, reg_out: torch.Tensor, lam: float) -> None:
        """From now on every update keeps ``sumsq`` (device double, the caller seeds it with the model's sum
        of squares) current and leaves ``lam * sqrt(sumsq)`` in ``reg_out`` (device double) at its end."""
        self.norm_track = (sumsq, reg_out, float(lam))

    def reset(self) -> None:
        self.workspace.zero_()
        self.acc.zero_()

    def make_args(self, payload_ptrs: Sequence[int], flag_ptrs: Sequence[Optional[int]], slot_capacity: int,
                  step: int, status: torch.Tensor, w: Optional[torch.Tensor] = None, lr: float = 0.0,
                  adam_m: Optional[torch.Tensor] = None, adam_v: Optional[torch.Tensor] = None,
                  adam_scale: float = 1.0, loss_out: Optional[torch.Tensor] = None,
                  out_sum: Optional[torch.Tensor] = None) -> L.DecodeArgs:
        a = L.DecodeArgs()
        world = len(payload_ptrs)
        for r in range(world):
            a.payload[r] = payload_ptrs[r]
            a.flag[r] = flag_ptrs[r]
        a.world, a.slot_capacity, a.step, a.dim = world, slot_capacity, step, self.dim
        a.w, a.adam_m, a.adam_v = L.ptr(w), L.ptr(adam_m), L.ptr(adam_v)
        a.lr, a.adam_scale = float(lr), float(adam_scale)
        if adam_m is not None and adam_v is not None:
            from .glm import moment_stride
            a.adam_stride = moment_stride(adam_m, adam_v)
        a.acc, a.key_scratch, a.key_capacity = L.ptr(self.acc), L.ptr(self.key_scratch), self.key_capacity
        a.loss_out, a.out_sum = L.ptr(loss_out), L.ptr(out_sum)
        a.workspace, a.status = L.ptr(self.workspace), L.ptr(status)
        a.budget_cycles = L.budget_cycles(self.budget_s)
        a.fused, a.grid, a.max_groups = int(self.fused), self.grid, self.max_groups
        a.val_scratch = L.ptr(self.val_scratch)
        a.table_scratch, a.table_capacity = L.ptr(self.table_scratch), self.table_capacity
        if self.norm_track is not None and w is not None:
            a.weight_sumsq, a.reg_out, a.reg_lambda = L.ptr(self.norm_track[0]), L.ptr(self.norm_track[1]), self.norm_track[2]
        return a

    def decode_update(self, payload_ptrs: Sequence[int], flag_ptrs: Sequence[Optional[int]], slot_capacity: int,
                      step: int, status: torch.Tensor, w: Optional[torch.Tensor] = None, lr: float = 0.0,
                      adam_m: Optional[torch.Tensor] = None, adam_v: Optional[torch.Tensor] = None,
                      adam_scale: float = 1.0, loss_out: Optional[torch.Tensor] = None,
                      out_sum: Optional[torch.Tensor] = None) -> None:
        a = self.make_args(payload_ptrs, flag_ptrs, slot_capacity, step, status, w, lr, adam_m, adam_v, adam_scale,
                           loss_out, out_sum)
        world = len(payload_ptrs)
        L.check(self.lib.skml_decode_update(C.byref(a), L.stream()), "skml_decode_update")
        L.count_launches(1 if self.fused else (2 if adam_v is not None else (world + 1 if world > 1 else 1)))

    def decode_sum(self, payloads: List[torch.Tensor], step: int = 0) -> torch.Tensor:
        """Single-GPU convenience: decodes the given payload buffers (one per rank, rank order)
        and returns the dense fp32 mean over ranks (accumulated into a zeroed buffer)."""
        out = torch.zeros(self.dim, dtype=torch.float32, device=self.device)
        status = torch.zeros(1, dtype=torch.int32, device=self.device)
        cap = min(p.numel() for p in payloads)
        self.decode_update([p.data_ptr() for p in payloads], [None] * len(payloads), cap, step, status, out_sum=out)
        st = read_status(status)
        if st:
            self.reset()
            from ..parallel.failure import check_status
            check_status(st, "in the decode kernel")
        return out
