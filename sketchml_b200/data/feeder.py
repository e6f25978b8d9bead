"""Host-to-device minibatch feeder: batches live in pinned host memory and are copied into
one of two device staging shards on a side stream while the previous batch is being used.

The reference keeps each worker's rows in executor memory and walks them with a cyclic
cursor (ml/data/DataSet.scala:15-21); this is the same walk for data that does not stay
resident on the GPU."""
from __future__ import annotations

from typing import List, Optional

import torch

from .dataset import CSRMatrix


class PinnedBatch:
    def __init__(self, m: CSRMatrix):
        self.rows, self.nnz, self.dim = m.rows, m.nnz, m.dim
        pad = (m.nnz + 3) // 4 * 4 + 4
        self.rowptr = torch.empty(m.rows + 1, dtype=torch.int64).pin_memory()
        self.rowptr.copy_(m.rowptr - m.rowptr[0])
        self.cols = torch.zeros(pad, dtype=torch.int32).pin_memory()
        self.cols[:m.nnz].copy_(m.cols)
        self.values = None
        if m.values is not None:
            self.values = torch.zeros(pad, dtype=torch.float32).pin_memory()
            self.values[:m.nnz].copy_(m.values)
        self.labels = torch.empty(m.rows, dtype=torch.float32).pin_memory()
        self.labels.copy_(m.labels)

    def h2d_bytes(self) -> int:
        n = self.rowptr.numel() * 8 + self.cols.numel() * 4 + self.labels.numel() * 4
        return n + (self.values.numel() * 4 if self.values is not None else 0)


class HostBatchFeeder:
    """Double-buffered pinned-host -> device pipeline of CSR minibatches."""

    def __init__(self, batches: List[PinnedBatch], device):
        from ..ops.glm import DeviceCSR
        self.batches = batches
        self.device = torch.device(device)
        rows = max(b.rows for b in batches)
        pad = max(b.cols.numel() for b in batches)
        has_vals = batches[0].values is not None
        self.copy_stream = torch.cuda.Stream(device=self.device)
        self.stage = []
        for _ in range(2):
            rp = torch.zeros(rows + 1, dtype=torch.int64, device=self.device)
            cols = torch.zeros(pad, dtype=torch.int32, device=self.device)
            vals = torch.zeros(pad, dtype=torch.float32, device=self.device) if has_vals else None
            lab = torch.zeros(rows, dtype=torch.float32, device=self.device)
            self.stage.append(DeviceCSR.from_parts(rp, cols, vals, lab, batches[0].dim, 0))
        self.ready = [torch.cuda.Event(), torch.cuda.Event()]
        self.free = [torch.cuda.Event(), torch.cuda.Event()]
        for e in self.free:
            e.record()
        avg = sum(b.nnz for b in batches) / max(1, sum(b.rows for b in batches))
        mx = max(int((b.rowptr[1:] - b.rowptr[:-1]).max()) for b in batches)
        for s in self.stage:
            s.avg_nnz, s.max_row_nnz = avg, mx

    def prefetch(self, i: int) -> None:
        b = self.batches[i % len(self.batches)]
        slot = i & 1
        st = self.stage[slot]
        with torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(self.free[slot])
            st.rowptr[:b.rows + 1].copy_(b.rowptr, non_blocking=True)
            st.cols[:b.cols.numel()].copy_(b.cols, non_blocking=True)
            if b.values is not None:
                st.values[:b.values.numel()].copy_(b.values, non_blocking=True)
            st.labels[:b.rows].copy_(b.labels, non_blocking=True)
            self.ready[slot].record()

    def get(self, i: int):
        """The device shard holding batch i (the current stream waits for its copy)."""
        slot = i & 1
        b = self.batches[i % len(self.batches)]
        torch.cuda.current_stream().wait_event(self.ready[slot])
        st = self.stage[slot]
        st.rows, st.nnz = b.rows, b.nnz
        return st, b.rows

    def release(self, i: int) -> None:
        """Call after the kernels reading batch i were launched."""
        self.free[i & 1].record()
