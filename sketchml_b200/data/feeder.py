"""Host-to-device minibatch feeder: batches live in pinned host memory and are copied into
one of two device staging shards on a side stream while the previous batch is being used.

The reference keeps each worker's rows in executor memory and walks them with a cyclic
cursor (ml/data/DataSet.scala:15-21); this is the same walk for data that does not stay
resident on the GPU."""
from __future__ import annotations

from typing import List

import torch

from .dataset import CSRMatrix


class PinnedBatch:
    """One minibatch in pinned host memory.

    ``packed=True`` stores the transport form that `skml_unpack_batch*` expands on the device:
    one contiguous buffer ``[row lengths uint8 (or rowptr int32) | labels int8 (or fp32) | meta |
    column indices]`` (sections 16-byte aligned). The column indices take ceil(log2(dim)) bits each, or 1..4 bytes + 2 flag bits
    each, or 1..8 nibbles + 3 flag bits each, whichever is shortest (``transport="bits"`` /
    ``"varbytes"`` / ``"varnibbles"`` forces one). Values (absent for
    binary features) always travel as fp32.

    ``local_ids=True`` (implies ``packed``) additionally replaces every column index by its position
    in the batch's sorted list of distinct columns and ships that list (delta-coded) with the batch.
    The distinct columns are the keys of the batch's sparse gradient, so the device scatters into a
    compact accumulator instead of a ``dim``-sized one and needs no touched-bitmap compaction."""

    def __init__(self, m: CSRMatrix, packed: bool = False, transport: str = None, local_ids: bool = False):
        self.rows, self.nnz, self.dim = m.rows, m.nnz, m.dim
        self.packed = bool(packed) or bool(local_ids)
        self.local_ids = bool(local_ids)
        pad = (m.nnz + 3) // 4 * 4 + 4
        self.pad = pad
        rowptr = (m.rowptr - m.rowptr[0]).to(torch.int64)
        self.max_row_nnz = int((rowptr[1:] - rowptr[:-1]).max()) if m.rows else 0
        self.values = None
        if m.values is not None:
            self.values = torch.zeros(pad, dtype=torch.float32).pin_memory()
            self.values[:m.nnz].copy_(m.values)
        if not self.packed:
            self.rowptr = torch.empty(m.rows + 1, dtype=torch.int64).pin_memory()
            self.rowptr.copy_(rowptr)
            self.cols = torch.zeros(pad, dtype=torch.int32).pin_memory()
            self.cols[:m.nnz].copy_(m.cols)
            self.labels = torch.empty(m.rows, dtype=torch.float32).pin_memory()
            self.labels.copy_(m.labels)
            return
        import numpy as np
        from ..compress import oracle
        if m.nnz >= 2 ** 31:
            raise ValueError("a packed batch holds fewer than 2^31 non-zeros")
        if self.local_ids and m.values is not None:
            raise NotImplementedError("local-id batches reorder the entries of a row: binary features only")
        self.bits = max(1, int(m.dim - 1).bit_length())
        lab = m.labels.to(torch.float32)
        self.labels8 = bool(torch.all(lab == lab.round()) and float(lab.abs().max() if m.rows else 0) <= 127)
        cols_np = m.cols.to(torch.int32).numpy()
        self.n_cols = 0
        ucol_var = None
        if self.local_ids:
            ucols = np.unique(cols_np)  # ascending
            self.n_cols = int(len(ucols))
            cols_np = np.searchsorted(ucols, cols_np).astype(np.int32)
            # inside a row the order of the entries is free: sort them and ship the gaps
            cols_np = oracle.row_sort_delta(rowptr.numpy(), cols_np)
            self.bits = max(1, int(max(self.n_cols - 1, 1)).bit_length())
            ucol_var = oracle.pack_varbytes(np.diff(ucols, prepend=0).astype(np.int32))
        # column indices: fixed width (ceil(log2(dim)) bits each) or byte-aligned variable width (1..4
        # bytes + 2 flag bits each, smaller when frequent features have small indices), whichever is shorter
        var = oracle.pack_varbytes(cols_np)
        fixed_bytes = 4 * ((m.nnz * self.bits + 31) // 32 + 2)
        a16 = lambda x: (x + 15) // 16 * 16
        var_bytes = a16(4 * len(var["flags"])) + a16(4 * len(var["block_offsets"])) + a16(len(var["bytes"]))
        nibv = oracle.pack_varnibbles(cols_np)
        nib_bytes = a16(4 * len(nibv["flags"])) + a16(4 * len(nibv["block_offsets"])) + a16(4 * len(nibv["words"]))
        sizes = {"bits": fixed_bytes, "varbytes": var_bytes, "varnibbles": nib_bytes}
        self.col_form = transport if transport is not None else min(sizes, key=sizes.get)
        if self.col_form not in sizes:
            raise ValueError(f"unknown column transport {self.col_form!r}")
        self.varbytes = self.col_form == "varbytes"
        if self.col_form == "varnibbles":  # same three sections as the byte-aligned form
            var = {"flags": nibv["flags"], "block_offsets": nibv["block_offsets"], "bytes": nibv["words"].view(np.uint8)}
        self.off_rowptr = 0
        self.rowlen8 = self.max_row_nnz <= 255  # row lengths as bytes instead of 32-bit row pointers
        self.off_labels = a16(m.rows if self.rowlen8 else 4 * (m.rows + 1))
        self.off_meta = a16(self.off_labels + (m.rows if self.labels8 else 4 * m.rows))
        self.off_cols = self.off_meta + 32
        if ucol_var is not None:  # [flags | block offsets | bytes] of the distinct-column deltas
            self.off_uflags = self.off_cols
            self.off_ublocks = a16(self.off_uflags + 4 * len(ucol_var["flags"]))
            self.off_ubytes = a16(self.off_ublocks + 4 * len(ucol_var["block_offsets"]))
            self.off_cols = a16(self.off_ubytes + len(ucol_var["bytes"]))

        def put(off, arr):
            raw = torch.from_numpy(np.ascontiguousarray(arr).view(np.uint8))
            self.buffer[off:off + raw.numel()].copy_(raw)

        if self.col_form != "bits":
            self.off_flags = self.off_cols
            self.off_blocks = a16(self.off_flags + 4 * len(var["flags"]))
            self.off_bytes = a16(self.off_blocks + 4 * len(var["block_offsets"]))
            total = a16(self.off_bytes + len(var["bytes"]))
            self.buffer = torch.zeros(total, dtype=torch.uint8).pin_memory()
            put(self.off_flags, var["flags"])
            put(self.off_blocks, var["block_offsets"])
            put(self.off_bytes, var["bytes"])
        else:
            words = oracle.pack_bits(cols_np, self.bits)  # uint32, two padding words included
            total = a16(self.off_cols + 4 * len(words))
            self.buffer = torch.zeros(total, dtype=torch.uint8).pin_memory()
            put(self.off_cols, words)
        put(self.off_meta, np.array([self.n_cols, 1 if self.n_cols else 0, 0, 0], dtype=np.int64))
        if ucol_var is not None:
            put(self.off_uflags, ucol_var["flags"])
            put(self.off_ublocks, ucol_var["block_offsets"])
            put(self.off_ubytes, ucol_var["bytes"])
        put(self.off_rowptr, (rowptr[1:] - rowptr[:-1]).to(torch.uint8).numpy() if self.rowlen8
            else rowptr.to(torch.int32).numpy())
        put(self.off_labels, lab.to(torch.int8).numpy() if self.labels8 else lab.numpy())

    def transport(self) -> str:
        if not self.packed:
            return "rowptr int64, labels fp32, column indices int32"
        cols = {"varbytes": "column indices 1-4 bytes each + 2 flag bits (byte-aligned variable width)",
                "varnibbles": "column indices 1-8 nibbles each + 3 flag bits (nibble-aligned variable width)",
                "bits": f"column indices bit-packed at {self.bits} bits"}[self.col_form]
        what = "batch-local column ids (sorted inside each row, as gaps)" if self.local_ids else "column indices"
        cols = cols.replace("column indices", what)
        extra = ", plus the batch's distinct columns as variable-width deltas" if self.local_ids else ""
        rp = "row lengths uint8" if self.rowlen8 else "rowptr int32"
        return f"{rp}, labels {'int8' if self.labels8 else 'fp32'}, {cols}{extra}, expanded on the device"

    def h2d_bytes(self) -> int:
        extra = self.values.numel() * 4 if self.values is not None else 0
        if self.packed:
            return self.buffer.numel() + extra
        return self.rowptr.numel() * 8 + self.cols.numel() * 4 + self.labels.numel() * 4 + extra


class HostBatchFeeder:
    """Double-buffered pinned-host -> device pipeline of CSR minibatches."""

    def __init__(self, batches: List[PinnedBatch], device):
        from ..ops.glm import DeviceCSR
        self.batches = batches
        self.device = torch.device(device)
        rows = max(b.rows for b in batches)
        pad = max(b.pad for b in batches)
        has_vals = batches[0].values is not None
        self.packed = batches[0].packed
        if any(b.packed != self.packed for b in batches):
            raise ValueError("all batches of a feeder use the same transport form")
        self.copy_stream = torch.cuda.Stream(device=self.device)
        # the expansion kernels run on their own stream, so that the copy engine can start the next
        # batch's transfer while this batch is being expanded
        self.unpack_stream = torch.cuda.Stream(device=self.device)
        self.copied = [torch.cuda.Event(), torch.cuda.Event()]
        self.stage, self.raw = [], []
        for _ in range(2):
            rp = torch.zeros(rows + 1, dtype=torch.int64, device=self.device)
            cols = torch.zeros(pad, dtype=torch.int32, device=self.device)
            vals = torch.zeros(pad, dtype=torch.float32, device=self.device) if has_vals else None
            lab = torch.zeros(rows, dtype=torch.float32, device=self.device)
            self.stage.append(DeviceCSR.from_parts(rp, cols, vals, lab, batches[0].dim, 0))
            if self.packed:
                self.raw.append(torch.zeros(max(b.buffer.numel() for b in batches), dtype=torch.uint8, device=self.device))
        self.local_ids = batches[0].local_ids
        if any(b.local_ids != self.local_ids for b in batches):
            raise ValueError("all batches of a feeder use the same transport form")
        if self.local_ids:
            nc = max(b.n_cols for b in batches) + 8
            self.ucols = [torch.zeros(nc, dtype=torch.int32, device=self.device) for _ in range(2)]
            self.udelta = torch.zeros(nc, dtype=torch.int32, device=self.device)
        self.ready = [torch.cuda.Event(), torch.cuda.Event()]
        self.free = [torch.cuda.Event(), torch.cuda.Event()]
        for e in self.free:
            e.record()
        avg = sum(b.nnz for b in batches) / max(1, sum(b.rows for b in batches))
        mx = max(b.max_row_nnz for b in batches)
        for s in self.stage:
            s.avg_nnz, s.max_row_nnz = avg, mx

    def prefetch(self, i: int) -> None:
        b = self.batches[i % len(self.batches)]
        slot = i & 1
        st = self.stage[slot]
        cs, us = self.copy_stream, self.unpack_stream
        with torch.cuda.stream(cs):
            cs.wait_event(self.free[slot])
            if self.packed:
                raw = self.raw[slot]
                raw[:b.buffer.numel()].copy_(b.buffer, non_blocking=True)
            else:
                st.rowptr[:b.rows + 1].copy_(b.rowptr, non_blocking=True)
                st.cols[:b.cols.numel()].copy_(b.cols, non_blocking=True)
                st.labels[:b.rows].copy_(b.labels, non_blocking=True)
            if b.values is not None:
                st.values[:b.values.numel()].copy_(b.values, non_blocking=True)
            self.copied[slot].record()
        if not self.packed:
            with torch.cuda.stream(cs):
                self.ready[slot].record()
            return
        from ..ops import lib as L
        with torch.cuda.stream(us):
            us.wait_event(self.copied[slot])
            base = raw.data_ptr()
            lab8 = base + b.off_labels if b.labels8 else None
            rp32 = None if b.rowlen8 else base + b.off_rowptr
            if b.rowlen8:  # st.rowptr[0] is and stays 0
                torch.cumsum(raw[b.off_rowptr:b.off_rowptr + b.rows], 0, dtype=torch.int64, out=st.rowptr[1:b.rows + 1])
            if b.col_form != "bits":
                fn = L.lib().skml_unpack_batch_varbytes if b.varbytes else L.lib().skml_unpack_batch_varnibbles
                L.check(fn(base + b.off_flags, base + b.off_blocks, base + b.off_bytes, b.nnz, L.ptr(st.cols), rp32, b.rows,
                           L.ptr(st.rowptr), lab8, L.ptr(st.labels), us.cuda_stream), "skml_unpack_batch_var*")
            else:
                L.check(L.lib().skml_unpack_batch(base + b.off_cols, b.bits, b.nnz, L.ptr(st.cols), rp32,
                                                  b.rows, L.ptr(st.rowptr), lab8, L.ptr(st.labels), us.cuda_stream),
                        "skml_unpack_batch")
            L.count_launches(1)
            if not b.labels8:
                st.labels[:b.rows].copy_(raw[b.off_labels:b.off_labels + 4 * b.rows].view(torch.float32))
            if b.local_ids:
                L.check(L.lib().skml_row_prefix(L.ptr(st.rowptr), b.rows, L.ptr(st.cols), us.cuda_stream), "skml_row_prefix")
                L.count_launches(1)
            if b.local_ids and b.n_cols:
                # the distinct columns: variable-width deltas -> int32 -> running sum
                L.check(L.lib().skml_unpack_batch_varbytes(base + b.off_uflags, base + b.off_ublocks, base + b.off_ubytes,
                                                           b.n_cols, L.ptr(self.udelta), None, 0, None, None, None,
                                                           us.cuda_stream), "skml_unpack_batch_varbytes")
                torch.cumsum(self.udelta[:b.n_cols], 0, dtype=torch.int32, out=self.ucols[slot][:b.n_cols])
                L.count_launches(2)
            self.ready[slot].record()

    def get(self, i: int):
        """The device shard holding batch i (the current stream waits for its copy)."""
        slot = i & 1
        b = self.batches[i % len(self.batches)]
        torch.cuda.current_stream().wait_event(self.ready[slot])
        st = self.stage[slot]
        st.rows, st.nnz = b.rows, b.nnz
        # local-id batch: (distinct columns on the device, their count, device address of {count, kind, 0, 0})
        st.lid = (self.ucols[slot], b.n_cols, self.raw[slot].data_ptr() + b.off_meta) if b.local_ids else None
        return st, b.rows

    def release(self, i: int) -> None:
        """Call after the kernels reading batch i were launched."""
        self.free[i & 1].record()
