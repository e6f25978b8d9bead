"""Column-major (transposed) index of a fixed minibatch, and the gradient that uses it.

When a shard's minibatches are fixed row slices (the cyclic cursor of the reference,
ml/data/DataSet.scala:15-21, with a shard size that is a multiple of the batch size), the set of
columns a batch touches never changes. Its transposed index is built once; a step then computes
the per-row coefficients and gathers them per column, which replaces the scatter into the
dim-sized accumulator, the touched bitmap and the compaction (see csrc/cuda/glm_kernels.cu).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import lib as L
from .glm import DeviceCSR

SHORT_MAX, MEDIUM_MAX, LONG_SEGMENT = 4, 512, 4096


@dataclass
class BatchIndex:
    lo: int
    rows: int
    n_cols: int
    colptr: torch.Tensor      # int32 [n_cols + 1]
    rowidx: torch.Tensor      # int32 [nnz], batch-local rows, column-major
    svals: Optional[torch.Tensor]
    ucols: torch.Tensor       # int32 [n_cols] ascending distinct columns = gradient keys
    bins: torch.Tensor        # int32: positions of short columns, then of medium columns
    long_col: torch.Tensor
    long_e0: torch.Tensor
    long_e1: torch.Tensor
    n_short: int
    n_medium: int
    n_long: int
    meta: torch.Tensor        # int64 [4] = {n_cols, 1, 0, 0}

    def nbytes(self) -> int:
        ts = [self.colptr, self.rowidx, self.ucols, self.bins, self.long_col, self.long_e0, self.long_e1]
        return sum(t.numel() * t.element_size() for t in ts) + (self.svals.numel() * 4 if self.svals is not None else 0)


def build_batch_index(csr: DeviceCSR, lo: int, hi: int) -> BatchIndex:
    dev = csr.cols.device
    e0, e1 = int(csr.rowptr[lo]), int(csr.rowptr[hi])
    cols = csr.cols[e0:e1]
    counts = (csr.rowptr[lo + 1:hi + 1] - csr.rowptr[lo:hi])
    rows = torch.repeat_interleave(torch.arange(hi - lo, device=dev, dtype=torch.int32), counts, output_size=e1 - e0)
    scol, order = torch.sort(cols, stable=True)
    rowidx = rows[order].contiguous()
    svals = None if csr.values is None else csr.values[e0:e1][order].contiguous()
    ucols, cnt = torch.unique_consecutive(scol, return_counts=True)
    n = int(ucols.numel())
    colptr = torch.zeros(n + 1, dtype=torch.int32, device=dev)
    colptr[1:] = torch.cumsum(cnt, 0).to(torch.int32)
    pos = torch.arange(n, device=dev, dtype=torch.int32)
    short = pos[cnt <= SHORT_MAX]
    medium = pos[(cnt > SHORT_MAX) & (cnt <= MEDIUM_MAX)]
    longs = pos[cnt > MEDIUM_MAX]
    nseg = (cnt[longs.long()] + LONG_SEGMENT - 1) // LONG_SEGMENT
    long_col = torch.repeat_interleave(longs, nseg)
    first = torch.cumsum(nseg, 0) - nseg
    seg = torch.arange(int(long_col.numel()), device=dev) - torch.repeat_interleave(first, nseg)
    le0 = colptr[long_col.long()].long() + seg * LONG_SEGMENT
    le1 = torch.minimum(le0 + LONG_SEGMENT, colptr[long_col.long() + 1].long())
    return BatchIndex(lo, hi - lo, n, colptr, rowidx, svals, ucols.to(torch.int32).contiguous(),
                      torch.cat([short, medium]).contiguous(), long_col.to(torch.int32).contiguous(),
                      le0.to(torch.int32).contiguous(), le1.to(torch.int32).contiguous(), int(short.numel()),
                      int(medium.numel()), int(long_col.numel()),
                      torch.tensor([n, 1 if n else 0, 0, 0], dtype=torch.int64, device=dev))


def glm_grad_transposed(csr: DeviceCSR, bi: BatchIndex, w: torch.Tensor, coef: torch.Tensor, out_vals: torch.Tensor,
                        partials: torch.Tensor, status: torch.Tensor, loss_id: int, lam: float,
                        budget_s: float = 1.0) -> None:
    """out_vals[:bi.n_cols] = gradient values (mean over the batch + lam * w) for keys bi.ucols;
    the objective loss sum is added into partials[1]."""
    lib = L.lib()
    L.check(lib.skml_glm_coef(L.ptr(csr.rowptr), L.ptr(csr.cols), L.ptr(csr.values), L.ptr(csr.labels), bi.lo, bi.rows,
                              csr.nnz_padded, float(csr.avg_nnz), L.ptr(w), loss_id, 1.0 / max(1, bi.rows),
                              partials.data_ptr() + 8, L.ptr(coef), L.ptr(status), L.budget_cycles(budget_s), L.stream()),
            "skml_glm_coef")
    L.check(lib.skml_colsum(L.ptr(bi.colptr), L.ptr(bi.rowidx), L.ptr(bi.svals), L.ptr(bi.ucols), L.ptr(bi.bins),
                            L.ptr(bi.long_col), L.ptr(bi.long_e0), L.ptr(bi.long_e1), bi.n_short, bi.n_medium, bi.n_long,
                            bi.n_cols, L.ptr(coef), L.ptr(w), float(lam), L.ptr(out_vals), L.stream()), "skml_colsum")
    L.count_launches(2)
