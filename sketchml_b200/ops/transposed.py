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
TILE_ROWS_MAX = 49152   # coefficients of one row tile in shared memory: 192 KB
PAIR_SEGMENT = 256      # longest entry list behind one partial sum
SEG_SLOTS = 256         # >= TILE_ROWS_MAX / PAIR_SEGMENT segments per (tile, column) pair


@dataclass
class TiledPart:
    """Row-tiled form of the index: entries in (tile, column, row) order with 16-bit tile-local rows, one
    partial sum per (tile, column) pair, the pairs of a column consecutive in (column, tile) order."""
    tile_rows: int
    n_tiles: int
    n_pairs: int
    tile_pair_ptr: torch.Tensor   # int32 [n_tiles + 1]
    pair_ptr: torch.Tensor        # int32 [n_pairs + 1]
    lrow: torch.Tensor            # int16 bit patterns of the unsigned tile-local rows [nnz]
    pair_dst: torch.Tensor        # int32 [n_pairs]
    col_pair_ptr: torch.Tensor    # int32 [n_cols + 1]
    partial: Optional[torch.Tensor] = None   # float32 scratch [>= n_pairs]; may be shared between indices


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
    tiled: Optional[TiledPart] = None   # when set, the per-column arrays above are empty

    def nbytes(self) -> int:
        ts = [self.colptr, self.rowidx, self.ucols, self.bins, self.long_col, self.long_e0, self.long_e1]
        if self.tiled is not None:
            ts += [self.tiled.tile_pair_ptr, self.tiled.pair_ptr, self.tiled.lrow, self.tiled.pair_dst, self.tiled.col_pair_ptr]
        return sum(t.numel() * t.element_size() for t in ts) + (self.svals.numel() * 4 if self.svals is not None else 0)


def _build_tiled(csr: DeviceCSR, lo: int, hi: int, e0: int, e1: int, rows: torch.Tensor) -> BatchIndex:
    dev = csr.cols.device
    nrows = hi - lo
    n_tiles = max(1, -(-nrows // TILE_ROWS_MAX))
    tile_rows = ((-(-nrows // n_tiles)) + 3) // 4 * 4
    cols = csr.cols[e0:e1].long()
    tile = (rows // tile_rows).long()
    skey, order = torch.sort((tile << 32) | cols, stable=True)   # (tile, column); rows stay ascending inside a pair
    local = (rows.long() - tile * tile_rows)[order]
    lrow = torch.where(local >= 32768, local - 65536, local).to(torch.int16).contiguous()   # unsigned 16-bit patterns
    svals = None if csr.values is None else csr.values[e0:e1][order].contiguous()
    # pairs of the frequent columns are cut into segments of PAIR_SEGMENT entries (each with its own partial sum),
    # so that no warp is left with one very long list
    pk0, pc0 = torch.unique_consecutive(skey, return_counts=True)
    start0 = torch.cumsum(pc0, 0) - pc0
    rank = torch.arange(e1 - e0, device=dev) - torch.repeat_interleave(start0, pc0, output_size=e1 - e0)
    seg = rank // PAIR_SEGMENT
    skey_seg = skey * SEG_SLOTS + seg            # still ascending: seg grows inside a pair
    pkey_seg, pcnt = torch.unique_consecutive(skey_seg, return_counts=True)
    pkey, pseg = pkey_seg // SEG_SLOTS, pkey_seg % SEG_SLOTS
    n_pairs = int(pkey.numel())
    pair_ptr = torch.zeros(n_pairs + 1, dtype=torch.int32, device=dev)
    pair_ptr[1:] = torch.cumsum(pcnt, 0).to(torch.int32)
    ptile, pcol = pkey >> 32, pkey & 0xFFFFFFFF
    tile_pair_ptr = torch.searchsorted(ptile, torch.arange(n_tiles + 1, device=dev)).to(torch.int32)
    skey2, perm = torch.sort(((pcol << 20) | ptile) * SEG_SLOTS + pseg)   # (column, tile, segment)
    skey2 = skey2 // SEG_SLOTS
    pair_dst = torch.empty(n_pairs, dtype=torch.int32, device=dev)
    pair_dst[perm] = torch.arange(n_pairs, dtype=torch.int32, device=dev)
    ucols, ccnt = torch.unique_consecutive(skey2 >> 20, return_counts=True)
    n = int(ucols.numel())
    col_pair_ptr = torch.zeros(n + 1, dtype=torch.int32, device=dev)
    col_pair_ptr[1:] = torch.cumsum(ccnt, 0).to(torch.int32)
    empty = torch.zeros(0, dtype=torch.int32, device=dev)
    part = TiledPart(tile_rows, n_tiles, n_pairs, tile_pair_ptr.contiguous(), pair_ptr, lrow, pair_dst, col_pair_ptr)
    return BatchIndex(lo, nrows, n, empty, empty, svals, ucols.to(torch.int32).contiguous(), empty, empty, empty, empty, 0, 0, 0,
                      torch.tensor([n, 1 if n else 0, 0, 0], dtype=torch.int64, device=dev), part)


def build_batch_index(csr: DeviceCSR, lo: int, hi: int, tiled: bool = False) -> BatchIndex:
    """``tiled``: the row-tiled form (coefficients of a row tile in shared memory, no atomics); needs fewer than
    2^20 tiles, i.e. any batch that fits a GPU."""
    dev = csr.cols.device
    e0, e1 = int(csr.rowptr[lo]), int(csr.rowptr[hi])
    cols = csr.cols[e0:e1]
    counts = (csr.rowptr[lo + 1:hi + 1] - csr.rowptr[lo:hi])
    rows = torch.repeat_interleave(torch.arange(hi - lo, device=dev, dtype=torch.int32), counts, output_size=e1 - e0)
    if tiled and e1 > e0:
        return _build_tiled(csr, lo, hi, e0, e1, rows)
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
    if bi.tiled is not None:
        tp = bi.tiled
        if tp.partial is None or tp.partial.numel() < tp.n_pairs:
            tp.partial = torch.zeros(max(tp.n_pairs, 1), dtype=torch.float32, device=coef.device)
        L.check(lib.skml_colsum_tiled(L.ptr(tp.tile_pair_ptr), L.ptr(tp.pair_ptr), L.ptr(tp.lrow), L.ptr(bi.svals),
                                      L.ptr(tp.pair_dst), L.ptr(tp.col_pair_ptr), L.ptr(bi.ucols), bi.rows, tp.tile_rows,
                                      tp.n_tiles, bi.n_cols, L.ptr(coef), L.ptr(w), float(lam), L.ptr(tp.partial),
                                      L.ptr(out_vals), L.stream()), "skml_colsum_tiled")
        L.count_launches(3)
        return
    L.check(lib.skml_colsum(L.ptr(bi.colptr), L.ptr(bi.rowidx), L.ptr(bi.svals), L.ptr(bi.ucols), L.ptr(bi.bins),
                            L.ptr(bi.long_col), L.ptr(bi.long_e0), L.ptr(bi.long_e1), bi.n_short, bi.n_medium, bi.n_long,
                            bi.n_cols, L.ptr(coef), L.ptr(w), float(lam), L.ptr(out_vals), L.stream()), "skml_colsum")
    L.count_launches(2)
