"""CSR row store and the cyclic minibatch cursor.

Reference: ml/data/DataSet.scala:15-21 (``loopingRead``: minibatches are consecutive
cyclic slices of the local shard, not random samples), ml/data/LabeledData.scala,
ml/algorithm/GeneralizedLinearModel.scala:56-67 (train/valid split; the reference
draws an unseeded coin per row, here the coin is a hash of (seed, global row id)).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import numpy as np
import torch

_MASK64 = (1 << 64) - 1


def _splitmix64_np(x: np.ndarray) -> np.ndarray:
    x = (x + np.uint64(0x9E3779B97F4A7C15)).astype(np.uint64)
    x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return x ^ (x >> np.uint64(31))


def row_coin(seed: int, global_row_ids: np.ndarray) -> np.ndarray:
    """Uniform [0,1) value per global row id; a pure function of (seed, id)."""
    with np.errstate(over="ignore"):
        h = _splitmix64_np(global_row_ids.astype(np.uint64) ^ np.uint64((seed * 0x9E3779B97F4A7C15 + 0xD1B54A32D192ED03) & _MASK64))
    return (h >> np.uint64(11)).astype(np.float64) * (1.0 / (1 << 53))


@dataclass
class CSRMatrix:
    """Rows of labelled sparse features. ``values is None`` means every stored
    entry is 1.0 (the reference's "dummy" format)."""
    rowptr: torch.Tensor            # int64 [rows + 1]
    cols: torch.Tensor              # int32 [nnz]
    values: Optional[torch.Tensor]  # float [nnz] or None
    labels: torch.Tensor            # float [rows]
    dim: int

    @property
    def rows(self) -> int:
        return int(self.rowptr.numel() - 1)

    @property
    def nnz(self) -> int:
        return int(self.cols.numel())

    @property
    def device(self):
        return self.cols.device

    def to(self, device, dtype=None, non_blocking=False) -> "CSRMatrix":
        v = self.values
        lab = self.labels
        if dtype is not None:
            v = None if v is None else v.to(dtype)
            lab = lab.to(dtype)
        return CSRMatrix(self.rowptr.to(device, non_blocking=non_blocking), self.cols.to(device, non_blocking=non_blocking),
                         None if v is None else v.to(device, non_blocking=non_blocking),
                         lab.to(device, non_blocking=non_blocking), self.dim)

    def select_rows(self, idx: torch.Tensor) -> "CSRMatrix":
        idx = idx.to(torch.int64)
        start = self.rowptr[idx]
        cnt = self.rowptr[idx + 1] - start
        new_ptr = torch.zeros(idx.numel() + 1, dtype=torch.int64, device=self.rowptr.device)
        torch.cumsum(cnt, 0, out=new_ptr[1:])
        total = int(new_ptr[-1])
        row_of = torch.repeat_interleave(torch.arange(idx.numel(), device=cnt.device), cnt, output_size=total)
        pos = torch.arange(total, device=cnt.device) - new_ptr[row_of] + start[row_of]
        return CSRMatrix(new_ptr, self.cols[pos], None if self.values is None else self.values[pos],
                         self.labels[idx], self.dim)

    def slice_rows(self, lo: int, hi: int) -> "CSRMatrix":
        a, b = int(self.rowptr[lo]), int(self.rowptr[hi])
        return CSRMatrix(self.rowptr[lo:hi + 1] - a, self.cols[a:b],
                         None if self.values is None else self.values[a:b], self.labels[lo:hi], self.dim)

    def row_ids(self) -> torch.Tensor:
        cnt = self.rowptr[1:] - self.rowptr[:-1]
        return torch.repeat_interleave(torch.arange(self.rows, device=cnt.device), cnt, output_size=self.nnz)

    def dense_values(self, dtype) -> torch.Tensor:
        if self.values is None:
            return torch.ones(self.nnz, dtype=dtype, device=self.cols.device)
        return self.values.to(dtype)

    @staticmethod
    def concat(parts: List["CSRMatrix"]) -> "CSRMatrix":
        ptrs, off = [torch.zeros(1, dtype=torch.int64)], 0
        for p in parts:
            ptrs.append(p.rowptr[1:] + off)
            off += p.nnz
        vals = None if any(p.values is None for p in parts) else torch.cat([p.values for p in parts])
        return CSRMatrix(torch.cat(ptrs), torch.cat([p.cols for p in parts]), vals,
                         torch.cat([p.labels for p in parts]), parts[0].dim)


class DataSet:
    """A shard of rows plus a cyclic read cursor (DataSet.scala:15-21)."""

    def __init__(self, matrix: CSRMatrix):
        self.matrix = matrix
        self.read_index = 0

    @property
    def size(self) -> int:
        return self.matrix.rows

    def batch_size(self, ratio: float) -> int:
        """``(size * ratio).toInt`` (GradientDescent.scala:28)."""
        return int(self.size * ratio)

    def looping_segments(self, count: int) -> List[Tuple[int, int]]:
        """Advances the cursor by ``count`` rows and returns the [lo, hi) row ranges
        that were read (more than one when the read wraps around the shard end)."""
        segs = []
        n = self.size
        if n == 0:
            return segs
        left = count
        while left > 0:
            take = min(left, n - self.read_index)
            segs.append((self.read_index, self.read_index + take))
            self.read_index = (self.read_index + take) % n
            left -= take
        return segs

    def looping_read(self, count: int) -> CSRMatrix:
        segs = self.looping_segments(count)
        parts = [self.matrix.slice_rows(lo, hi) for lo, hi in segs]
        return parts[0] if len(parts) == 1 else CSRMatrix.concat(parts)


def shard_rows(total_rows: int, rank: int, world: int) -> Tuple[int, int]:
    """Even contiguous shards; the first ``total % world`` ranks get one extra row."""
    base, extra = divmod(total_rows, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def split_train_valid(matrix: CSRMatrix, valid_ratio: float, seed: int, global_offset: int = 0):
    """Row goes to validation iff coin(seed, global id) <= valid_ratio, else training."""
    if valid_ratio <= 0:
        return matrix, matrix.slice_rows(0, 0)
    ids = np.arange(global_offset, global_offset + matrix.rows, dtype=np.uint64)
    coin = row_coin(seed, ids)
    train = torch.from_numpy(np.nonzero(coin > valid_ratio)[0])
    valid = torch.from_numpy(np.nonzero(coin <= valid_ratio)[0])
    return matrix.select_rows(train.to(matrix.rowptr.device)), matrix.select_rows(valid.to(matrix.rowptr.device))
