"""Python wrappers of the GLM kernels (gradient, compaction, validation, updates)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch

from ..data import CSRMatrix
from . import lib as L


class DeviceCSR:
    """A CSR shard in device memory, with ``cols`` / ``values`` padded to a multiple of 4
    elements so that 16-byte bulk copies of row tiles never read past the allocation."""

    def __init__(self, m: CSRMatrix, device):
        dev = torch.device(device)
        nnz = m.nnz
        self.rows, self.dim, self.nnz = m.rows, m.dim, nnz
        self.nnz_padded = (nnz + 3) // 4 * 4 + 4
        self.rowptr = m.rowptr.to(dev, torch.int64).contiguous()
        self.cols = torch.zeros(self.nnz_padded, dtype=torch.int32, device=dev)
        self.cols[:nnz] = m.cols.to(dev)
        self.values = None
        if m.values is not None:
            self.values = torch.zeros(self.nnz_padded, dtype=torch.float32, device=dev)
            self.values[:nnz] = m.values.to(dev, torch.float32)
        self.labels = m.labels.to(dev, torch.float32).contiguous()
        self.avg_nnz = nnz / max(1, m.rows)
        d = self.rowptr[1:] - self.rowptr[:-1]
        self.max_row_nnz = int(d.max()) if m.rows else 0

    @classmethod
    def from_parts(cls, rowptr, cols_padded, values_padded, labels, dim, nnz):
        self = cls.__new__(cls)
        self.rows, self.dim, self.nnz = int(rowptr.numel() - 1), dim, nnz
        self.nnz_padded = int(cols_padded.numel())
        self.rowptr, self.cols, self.values, self.labels = rowptr, cols_padded, values_padded, labels
        self.avg_nnz = nnz / max(1, self.rows)
        self.max_row_nnz = int((rowptr[1:] - rowptr[:-1]).max()) if self.rows else 0
        return self

    def to_matrix(self) -> CSRMatrix:
        return CSRMatrix(self.rowptr, self.cols[:self.nnz], None if self.values is None else self.values[:self.nnz],
                         self.labels, self.dim)


@dataclass
class GlmState:
    """Per-model device buffers of the gradient pipeline."""
    dim: int
    n_max: int
    g: torch.Tensor            # fp32 [dim] accumulator, all zero between steps
    bitmap: torch.Tensor       # uint32-as-int32 [ceil(dim/32)], all zero between steps
    keys: torch.Tensor         # int32 [n_max]
    vals: torch.Tensor         # fp32 [n_max]
    meta: torch.Tensor         # int64 [4]: nnz, kind
    block_counts: torch.Tensor
    dense_vals: Optional[torch.Tensor]
    status: torch.Tensor       # int32 [1]
    partials: torch.Tensor     # fp64 [4]: batch size, objective loss sum, reg loss, spare

    @classmethod
    def create(cls, dim: int, n_max: int, device, allow_dense: bool = False) -> "GlmState":
        dev = torch.device(device)
        n_max = int(min(max(n_max, 1), dim))
        nwords = (dim + 31) // 32
        nblocks = int(L.lib().skml_compact_blocks(dim))
        return cls(dim, n_max, torch.zeros(dim, dtype=torch.float32, device=dev),
                   torch.zeros(nwords + 4, dtype=torch.int32, device=dev),
                   torch.zeros(n_max, dtype=torch.int32, device=dev), torch.zeros(n_max, dtype=torch.float32, device=dev),
                   torch.zeros(4, dtype=torch.int64, device=dev), torch.zeros(nblocks + 1, dtype=torch.int32, device=dev),
                   torch.zeros(dim, dtype=torch.float32, device=dev) if allow_dense else None,
                   torch.zeros(1, dtype=torch.int32, device=dev), torch.zeros(4, dtype=torch.float64, device=dev))


def glm_grad(csr: DeviceCSR, segments: List[Tuple[int, int]], w: torch.Tensor, st: GlmState, loss_id: int,
             batch_size: int, hot: int = 8192, budget_s: float = 1.0) -> None:
    """Adds the batch gradient (mean over ``batch_size`` rows) into ``st.g`` / ``st.bitmap`` and
    the objective loss sum into ``st.partials[1]``. ``segments`` are [lo, hi) row ranges."""
    lib = L.lib()
    inv = 1.0 / max(1, batch_size)
    for lo, hi in segments:
        if hi <= lo:
            continue
        L.check(lib.skml_glm_grad(L.ptr(csr.rowptr), L.ptr(csr.cols), L.ptr(csr.values), L.ptr(csr.labels), lo, hi - lo,
                                  csr.nnz_padded, float(csr.avg_nnz), L.ptr(w), L.ptr(st.g), L.ptr(st.bitmap), loss_id,
                                  inv, int(min(hot, st.dim) // 32 * 32), st.partials.data_ptr() + 8, L.ptr(st.status),
                                  L.budget_cycles(budget_s), L.stream()), "skml_glm_grad")
        L.count_launches(1)


def glm_validate(csr: DeviceCSR, w: torch.Tensor, loss_id: int, status: torch.Tensor,
                 margins: Optional[torch.Tensor] = None, budget_s: float = 1.0) -> torch.Tensor:
    """Returns a device fp64 tensor [sum loss, TP, TN, FP, FN, n]."""
    acc = torch.zeros(6, dtype=torch.float64, device=w.device)
    if csr.rows:
        L.check(L.lib().skml_glm_validate(L.ptr(csr.rowptr), L.ptr(csr.cols), L.ptr(csr.values), L.ptr(csr.labels), 0,
                                          csr.rows, csr.nnz_padded, float(csr.avg_nnz), L.ptr(w), loss_id, L.ptr(acc),
                                          L.ptr(margins), L.ptr(status), L.budget_cycles(budget_s), L.stream()),
                "skml_glm_validate")
        L.count_launches(1)
    acc[5] = csr.rows
    return acc


def compact_gradient(st: GlmState, w: torch.Tensor, lam: float) -> None:
    """``st.g`` + ``st.bitmap`` -> sorted ``st.keys`` / ``st.vals`` (or ``st.dense_vals``), count and
    kind in ``st.meta``; clears the accumulator and the bitmap."""
    L.check(L.lib().skml_compact(L.ptr(st.g), L.ptr(w), L.ptr(st.bitmap), st.dim, float(lam), L.ptr(st.block_counts),
                                 L.ptr(st.meta), L.ptr(st.keys), L.ptr(st.vals), L.ptr(st.dense_vals), st.n_max,
                                 L.ptr(st.status), L.stream()), "skml_compact")
    L.count_launches(3)


def moment_stride(m, v) -> int:
    """Elements between the Adam moments of neighbouring coordinates: 1 for plain arrays, 4 when m and v are
    columns 0 and 1 of one [dim, 4] array (both moments of a coordinate then share a memory sector)."""
    if m is None or v is None:
        return 1
    sm, sv = int(m.stride(0)), int(v.stride(0))
    if sm != sv or sm not in (1, 4) or (sm == 4 and v.data_ptr() != m.data_ptr() + 4):
        raise ValueError("Adam moments must be two plain arrays or columns 0 and 1 of one [dim, 4] float32 array")
    return sm


def update_dense(w, g, scale: float, lr: float, m=None, v=None, adam_scale: float = 1.0, sparse_only: bool = False):
    L.check(L.lib().skml_update_dense(L.ptr(w), L.ptr(m), L.ptr(v), L.ptr(g), w.numel(), scale, int(v is not None), lr,
                                      adam_scale, int(sparse_only), moment_stride(m, v), L.stream()), "skml_update_dense")


def update_gathered(w, acc, keys, counts, stride: int, lists: int, scale: float, lr: float, m=None, v=None,
                    adam_scale: float = 1.0):
    """Applies ``acc[key] * scale`` on the coordinates of the gathered key lists and clears them."""
    L.check(L.lib().skml_update_gathered(L.ptr(w), L.ptr(m), L.ptr(v), L.ptr(acc), L.ptr(keys), L.ptr(counts), stride,
                                         lists, scale, int(v is not None), lr, adam_scale, moment_stride(m, v), L.stream()),
            "skml_update_gathered")
    L.count_launches(lists)


def update_sparse(w, keys, vals, n_ptr: Optional[torch.Tensor], n_max: int, scale: float, lr: float, m=None, v=None,
                  adam_scale: float = 1.0):
    L.check(L.lib().skml_update_sparse(L.ptr(w), L.ptr(m), L.ptr(v), L.ptr(keys), L.ptr(vals), L.ptr(n_ptr), n_max,
                                       scale, int(v is not None), lr, adam_scale, moment_stride(m, v), L.stream()),
            "skml_update_sparse")
