"""Host-side gradient containers (torch tensors) and the compressor factory.

Reference: ml/gradient/Gradient.scala:18-182 (factory ``compress``, ``sum``,
``evaluateCompression``, abstract API, ``ZeroGradient``), Kind.scala,
DenseDoubleGradient.scala:10-95, SparseDoubleGradient.scala:8-48,
DenseFloatGradient.scala / SparseFloatGradient.scala (fp32 cast),
SketchGradient.scala:24-70, FixedPointGradient.scala:39-75, ZipGradient.scala:27-129.

The compressed kinds keep their wire form (an SKML payload, or bit words) produced by
the C++ oracle; the GPU training path never builds these objects, it runs the fused
kernels on device buffers instead.
"""
from __future__ import annotations

import enum
from typing import Iterable, Optional

import numpy as np
import torch

from .. import config as C
from ..compress import oracle

EPS = 1e-8


class Kind(enum.Enum):
    ZeroGradient = 0
    DenseDouble = 1
    SparseDouble = 2
    DenseFloat = 3
    SparseFloat = 4
    Sketch = 5
    FixedPoint = 6
    Zip = 7


class Gradient:
    kind = None

    def __init__(self, dim: int):
        self.dim = int(dim)

    # --- API of Gradient.scala:70-140 ---
    def plus_by(self, other: "Gradient") -> "Gradient":
        raise NotImplementedError(f"Cannot add to {self.kind}")

    def times_by(self, x: float) -> None:
        raise NotImplementedError

    def count_nnz(self) -> int:
        raise NotImplementedError

    def to_dense(self) -> "DenseDoubleGradient":
        raise NotImplementedError

    def to_sparse(self) -> "SparseDoubleGradient":
        raise NotImplementedError

    def to_auto(self) -> "Gradient":
        raise NotImplementedError

    def nbytes(self) -> int:
        """Bytes this gradient would put on the wire."""
        raise NotImplementedError


class _Zero(Gradient):
    """Identity element of ``plus_by`` (Gradient.scala:145-181)."""
    kind = Kind.ZeroGradient

    def __init__(self):
        super().__init__(0)

    def plus_by(self, other):
        return other

    def times_by(self, x):
        pass

    def count_nnz(self):
        return 0

    def to_auto(self):
        return self

    def nbytes(self):
        return 0


ZeroGradient = _Zero()


class DenseDoubleGradient(Gradient):
    kind = Kind.DenseDouble
    dtype = torch.float64

    def __init__(self, dim: int, values: Optional[torch.Tensor] = None):
        super().__init__(dim)
        self.values = torch.zeros(dim, dtype=self.dtype) if values is None else values.to(self.dtype)
        if self.values.numel() != dim:
            raise ValueError("value count does not match dim")

    def plus_by(self, other: Gradient) -> "DenseDoubleGradient":
        if other.kind is Kind.ZeroGradient:
            return self
        if other.dim != self.dim:
            raise ValueError("Adding gradients with different dimensions")
        o = other if other.kind in (Kind.DenseDouble, Kind.SparseDouble, Kind.DenseFloat, Kind.SparseFloat) \
            else other.to_auto()
        if hasattr(o, "indices"):
            self.values.index_add_(0, o.indices.long(), o.values.to(self.dtype))
        else:
            self.values += o.values.to(self.dtype)
        return self

    def plus_by_features(self, cols: torch.Tensor, vals: torch.Tensor) -> None:
        """``plusBy(x, scalar)`` for a whole batch: scatter-add (DenseDoubleGradient.scala:51-57)."""
        self.values.index_add_(0, cols.long(), vals.to(self.dtype))

    def times_by(self, x: float) -> None:
        self.values *= x

    def count_nnz(self) -> int:
        return int((self.values.abs() > EPS).sum())

    def to_dense(self):
        return self

    def to_sparse(self) -> "SparseDoubleGradient":
        idx = torch.nonzero(self.values.abs() > EPS).flatten()
        return SparseDoubleGradient(self.dim, idx.to(torch.int32), self.values[idx])

    def to_auto(self) -> Gradient:
        """Dense iff nnz > 2/3 dim (DenseDoubleGradient.scala:92-95)."""
        nnz = self.count_nnz()
        if nnz > self.dim * 2 // 3 or nnz == 0:
            return self
        return self.to_sparse()

    def nbytes(self):
        return self.values.numel() * self.values.element_size()


class SparseDoubleGradient(Gradient):
    kind = Kind.SparseDouble
    dtype = torch.float64

    def __init__(self, dim: int, indices: torch.Tensor, values: torch.Tensor, check: bool = True):
        super().__init__(dim)
        self.indices = indices.to(torch.int32)
        self.values = values.to(self.dtype)
        if self.indices.numel() != self.values.numel():
            raise ValueError("index and value counts differ")
        if check and self.indices.numel():
            if int(self.indices[0]) < 0 or int(self.indices[-1]) >= dim:
                raise ValueError("gradient index out of range")
            if self.indices.numel() > 1 and not bool((self.indices[1:] > self.indices[:-1]).all()):
                raise ValueError("gradient indices must be strictly increasing")

    def times_by(self, x):
        self.values *= x

    def count_nnz(self):
        return int(self.indices.numel())

    def to_dense(self) -> DenseDoubleGradient:
        d = DenseDoubleGradient(self.dim)
        keep = self.values.abs() > EPS
        d.values[self.indices[keep].long()] = self.values[keep].to(d.dtype)
        return d

    def to_sparse(self):
        return self

    def to_auto(self):
        return self.to_dense() if self.count_nnz() > self.dim * 2 // 3 else self

    def nbytes(self):
        return self.indices.numel() * (4 + self.values.element_size())


class DenseFloatGradient(DenseDoubleGradient):
    """The "Float" compressor: values cast to fp32 (DenseFloatGradient.scala:20-31)."""
    kind = Kind.DenseFloat
    dtype = torch.float32

    def to_dense(self):
        return DenseDoubleGradient(self.dim, self.values.double())

    def to_sparse(self):
        return self.to_dense().to_sparse()

    def to_auto(self):
        return self.to_dense().to_auto()


class SparseFloatGradient(SparseDoubleGradient):
    kind = Kind.SparseFloat
    dtype = torch.float32

    def to_sparse(self):
        return SparseDoubleGradient(self.dim, self.indices, self.values.double(), check=False)

    def to_dense(self):
        return self.to_sparse().to_dense()

    def to_auto(self):
        return self.to_sparse().to_auto()


class SketchGradient(Gradient):
    """Quantile-bucket quantisation + grouped MinMaxSketch + delta-coded keys
    (SketchGradient.scala:35-48); dense gradients keep one bucket code per coordinate
    (SketchGradient.scala:24-33)."""
    kind = Kind.Sketch

    def __init__(self, grad: Optional[Gradient], conf: C.MLConf, step: int = 0, rank: int = 0, world: int = 1,
                 payload: Optional[bytes] = None, loss_partials=None):
        if payload is not None:
            self.payload = payload
            super().__init__(oracle.parse(payload)["dim"])
            return
        super().__init__(grad.dim)
        opts = conf.sketch_options(step, rank, world)
        if loss_partials is not None:
            opts["loss_partials"] = list(loss_partials)
        np_dtype = np.float64 if conf.dtype == "float64" else np.float32
        if grad.kind in (Kind.DenseDouble, Kind.DenseFloat):
            self.payload = oracle.compress_dense(grad.values.cpu().numpy().astype(np_dtype), opts)
        elif grad.kind in (Kind.SparseDouble, Kind.SparseFloat):
            self.payload = oracle.compress_sparse(grad.indices.cpu().numpy(), grad.values.cpu().numpy().astype(np_dtype),
                                                  grad.dim, opts)
        elif grad.kind is Kind.ZeroGradient:
            self.payload = oracle.compress_sparse(np.zeros(0, np.int32), np.zeros(0, np_dtype), conf.feature_num, opts)
        else:
            raise ValueError(f"Cannot create {self.kind} from {grad.kind}")

    def times_by(self, x: float) -> None:
        self.payload = oracle.payload_times_by(self.payload, float(x))

    def count_nnz(self) -> int:
        return int(oracle.parse(self.payload)["nnz"])

    def decode(self):
        kind, keys, vals = oracle.decompress(self.payload)
        return kind, torch.from_numpy(keys), torch.from_numpy(vals).double()

    def to_dense(self) -> DenseDoubleGradient:
        kind, keys, vals = self.decode()
        d = DenseDoubleGradient(self.dim)
        d.values[keys.long()] = vals
        return d

    def to_sparse(self) -> SparseDoubleGradient:
        kind, keys, vals = self.decode()
        return SparseDoubleGradient(self.dim, keys, vals, check=False)

    def to_auto(self) -> Gradient:
        kind, keys, vals = self.decode()
        if kind == 2:
            return DenseDoubleGradient(self.dim, vals).to_auto()
        if kind == 0:
            return ZeroGradient
        return SparseDoubleGradient(self.dim, keys, vals, check=False).to_auto()

    def nbytes(self):
        return len(self.payload)


class FixedPointGradient(Gradient):
    """Baseline: sign + (b-1)-bit magnitude relative to the L2 norm, keys sent raw
    (FixedPointGradient.scala:39-75)."""
    kind = Kind.FixedPoint

    def __init__(self, grad: Gradient, num_bits: int, seed: int = 0):
        super().__init__(grad.dim)
        if grad.kind in (Kind.DenseDouble, Kind.DenseFloat):
            self.indices = None
        elif grad.kind in (Kind.SparseDouble, Kind.SparseFloat):
            self.indices = grad.indices
        else:
            raise ValueError(f"Cannot create {self.kind} from {grad.kind}")
        self.code = oracle.fixed_point_encode(grad.values.double().cpu().numpy(), num_bits, seed)

    def times_by(self, x):
        self.code["norm"] *= x

    def count_nnz(self):
        return int(self.code["size"])

    def _values(self):
        return torch.from_numpy(oracle.fixed_point_decode(self.code))

    def to_dense(self):
        if self.indices is None:
            return DenseDoubleGradient(self.dim, self._values())
        return self.to_sparse().to_dense()

    def to_sparse(self):
        if self.indices is None:
            return self.to_dense().to_sparse()
        return SparseDoubleGradient(self.dim, self.indices, self._values(), check=False)

    def to_auto(self):
        return (self.to_dense() if self.indices is None else self.to_sparse()).to_auto()

    def nbytes(self):
        n = int(self.code["size"])
        return 8 + (n * int(self.code["num_bits"]) + 7) // 8 + (0 if self.indices is None else 4 * n)


class ZipGradient(Gradient):
    """Baseline: ZipML-style variance-driven bucket merging, keys sent raw
    (ZipGradient.scala:27-129)."""
    kind = Kind.Zip

    def __init__(self, grad: Gradient, bin_num: int):
        super().__init__(grad.dim)
        if grad.kind in (Kind.DenseDouble, Kind.DenseFloat):
            self.indices = None
        elif grad.kind in (Kind.SparseDouble, Kind.SparseFloat):
            self.indices = grad.indices
        else:
            raise ValueError(f"Cannot create {self.kind} from {grad.kind}")
        self.q = oracle.zipml_quantize(grad.values.double().cpu().numpy(), bin_num)
        self.scale = 1.0

    def times_by(self, x):
        self.scale *= x

    def count_nnz(self):
        return len(self.q["bins"])

    def _values(self):
        return torch.from_numpy(self.q["values"][self.q["bins"]] * self.scale)

    def to_dense(self):
        if self.indices is None:
            return DenseDoubleGradient(self.dim, self._values())
        return self.to_sparse().to_dense()

    def to_sparse(self):
        if self.indices is None:
            return self.to_dense().to_sparse()
        return SparseDoubleGradient(self.dim, self.indices, self._values(), check=False)

    def to_auto(self):
        return (self.to_dense() if self.indices is None else self.to_sparse()).to_auto()

    def nbytes(self):
        n = len(self.q["bins"])
        code = 1 if self.q["bin_num"] <= 256 else 2
        return 28 + 8 * (self.q["bin_num"] - 1) + n * code + (0 if self.indices is None else 4 * n)


def compress(grad: Gradient, conf: C.MLConf, step: int = 0, rank: int = 0, world: int = 1,
             loss_partials=None) -> Gradient:
    """Factory by compressor name (Gradient.scala:18-42)."""
    name = conf.compressor
    if name == C.COMPRESSOR_NONE or grad.kind is Kind.ZeroGradient and name != C.COMPRESSOR_SKETCH:
        return grad
    if name == C.COMPRESSOR_FLOAT:
        if grad.kind is Kind.DenseDouble:
            return DenseFloatGradient(grad.dim, grad.values)
        if grad.kind is Kind.SparseDouble:
            return SparseFloatGradient(grad.dim, grad.indices, grad.values, check=False)
        return grad
    if name == C.COMPRESSOR_SKETCH:
        return SketchGradient(grad, conf, step, rank, world, loss_partials=loss_partials)
    if name == C.COMPRESSOR_FIXED_POINT:
        return FixedPointGradient(grad, conf.fixed_point_bit_num, seed=conf.seed * 1315423911 + step * 8191 + rank)
    if name == C.COMPRESSOR_ZIP:
        return ZipGradient(grad, conf.quant_bin_num)
    raise ValueError("Unrecognizable gradient compressor: " + name)


def sum_gradients(dim: int, grads: Iterable[Gradient]) -> Gradient:
    """Dense fp64 sum of the workers' gradients, then ``to_auto`` (Gradient.scala:44-49)."""
    total = DenseDoubleGradient(dim)
    for g in grads:
        if g.kind is not Kind.ZeroGradient and g.dim != dim:
            raise ValueError("Adding gradients with different dimensions")
        total.plus_by(g)
    return total.to_auto()


def evaluate_compression(origin: Gradient, comp: Gradient) -> dict:
    """Squared euclidean distance, cosine and size ratio between a gradient and its
    decoded compressed form (Gradient.scala:51-67)."""
    a = origin.to_dense().values.double()
    b = comp.to_auto()
    b = (b.to_dense().values.double() if b.kind is not Kind.ZeroGradient else torch.zeros_like(a))
    eu = float(((a - b) ** 2).sum())
    den = float(torch.linalg.vector_norm(a) * torch.linalg.vector_norm(b))
    cos = float((a * b).sum()) / den if den > 0 else 0.0
    raw = origin.nbytes()
    return {"euclidean": eu, "cosine": cos, "raw_bytes": raw, "compressed_bytes": comp.nbytes(),
            "ratio": raw / max(1, comp.nbytes()),
            "rel_l2": float(np.sqrt(eu) / max(float(torch.linalg.vector_norm(a)), 1e-300))}
