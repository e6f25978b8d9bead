"""Device-side synthetic data generator (counter-based random numbers; no host copy).

Same rules as ``sketchml_b200.data.synthetic`` (Zipf columns without replacement inside a
row, binary / unit-L2 uniform / normal values, labels from a planted weight vector); the
random streams differ, so it is checked statistically against the numpy generator."""
from __future__ import annotations

import torch

from ..data.synthetic import SyntheticSpec
from . import lib as L
from .glm import DeviceCSR

_VALUE_KIND = {"binary": 0, "uniform_l2": 1, "normal": 2}
_TASK = {"logistic": 0, "svm": 1, "regression": 2}


def generate_gpu(spec: SyntheticSpec, row_offset: int, rows: int, device, wstar: torch.Tensor = None):
    """Returns (DeviceCSR of rows [row_offset, row_offset + rows), planted weights)."""
    dev = torch.device(device)
    lib = L.lib()
    k = spec.nnz_per_row
    if wstar is None:
        wstar = torch.empty(spec.dim, dtype=torch.float32, device=dev)
        L.check(lib.skml_gen_wstar(L.ptr(wstar), spec.dim, float(spec.wstar_density), spec.seed + 7919, L.stream()),
                "skml_gen_wstar")
    nnz = rows * k
    padded = (nnz + 3) // 4 * 4 + 4
    cols = torch.zeros(padded, dtype=torch.int32, device=dev)
    vals = None if spec.values == "binary" else torch.zeros(padded, dtype=torch.float32, device=dev)
    labels = torch.empty(rows, dtype=torch.float32, device=dev)
    if rows:
        rc = lib.skml_gen_rows(L.ptr(cols), L.ptr(vals), L.ptr(labels), row_offset, rows, spec.dim, k, float(spec.zipf_s),
                               _VALUE_KIND[spec.values], _TASK[spec.task], float(spec.noise), L.ptr(wstar), spec.seed,
                               L.stream())
        if rc == -1:
            raise ValueError("nnz_per_row must be in [1, min(256, dim)] for the device generator")
        L.check(rc, "skml_gen_rows")
    rowptr = torch.arange(0, (rows + 1) * k, k, dtype=torch.int64, device=dev)
    return DeviceCSR.from_parts(rowptr, cols, vals, labels, spec.dim, nnz), wstar
