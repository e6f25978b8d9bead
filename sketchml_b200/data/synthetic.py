"""Synthetic data of the shapes named by the benchmark configurations.

Columns of a row are drawn from a Zipf(s) law over ``dim`` features without replacement
inside the row (or uniformly when ``zipf_s == 0``); values are 1.0 ("binary"),
Uniform(0,1) scaled to unit L2 norm per row ("uniform_l2") or N(0,1) ("normal").
A planted weight vector ``w*`` (N(0,1) on a random fraction of features) gives labels:
Bernoulli(sigmoid(x.w*)) for logistic regression, sign(x.w* + noise) for the SVM and
x.w* + noise for least squares.

This module is the numpy generator for small cases and the oracle of the device
generator (``sketchml_b200.ops.datagen``), which restates the same rules with
counter-based random numbers and runs on the GPU for the 50M-200M row configurations.
The reference reads text files only (ml/data/Parser.scala); it has no generator.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from .dataset import CSRMatrix


@dataclass
class SyntheticSpec:
    rows: int
    dim: int
    nnz_per_row: int
    zipf_s: float = 1.1
    values: str = "binary"          # binary | uniform_l2 | normal
    task: str = "logistic"          # logistic | svm | regression
    wstar_density: float = 0.1
    noise: float = 0.0
    seed: int = 0


def zipf_inverse_cdf(u: np.ndarray, dim: int, s: float) -> np.ndarray:
    """Continuous approximation of the Zipf(s) inverse CDF on ranks 1..dim: the density
    x^-s on [1, dim+1) is inverted in closed form and floored. Returns 0-based ranks."""
    if s == 0.0:
        return np.minimum((u * dim).astype(np.int64), dim - 1)
    if abs(s - 1.0) < 1e-9:
        x = np.exp(u * np.log(dim + 1.0))
    else:
        a = 1.0 - s
        top = (dim + 1.0) ** a
        x = (1.0 + u * (top - 1.0)) ** (1.0 / a)
    return np.clip(x.astype(np.int64) - 1, 0, dim - 1)


def planted_weights(spec: SyntheticSpec) -> np.ndarray:
    rng = np.random.default_rng(spec.seed + 7919)
    w = np.zeros(spec.dim, dtype=np.float64)
    if spec.wstar_density >= 1.0:
        w[:] = rng.normal(size=spec.dim)
    else:
        m = rng.random(spec.dim) < spec.wstar_density
        w[m] = rng.normal(size=int(m.sum()))
    return w


def generate_cpu(spec: SyntheticSpec, row_offset: int = 0, rows: int | None = None,
                 dtype: torch.dtype = torch.float32):
    """Rows [row_offset, row_offset + rows) of the data set; returns (CSRMatrix, w*)."""
    rows = spec.rows if rows is None else rows
    k = spec.nnz_per_row
    if k > spec.dim:
        raise ValueError("nnz_per_row exceeds dim")
    w = planted_weights(spec)
    cols = np.empty((rows, k), dtype=np.int64)
    for i in range(rows):
        rng = np.random.default_rng((spec.seed * 1000003 + row_offset + i) & 0xFFFFFFFF)
        got = set()
        out = []
        while len(out) < k:
            c = zipf_inverse_cdf(rng.random(2 * k), spec.dim, spec.zipf_s)
            for x in c:
                xi = int(x)
                if xi not in got:
                    got.add(xi)
                    out.append(xi)
                    if len(out) == k:
                        break
        cols[i] = np.sort(np.asarray(out, dtype=np.int64))
    rng = np.random.default_rng(spec.seed + 104729 + row_offset)
    if spec.values == "binary":
        vals = None
        dense_vals = np.ones((rows, k))
    elif spec.values == "uniform_l2":
        dense_vals = rng.random((rows, k)) + 1e-12
        dense_vals /= np.linalg.norm(dense_vals, axis=1, keepdims=True)
        vals = dense_vals
    elif spec.values == "normal":
        dense_vals = rng.normal(size=(rows, k))
        vals = dense_vals
    else:
        raise ValueError("unknown value kind " + spec.values)
    margin = (w[cols] * dense_vals).sum(axis=1)
    if spec.task == "logistic":
        p = 1.0 / (1.0 + np.exp(-margin))
        y = np.where(rng.random(rows) < p, 1.0, -1.0)
    elif spec.task == "svm":
        y = np.where(margin + spec.noise * rng.normal(size=rows) >= 0, 1.0, -1.0)
    elif spec.task == "regression":
        y = margin + spec.noise * rng.normal(size=rows)
    else:
        raise ValueError("unknown task " + spec.task)
    rowptr = torch.arange(0, (rows + 1) * k, k, dtype=torch.int64)
    m = CSRMatrix(rowptr, torch.from_numpy(cols.reshape(-1).astype(np.int32)),
                  None if vals is None else torch.from_numpy(vals.reshape(-1)).to(dtype),
                  torch.from_numpy(y).to(dtype), spec.dim)
    return m, w
