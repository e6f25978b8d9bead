"""Text parsers producing CSR tensors.

Reference: ml/data/Parser.scala:10-76. ``libsvm``: "label idx:val idx:val ..." split on
single spaces, indices used as given (no 1->0 shift); ``csv``: "label,v,v,..." dense;
``dummy``: "label,idx,idx,..." with every value 1.0. With ``neg_y`` any label that is
not within 1e-8 of 1 becomes -1 (Parser.scala:28-30). The reference always parses with
``neg_y = true``, which also binarises regression targets; here the caller chooses.
"""
from __future__ import annotations

from typing import Iterable, Optional

import numpy as np
import torch

from .dataset import CSRMatrix, shard_rows

EPS = 1e-8


def _label(tok: str, neg_y: bool) -> float:
    y = float(tok)
    if neg_y and abs(y - 1.0) > EPS:
        y = -1.0
    return y


def parse_libsvm(line: str, max_dim: int, neg_y: bool = True):
    parts = line.strip().split(" ")
    if not parts or parts[0] == "":
        return None
    y = _label(parts[0], neg_y)
    idx, val = [], []
    for tok in parts[1:]:
        tok = tok.strip()
        if not tok:
            continue
        k, v = tok.split(":")
        idx.append(int(k))
        val.append(float(v))
    return y, idx, val


def parse_csv(line: str, max_dim: int, neg_y: bool = True):
    parts = line.strip().split(",")
    if not parts or parts[0] == "":
        return None
    y = _label(parts[0], neg_y)
    val = [float(t) for t in parts[1:]]
    return y, list(range(len(val))), val


def parse_dummy(line: str, max_dim: int, neg_y: bool = True):
    parts = line.strip().split(",")
    if not parts or parts[0] == "":
        return None
    y = _label(parts[0], neg_y)
    idx = [int(t) for t in parts[1:] if t.strip()]
    return y, idx, None


_PARSERS = {"libsvm": parse_libsvm, "csv": parse_csv, "dummy": parse_dummy}


def parse_lines(lines: Iterable[str], fmt: str, max_dim: int, neg_y: bool = True,
                dtype: torch.dtype = torch.float32) -> CSRMatrix:
    if fmt not in _PARSERS:
        raise ValueError("Unknown file format: " + fmt)
    parse = _PARSERS[fmt]
    rowptr, cols, vals, labels = [0], [], [], []
    implicit = fmt == "dummy"
    dup_rows = 0
    for line in lines:
        if not line.strip():
            continue
        rec = parse(line, max_dim, neg_y)
        if rec is None:
            continue
        y, idx, val = rec
        if idx and (min(idx) < 0 or max(idx) >= max_dim):
            raise ValueError(f"feature index out of range [0, {max_dim}) in line: {line[:80]!r}")
        order = np.argsort(np.asarray(idx, dtype=np.int64), kind="stable") if idx else []
        # a feature listed twice in one row is merged (values add up): the kernels rely on
        # distinct columns inside a row
        last = None
        for i in order:
            c = int(idx[i])
            x = 1.0 if val is None else float(val[i])
            if c == last:
                dup_rows += 1
                vals[-1] += x
            else:
                cols.append(c)
                vals.append(x)
                last = c
        labels.append(y)
        rowptr.append(len(cols))
    return CSRMatrix(
        torch.tensor(rowptr, dtype=torch.int64), torch.tensor(cols, dtype=torch.int32),
        None if (implicit and dup_rows == 0) else torch.tensor(vals, dtype=dtype), torch.tensor(labels, dtype=dtype),
        max_dim)


def parse_text_native(text: str, fmt: str, max_dim: int, neg_y: bool = True,
                      dtype: torch.dtype = torch.float32) -> CSRMatrix:
    """Same result as ``parse_lines`` through the C++ parser of the oracle module (one pass over
    the bytes; used for files, where the Python loop above would dominate the load time)."""
    from ..compress import oracle
    try:
        rowptr, cols, vals, labels, implicit = oracle.parse_text(text, fmt, int(max_dim), bool(neg_y))
    except oracle.SketchMLError as e:
        raise ValueError(str(e)) from e
    return CSRMatrix(torch.from_numpy(rowptr), torch.from_numpy(cols),
                     None if implicit else torch.from_numpy(vals).to(dtype), torch.from_numpy(labels).to(dtype), max_dim)


def load_data(path: str, fmt: str, max_dim: int, rank: int = 0, world: int = 1, neg_y: bool = True,
              dtype: torch.dtype = torch.float32, limit: Optional[int] = None) -> tuple:
    """Reads ``path`` and returns (this rank's contiguous shard, global offset of its
    first row, total rows). The reference's ``repartition(workerNum)`` is replaced by
    even contiguous shards so the assignment is a pure function of (rows, rank, world)."""
    with open(path, "r") as f:
        lines = [ln for ln in f if ln.strip()]
    if limit is not None:
        lines = lines[:limit]
    lo, hi = shard_rows(len(lines), rank, world)
    return parse_text_native("".join(lines[lo:hi]), fmt, max_dim, neg_y, dtype), lo, len(lines)
