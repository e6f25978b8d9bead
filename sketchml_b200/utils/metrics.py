"""Structured metrics (JSON lines) plus a human-readable log.

The reference logs through slf4j/log4j at INFO with the pattern "%d %C %p - %m%n"
(ml/src/main/resources/log4j.properties): per batch the batch size, objective loss, reg
loss and batch loss; per epoch train loss, validation loss, accuracy ("precision"),
true/false recall; per compression the source and target kind and time. The same
quantities are emitted here, plus samples/s, payload bytes, compression ratios against
8 B and 12 B per non-zero, and per-phase device times."""
from __future__ import annotations

import json
import logging
import sys
import time
from typing import Optional

_FMT = "%(asctime)s %(name)s %(levelname)s - %(message)s"


def get_logger(name: str = "sketchml_b200", level: int = logging.INFO) -> logging.Logger:
    lg = logging.getLogger(name)
    if not lg.handlers:
        h = logging.StreamHandler(sys.stderr)
        h.setFormatter(logging.Formatter(_FMT))
        lg.addHandler(h)
        lg.setLevel(level)
        lg.propagate = False
    return lg


class MetricsLogger:
    def __init__(self, path: Optional[str] = None, rank: int = 0):
        self.rank = rank
        self.records = []
        self._f = open(path, "a") if (path and rank == 0) else None

    def log(self, event: str, **fields) -> dict:
        rec = {"event": event, "ts": time.time(), "rank": self.rank}
        rec.update(fields)
        self.records.append(rec)
        if self._f:
            self._f.write(json.dumps(rec, default=float) + "\n")
            self._f.flush()
        return rec

    def of(self, event: str):
        return [r for r in self.records if r["event"] == event]

    def close(self) -> None:
        if self._f:
            self._f.close()
            self._f = None


def rank_sum_auc(scores, labels, java_compat: bool = False) -> float:
    """Area under the ROC curve by the rank-sum formula over the scores sorted ascending
    (ml/util/ValidationUtil.scala:69-82): with M positives (label 1) and N others,
    AUC = (sum of the positives' ranks - M (M + 1) / 2) / (M N). The reference adds up 0-based positions
    instead of ranks, which lowers its figure by 1 / N; ``java_compat`` reproduces that. Works on torch
    tensors of any device (one sort)."""
    import torch
    s = torch.as_tensor(scores).double().flatten()
    y = torch.as_tensor(labels).to(s.device).flatten()
    pos = (y == 1)[torch.argsort(s, stable=True)]
    m, n = int(pos.sum()), int((~pos).sum())
    if m == 0 or n == 0:
        return float("nan")
    ranks = torch.arange(0 if java_compat else 1, s.numel() + (0 if java_compat else 1), device=s.device, dtype=torch.float64)
    return float((ranks[pos].sum() - m * (m + 1) / 2.0) / m / n)
