"""Per-phase timers. The reference logs wall-clock deltas per phase
(ml/algorithm/GeneralizedLinearModel.scala:46-175, ml/objective/GradientDescent.scala:24-47,
ml/objective/Adam.scala:28-34); here GPU phases are timed with CUDA events on the
launching stream, host phases with ``perf_counter``, and NVTX ranges carry the same names."""
from __future__ import annotations

import contextlib
import time
from collections import defaultdict
from typing import Callable, Dict

import torch


class PhaseTimer:
    def __init__(self, use_cuda: bool = False, enabled: bool = True):
        self.use_cuda = use_cuda and torch.cuda.is_available()
        self.enabled = enabled
        self.total_ms: Dict[str, float] = defaultdict(float)
        self.count: Dict[str, int] = defaultdict(int)
        self._pending = []

    @contextlib.contextmanager
    def phase(self, name: str):
        if not self.enabled:
            yield
            return
        if self.use_cuda:
            torch.cuda.nvtx.range_push(name)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            try:
                yield
            finally:
                b.record()
                torch.cuda.nvtx.range_pop()
                self._pending.append((name, a, b))
        else:
            t0 = time.perf_counter()
            try:
                yield
            finally:
                self.total_ms[name] += (time.perf_counter() - t0) * 1e3
                self.count[name] += 1

    def flush(self) -> None:
        """Resolves recorded CUDA events (synchronises once)."""
        if self._pending:
            torch.cuda.synchronize()
            for name, a, b in self._pending:
                self.total_ms[name] += a.elapsed_time(b)
                self.count[name] += 1
            self._pending.clear()

    def summary(self) -> Dict[str, dict]:
        self.flush()
        return {k: {"total_ms": v, "count": self.count[k], "mean_ms": v / max(1, self.count[k])}
                for k, v in self.total_ms.items()}

    def reset(self) -> None:
        self.flush()
        self.total_ms.clear()
        self.count.clear()


def cuda_time_ms(fn: Callable[[], None], warmup: int = 3, iters: int = 10, flush_l2: bool = True) -> float:
    """Median device time of ``fn`` in ms: warm-up, then CUDA events around each call on
    the current stream, with an L2 flush (write of a 256 MiB buffer) between calls."""
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush_l2 else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.fill_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    times.sort()
    return times[len(times) // 2]
