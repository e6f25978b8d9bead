"""Failure detection and host-side fault injection.

The reference has none of its own (a lost Spark executor loses weights, optimizer state
and data, ml/algorithm/GeneralizedLinearModel.scala:21-31). Here:

* every rank publishes a heartbeat (its step counter) in the rendezvous store and checks
  its peers' before each step;
* every received payload is validated (magic, version, header checksum, step, source
  rank, sizes) before any section is touched;
* device-side waits are bounded: on expiry a kernel writes a status word which the host
  turns into ``StepTimeout``;
* faults are injected on the host only: a rank can skip publishing, publish a stale step
  or corrupt a header byte of a host-staged payload. Nothing here faults, traps or hangs
  a GPU.
"""
from __future__ import annotations

import struct
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional

from ..compress import oracle
from .comm import CommFailure

# status words written by kernels (csrc/cuda/skml_device.cuh)
STATUS_OK = 0
STATUS_TIMEOUT_BARRIER = 1
STATUS_TIMEOUT_PEER = 2
STATUS_BAD_HEADER = 3
STATUS_CAPACITY = 4
STATUS_BAD_INPUT = 5
STATUS_NAMES = {0: "ok", 1: "grid barrier timed out", 2: "peer payload did not arrive in time",
                3: "payload header failed validation", 4: "payload exceeds slot capacity",
                5: "invalid kernel input"}


class PayloadError(RuntimeError):
    """A received payload failed validation."""


class StepTimeout(RuntimeError):
    """A bounded device-side or host-side wait expired."""


class PeerLost(CommFailure):
    """A peer's heartbeat is missing or stale."""


def validate_payload(buf: bytes, expect_step: Optional[int] = None, expect_rank: Optional[int] = None,
                     expect_dim: Optional[int] = None) -> dict:
    try:
        p = oracle.parse(buf)
    except oracle.SketchMLError as e:
        raise PayloadError(str(e)) from e
    if expect_step is not None and p["step"] != expect_step:
        raise PayloadError(f"stale payload: step {p['step']} received, step {expect_step} expected")
    if expect_rank is not None and p["rank"] != expect_rank:
        raise PayloadError(f"payload from rank {p['rank']} found in the slot of rank {expect_rank}")
    if expect_dim is not None and p["dim"] != expect_dim:
        raise PayloadError(f"payload dim {p['dim']} does not match model dim {expect_dim}")
    return p


def check_status(status: int, where: str = "") -> None:
    """Turns a kernel status word into an exception (the GPU context stays usable)."""
    code = status & 0xFF
    if code == STATUS_OK:
        return
    detail = f"{STATUS_NAMES.get(code, 'unknown status')} (status word 0x{status:x}) {where}".strip()
    if code in (STATUS_TIMEOUT_BARRIER, STATUS_TIMEOUT_PEER):
        raise StepTimeout(detail)
    if code == STATUS_BAD_HEADER:
        raise PayloadError(detail)
    raise RuntimeError(detail)


@dataclass
class FaultInjector:
    """Host-side hooks used by tests: ``skip_publish_steps`` makes this rank not send its
    payload at those steps; ``stale_steps`` re-sends the previous step's payload;
    ``corrupt_steps`` flips one header byte of the outgoing host-staged payload;
    ``exit_at_step`` makes the rank raise SystemExit between steps."""
    skip_publish_steps: set = field(default_factory=set)
    stale_steps: set = field(default_factory=set)
    corrupt_steps: set = field(default_factory=set)
    exit_at_step: Optional[int] = None
    _last: Optional[bytes] = None

    def outgoing(self, step: int, payload: bytes) -> Optional[bytes]:
        out = payload
        if step in self.stale_steps and self._last is not None:
            out = self._last
        if step in self.corrupt_steps:
            b = bytearray(out)
            b[24] ^= 0x5A  # a byte of the step field: the checksum no longer matches
            out = bytes(b)
        self._last = payload
        if step in self.skip_publish_steps:
            return None
        return out

    def between_steps(self, step: int) -> None:
        if self.exit_at_step is not None and step == self.exit_at_step:
            raise SystemExit(17)


class Heartbeat:
    """Step counters in the rendezvous store. ``check`` raises PeerLost when a peer is
    more than ``max_lag`` steps behind for longer than ``timeout_s``."""

    def __init__(self, comm, timeout_s: float = 30.0, max_lag: int = 1):
        self.comm, self.timeout_s, self.max_lag = comm, timeout_s, max_lag

    def beat(self, step: int) -> None:
        self.comm.store_set(f"skml/hb/{self.comm.rank}", f"{step}:{time.time():.3f}")

    def mark_failed(self, reason: str) -> None:
        self.comm.store_set(f"skml/failed/{self.comm.rank}", reason)

    def peers(self) -> Dict[int, Optional[int]]:
        out = {}
        for r in range(self.comm.world):
            v = self.comm.store_get(f"skml/hb/{r}")
            out[r] = int(v.split(":")[0]) if v else None
        return out

    def check(self, step: int) -> None:
        deadline = time.time() + self.timeout_s
        while True:
            bad: List[str] = []
            for r in range(self.comm.world):
                if r == self.comm.rank:
                    continue
                f = self.comm.store_get(f"skml/failed/{r}")
                if f:
                    raise PeerLost(f"rank {r} reported failure: {f}")
                v = self.comm.store_get(f"skml/hb/{r}")
                s = int(v.split(":")[0]) if v else None
                if s is None or s + self.max_lag < step:
                    bad.append(f"rank {r} at step {s}")
            if not bad:
                return
            if time.time() > deadline:
                raise PeerLost(f"step {step}: no heartbeat from " + ", ".join(bad))
            time.sleep(0.01)
