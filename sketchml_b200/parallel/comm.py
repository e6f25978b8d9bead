"""Host-side collective layer over ``torch.distributed`` (gloo on CPU, NCCL on GPUs).

It replaces the Spark actions the reference uses as its only communication layer
(ml/algorithm/GeneralizedLinearModel.scala:49-67 rank discovery and counts, :127-135
scalar reduce, :145-148 gather of compressed gradients, :155-156 broadcast + barrier,
:163-168 validation reduce). The compressed-gradient exchange of the GPU path does not
go through this file; it is done inside the fused kernels over peer memory
(``sketchml_b200.parallel.exchange``).
"""
from __future__ import annotations

import datetime
import os
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


class CommFailure(RuntimeError):
    """A collective did not complete: a peer is missing, late, or sent a bad message."""


class LocalComm:
    """world_size == 1: every collective is the identity."""
    rank, world, backend = 0, 1, "local"

    def all_gather_bytes(self, b: bytes) -> List[bytes]:
        return [b]

    def all_reduce_sum(self, xs: Sequence[float]) -> List[float]:
        return [float(x) for x in xs]

    def all_reduce_tensor(self, t: torch.Tensor) -> torch.Tensor:
        return t

    def broadcast_object(self, obj, src: int = 0):
        return obj

    def barrier(self) -> None:
        pass

    def store_set(self, key: str, value: str) -> None:
        self.__dict__.setdefault("_kv", {})[key] = value

    def store_get(self, key: str) -> Optional[str]:
        return self.__dict__.get("_kv", {}).get(key)

    def close(self) -> None:
        pass


class TorchComm:
    """One process per rank; created from the RANK / WORLD_SIZE / MASTER_* environment."""

    def __init__(self, backend: str = "gloo", timeout_s: float = 300.0, device: Optional[torch.device] = None):
        self.backend = backend
        self.device = device or torch.device("cpu")
        self._own = False
        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29531")
            kw = {}
            if backend == "nccl" and self.device.type == "cuda":
                kw["device_id"] = self.device
            dist.init_process_group(backend=backend, timeout=datetime.timedelta(seconds=timeout_s), **kw)
            self._own = True
        self.rank = dist.get_rank()
        self.world = dist.get_world_size()
        self._store = None

    def _wrap(self, fn, *a, **k):
        try:
            return fn(*a, **k)
        except (RuntimeError, dist.DistBackendError) as e:  # timeout, closed connection, peer exit
            raise CommFailure(f"rank {self.rank}: collective failed: {e}") from e

    def all_gather_bytes(self, b: bytes) -> List[bytes]:
        n = torch.tensor([len(b)], dtype=torch.int64, device=self.device)
        sizes = [torch.zeros_like(n) for _ in range(self.world)]
        self._wrap(dist.all_gather, sizes, n)
        cap = int(max(int(s) for s in sizes))
        buf = torch.zeros(max(cap, 1), dtype=torch.uint8, device=self.device)
        if len(b):
            buf[:len(b)] = torch.frombuffer(bytearray(b), dtype=torch.uint8).to(self.device)
        out = [torch.zeros_like(buf) for _ in range(self.world)]
        self._wrap(dist.all_gather, out, buf)
        return [bytes(o[:int(s)].cpu().numpy().tobytes()) for o, s in zip(out, sizes)]

    def all_reduce_sum(self, xs: Sequence[float]) -> List[float]:
        t = torch.tensor(list(xs), dtype=torch.float64, device=self.device)
        self._wrap(dist.all_reduce, t)
        return t.cpu().tolist()

    def all_reduce_tensor(self, t: torch.Tensor) -> torch.Tensor:
        self._wrap(dist.all_reduce, t)
        return t

    def broadcast_object(self, obj, src: int = 0):
        box = [obj]
        self._wrap(dist.broadcast_object_list, box, src=src)
        return box[0]

    def barrier(self) -> None:
        self._wrap(dist.barrier)

    def _kv(self):
        if self._store is None:
            self._store = dist.distributed_c10d._get_default_store()
        return self._store

    def store_set(self, key: str, value: str) -> None:
        self._kv().set(key, value)

    def store_get(self, key: str) -> Optional[str]:
        st = self._kv()
        try:
            if hasattr(st, "check") and not st.check([key]):
                return None
            return st.get(key).decode()
        except Exception:
            return None

    def close(self) -> None:
        if self._own and dist.is_initialized():
            dist.destroy_process_group()


def make_comm(backend: str = "auto", timeout_s: float = 300.0, device: Optional[torch.device] = None):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1 and not dist.is_initialized():
        return LocalComm()
    if backend == "auto":
        backend = "nccl" if (device is not None and device.type == "cuda") else "gloo"
    return TorchComm(backend, timeout_s, device)
