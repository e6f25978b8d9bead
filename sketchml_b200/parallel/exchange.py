"""Peer-memory receive regions for the fused gradient exchange.

Every rank owns one region ``[arrival flags][2 parities x world payload slots]`` in its own
GPU memory and maps every peer's region (CUDA IPC, one process per GPU on one node). The
compress kernel of rank r stores its payload into slot ``[step & 1][r]`` of EVERY region
and then releases the matching arrival flag; the decode kernel of each rank reads only its
own region. This replaces the reference's gather-to-driver + broadcast
(ml/algorithm/GeneralizedLinearModel.scala:145-156).

Slot reuse needs no acknowledgement: a rank can start step t+2 only after it decoded step
t+1, which needs every peer's step t+1 payload, which a peer produces only after it has
finished decoding step t; so the slot of parity t is never overwritten while in use.

Only plain peer loads and stores are used (no multicast objects), so a rank that leaves
between steps cannot fault its peers' GPUs.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch

from ..ops import lib as L
from ..ops.codec import FLAG_BYTES, ExchangeRegionView


class _RawDeviceBytes:
    """CUDA array interface over a raw device pointer, so that torch can view the bytes without owning them."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1", "data": (int(ptr), False), "version": 2}


class PeerExchange:
    def __init__(self, comm, slot_capacity: int, device: torch.device):
        self.comm = comm
        self.rank, self.world = comm.rank, comm.world
        if self.world > L.MAX_PEERS:
            raise ValueError(f"at most {L.MAX_PEERS} ranks are supported by the peer exchange")
        self.device = device
        self.slot_capacity = int((slot_capacity + 255) // 256 * 256)
        nbytes = ExchangeRegionView.region_bytes(self.world, self.slot_capacity)
        # an allocation of its own, outside the caching allocator: the IPC handle names exactly this buffer
        raw = C.c_void_p()
        with torch.cuda.device(device):
            L.check(L.lib().skml_region_alloc(nbytes, C.byref(raw)), "cudaMalloc(receive region)")
        self._raw = raw.value
        self.region = torch.as_tensor(_RawDeviceBytes(self._raw, nbytes), device=device)
        self._opened: List[int] = []
        self.views: List[ExchangeRegionView] = [None] * self.world
        self.views[self.rank] = ExchangeRegionView(self.region.data_ptr(), self.world, self.slot_capacity)
        if self.world > 1:
            self._map_peers()

    def _map_peers(self) -> None:
        lib = L.lib()
        handle = (C.c_ubyte * 64)()
        # the handle names the allocation that contains the pointer; send the offset too
        L.check(lib.skml_ipc_get_handle(self.region.data_ptr(), C.addressof(handle)), "cudaIpcGetMemHandle")
        blob = bytes(handle) + int(0).to_bytes(8, "little")  # the region starts its allocation
        blobs = self.comm.all_gather_bytes(blob)
        for r, b in enumerate(blobs):
            if r == self.rank:
                continue
            h = (C.c_ubyte * 64).from_buffer_copy(b[:64])
            off = int.from_bytes(b[64:72], "little")
            p = C.c_void_p()
            L.check(lib.skml_ipc_open_handle(C.addressof(h), C.byref(p)), f"cudaIpcOpenMemHandle(rank {r})")
            self._opened.append(p.value)
            self.views[r] = ExchangeRegionView(p.value + off, self.world, self.slot_capacity)
        self.comm.barrier()

    # --- pointers for one step -------------------------------------------------
    def send_ptrs(self, step: int):
        """(payload slot of this rank in every region, matching flag addresses)."""
        par = step & 1
        return ([v.slot(par, self.rank) for v in self.views], [v.flag(par, self.rank) for v in self.views])

    def recv_ptrs(self, step: int):
        """(all ranks' slots in this rank's region, their flag addresses)."""
        par = step & 1
        me = self.views[self.rank]
        return ([me.slot(par, r) for r in range(self.world)], [me.flag(par, r) for r in range(self.world)])

    def local_slot(self, step: int, src: int) -> torch.Tensor:
        par = step & 1
        off = FLAG_BYTES + (par * self.world + src) * self.slot_capacity
        return self.region[off:off + self.slot_capacity]

    def close(self) -> None:
        lib = L.lib()
        for p in self._opened:
            lib.skml_ipc_close(p)
        self._opened.clear()
        if getattr(self, "_raw", None):
            # peers store into this region only for a step whose decode this rank has already finished
            # (the decode needs every peer's payload), so nothing of theirs is in flight here any more
            torch.cuda.synchronize(self.device)
            self.region = None
            lib.skml_region_free(self._raw)
            self._raw = None
