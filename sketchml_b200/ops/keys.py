"""DeltaAdaptive key codec on the device as a stand-alone call.

The reference's live key encoder (binary/DeltaAdaptiveEncoder.java:23-146): an adaptive
variable-width bit code for sorted keys. The training step does not come through here: with
``key_encoder="delta_adaptive"`` the fused compress and decode kernels write and read this format
themselves, chunk by chunk, without leaving the device (csrc/cuda/compress_kernels.cu,
decode_common.cuh). This module is the library form of the codec, `encode(keys) -> AdaptiveKeys`
and back, bit for bit equal to the CPU oracle (`oracle.delta_adaptive_encode`). It returns tensors
of exactly the encoded size, which depends on the data, so `encode` reads the status, the chosen
mode and the two bit counts back to the host in one copy; the kernels are maps over keys or words
(csrc/cuda/keys_kernels.cu) with `torch.cumsum` between them.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import lib as L


@dataclass
class AdaptiveKeys:
    size: int
    num_intervals: int
    flag_kind: int            # 0 = fixed-width flags, 1 = unary flags
    flag_bits: int
    delta_bits: int
    flag_words: torch.Tensor  # int64 on the device: java.util.BitSet words, ceil(flag_bits / 64) of them
    delta_words: torch.Tensor

    def to_oracle_dict(self) -> dict:
        import numpy as np
        return {"size": self.size, "num_intervals": self.num_intervals, "flag_kind": self.flag_kind,
                "flag_words": self.flag_words.cpu().numpy().view(np.uint64), "flag_bits": self.flag_bits,
                "delta_words": self.delta_words.cpu().numpy().view(np.uint64), "delta_bits": self.delta_bits}

    def nbytes_wire(self) -> int:
        """Bytes of the reference's field layout: 3 ints + flag + 2 counted word arrays."""
        return 4 + 4 + 1 + 4 + 8 * self.flag_words.numel() + 4 + 8 * self.delta_words.numel()


def _words(bits: int, device) -> torch.Tensor:
    # 64-bit words plus one spare: readers fetch the 32-bit word after the one a value starts in
    return torch.zeros((bits + 63) // 64 + 1, dtype=torch.int64, device=device)


def encode(keys: torch.Tensor) -> AdaptiveKeys:
    """keys: strictly increasing non-negative int32 on the device (synchronises to size the outputs)."""
    if keys.dtype != torch.int32 or not keys.is_cuda:
        raise ValueError("keys must be a CUDA int32 tensor")
    keys = keys.contiguous()
    n, dev, lib = keys.numel(), keys.device, L.lib()
    hist = torch.zeros(32, dtype=torch.int32, device=dev)
    params = torch.zeros(2, dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    L.check(lib.skml_da_analyze(L.ptr(keys), n, L.ptr(hist), L.ptr(params), L.ptr(status), L.stream()), "skml_da_analyze")
    flag_w = torch.zeros(max(n, 1), dtype=torch.int32, device=dev)
    delta_w = torch.zeros(max(n, 1), dtype=torch.int32, device=dev)
    L.check(lib.skml_da_widths(L.ptr(keys), n, L.ptr(params), L.ptr(flag_w), L.ptr(delta_w), L.stream()), "skml_da_widths")
    flag_incl = torch.cumsum(flag_w[:n], 0, dtype=torch.int64) if n else torch.zeros(0, dtype=torch.int64, device=dev)
    delta_incl = torch.cumsum(delta_w[:n], 0, dtype=torch.int64) if n else torch.zeros(0, dtype=torch.int64, device=dev)
    # the one read-back of the call: status, mode and the two stream lengths together
    zero = torch.zeros(1, dtype=torch.int64, device=dev)
    st, m, kind, flag_bits, delta_bits = (int(x) for x in torch.cat(
        [status.long(), params.long(), flag_incl[-1:] if n else zero, delta_incl[-1:] if n else zero]).tolist())
    if st & 1:
        raise ValueError("keys must be non-negative and strictly increasing")
    fw, dw = _words(flag_bits, dev), _words(delta_bits, dev)
    L.check(lib.skml_da_pack(L.ptr(keys), n, L.ptr(params), L.ptr(flag_incl), L.ptr(delta_incl), L.ptr(fw), L.ptr(dw),
                             L.stream()), "skml_da_pack")
    L.count_launches(4 if n else 1)
    return AdaptiveKeys(n, m, kind, flag_bits, delta_bits, fw[:(flag_bits + 63) // 64], dw[:(delta_bits + 63) // 64])


def decode(e: AdaptiveKeys) -> torch.Tensor:
    """Returns the int32 keys on the device."""
    dev, lib, n = e.delta_words.device, L.lib(), e.size
    if n == 0:
        return torch.zeros(0, dtype=torch.int32, device=dev)
    pad = torch.zeros(1, dtype=torch.int64, device=dev)
    fw = torch.cat([e.flag_words.to(torch.int64), pad]).contiguous()
    dw = torch.cat([e.delta_words.to(torch.int64), pad]).contiguous()
    b = 32 // e.num_intervals
    if e.flag_kind == 0:
        fb = e.num_intervals.bit_length() - 1
        iv = torch.zeros(n, dtype=torch.int32, device=dev)
        L.check(lib.skml_da_fixed_iv(L.ptr(fw), n, fb, L.ptr(iv), L.stream()), "skml_da_fixed_iv")
        L.count_launches(1)
    else:
        nw = (e.flag_bits + 31) // 32
        zeros = torch.zeros(max(nw, 1), dtype=torch.int32, device=dev)
        L.check(lib.skml_da_zero_count(L.ptr(fw), e.flag_bits, L.ptr(zeros), L.stream()), "skml_da_zero_count")
        zeros_incl = torch.cumsum(zeros, 0, dtype=torch.int64)
        pos = torch.full((n,), -1, dtype=torch.int64, device=dev)
        L.check(lib.skml_da_zero_pos(L.ptr(fw), e.flag_bits, L.ptr(zeros_incl), n, L.ptr(pos), L.stream()), "skml_da_zero_pos")
        L.count_launches(2)
        prev = torch.cat([pos.new_full((1,), -1), pos[:-1]])
        iv = (pos - prev - 1).to(torch.int32)
    delta_w = (iv * b).contiguous()
    delta_incl = torch.cumsum(delta_w, 0, dtype=torch.int64)
    deltas = torch.zeros(n, dtype=torch.int64, device=dev)
    L.check(lib.skml_da_extract(L.ptr(dw), n, L.ptr(delta_w), L.ptr(delta_incl), L.ptr(deltas), L.stream()), "skml_da_extract")
    L.count_launches(1)
    return torch.cumsum(deltas, 0).to(torch.int32)
