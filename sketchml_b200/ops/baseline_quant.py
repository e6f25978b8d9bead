"""Device versions of the two baseline value quantizers.

FixedPoint: `FixedPointCodec` wraps the pack / unpack kernels (csrc/cuda/baseline_kernels.cu):
the b-bit codes are what travels between ranks (4 + b/8 bytes per non-zero), keys raw as in
the reference (ml/gradient/FixedPointGradient.scala:27-30). `fixed_point_roundtrip` is the
same arithmetic in torch ops, kept for the dense gradient kind.

Zip: `ZipCodec` wraps the ZipML kernels (csrc/cuda/zipml_kernels.cu): split search, one bucket
code per value and the table of bucket midpoints; codes, table and raw keys are what travels
(keys raw as in the reference, ml/gradient/ZipGradient.scala:27-30).

Reference: ml/gradient/FixedPointGradient.scala:39-75 (sign + (b-1)-bit magnitude of
floor(|v| / ||v||_2 * max) + Bernoulli(1/2)), ml/gradient/ZipGradient.scala:70-129 (sorted
values, prefix sums of v and v^2, repeated halving of the split candidates keeping the
bin_num/2 adjacent pairs with the largest squared error, bucket midpoints as decode values).
"""
from __future__ import annotations

import torch

from . import lib as L


class FixedPointCodec:
    """Packs the values of a sparse gradient of up to ``n_max`` entries into ``bits``-bit codes
    and decodes several ranks' (keys, codes, norm) lists back into a dense sum."""

    def __init__(self, n_max: int, bits: int, world: int, device):
        if not 2 <= bits < 30:
            raise ValueError(f"Bit num out of range: {bits}")
        self.lib = L.lib()
        self.n_max, self.bits, self.world = int(n_max), int(bits), int(world)
        self.code_stride = (int(self.lib.skml_fixedpoint_code_bytes(self.n_max, bits)) + 15) // 16 * 16
        self.scratch = torch.zeros(int(self.lib.skml_fixedpoint_scratch_bytes()) // 8, dtype=torch.float64, device=device)
        self.codes = torch.zeros(self.code_stride, dtype=torch.uint8, device=device)
        self.norm = torch.zeros(1, dtype=torch.float64, device=device)
        if world > 1:
            self.all_codes = torch.zeros((world, self.code_stride), dtype=torch.uint8, device=device)
            self.all_norms = torch.zeros(world, dtype=torch.float64, device=device)

    def pack(self, vals: torch.Tensor, n: torch.Tensor, seed: int) -> None:
        """vals[:n] -> self.codes, self.norm (n: device int64 scalar / 1-element view)."""
        L.check(self.lib.skml_fixedpoint_pack(L.ptr(vals), L.ptr(n), self.n_max, self.bits, int(seed) & (2 ** 64 - 1),
                                              L.ptr(self.scratch), L.ptr(self.codes), L.ptr(self.norm), L.stream()),
                "skml_fixedpoint_pack")
        L.count_launches(2)

    def unpack(self, keys: torch.Tensor, codes: torch.Tensor, norms: torch.Tensor, counts: torch.Tensor, lists: int,
               acc: torch.Tensor = None, vals_out: torch.Tensor = None) -> None:
        L.check(self.lib.skml_fixedpoint_unpack_scatter(L.ptr(acc), L.ptr(keys), L.ptr(codes), L.ptr(norms), L.ptr(counts),
                                                        self.n_max, self.code_stride, lists, self.bits, L.ptr(vals_out),
                                                        L.stream()), "skml_fixedpoint_unpack_scatter")
        L.count_launches(lists)  # one launch per list: the lists reach a coordinate in list order on every rank

    def wire_bytes(self, n: int) -> int:
        """Bytes one rank contributes for n non-zeros: raw keys, codes, count and norm."""
        return 4 * n + (n + 7) // 8 * self.bits + 16


def fixed_point_roundtrip(vals: torch.Tensor, n: torch.Tensor, num_bits: int, seed: int) -> None:
    """In place on vals[:n] (n is a device scalar; entries beyond n are ignored)."""
    idx = torch.arange(vals.numel(), device=vals.device)
    live = idx < n
    v = torch.where(live, vals, torch.zeros_like(vals)).double()
    norm = torch.linalg.vector_norm(v)
    mx = float((1 << (num_bits - 1)) - 1)
    g = torch.Generator(device=vals.device)
    g.manual_seed(int(seed) & 0x7FFFFFFFFFFFFFFF)
    sigma = torch.randint(0, 2, (vals.numel(),), generator=g, device=vals.device).double()
    code = torch.where(norm > 0, torch.floor(v.abs() / norm.clamp_min(1e-300) * mx) + sigma, torch.zeros_like(v))
    code = code.clamp_max(mx)  # the reference lets this overflow into the sign bit
    out = (code / mx * norm) * torch.sign(v)
    vals.copy_(torch.where(live, out.float(), vals))


class ZipCodec:
    """ZipML quantizer on the device for up to ``n_max`` values: ``pack`` leaves one bucket code per value
    (``code_bytes`` each) and the table of bucket midpoints; these and the raw keys are what travels
    between ranks. No step of it reads anything back to the host."""

    def __init__(self, n_max: int, bin_num: int, world: int, device):
        self.lib = L.lib()
        self.n_max, self.bin_num, self.world = int(n_max), int(bin_num), int(world)
        if not 2 <= self.bin_num <= 8190:
            raise ValueError(f"Zip compressor: bin number out of range: {bin_num}")
        self.code_bytes = int(self.lib.skml_zipml_code_bytes(self.bin_num))
        self.table_len = int(self.lib.skml_zipml_table_len(self.bin_num))
        self.code_stride = (self.n_max * self.code_bytes + 15) // 16 * 16
        self.scratch_bytes = int(self.lib.skml_zipml_scratch_bytes(self.n_max))
        if self.scratch_bytes <= 0:
            raise ValueError(f"Zip compressor: cannot size the scratch for {n_max} values")
        self.scratch = torch.zeros(self.scratch_bytes, dtype=torch.uint8, device=device)
        self.codes = torch.zeros(self.code_stride, dtype=torch.uint8, device=device)
        self.splits = torch.zeros(self.table_len, dtype=torch.float32, device=device)
        self.mids = torch.zeros(self.table_len, dtype=torch.float32, device=device)
        self.meta = torch.zeros(4, dtype=torch.int32, device=device)
        self.range = torch.zeros(2, dtype=torch.float32, device=device)
        if world > 1:
            self.all_codes = torch.zeros((world, self.code_stride), dtype=torch.uint8, device=device)
            self.all_mids = torch.zeros((world, self.table_len), dtype=torch.float32, device=device)

    def pack(self, vals: torch.Tensor, n: torch.Tensor) -> None:
        """vals[:n] -> self.codes, self.mids, self.meta (n: device int64 scalar / 1-element view)."""
        L.check(self.lib.skml_zipml_pack(L.ptr(vals), L.ptr(n), self.n_max, self.bin_num, L.ptr(self.scratch),
                                         self.scratch_bytes, L.ptr(self.splits), L.ptr(self.mids), L.ptr(self.meta),
                                         L.ptr(self.range), L.ptr(self.codes), L.stream()), "skml_zipml_pack")
        L.count_launches(4)

    def unpack(self, keys, codes: torch.Tensor, mids: torch.Tensor, counts: torch.Tensor, lists: int,
               acc: torch.Tensor = None, vals_out: torch.Tensor = None) -> None:
        L.check(self.lib.skml_zipml_unpack_scatter(L.ptr(acc), L.ptr(keys), L.ptr(codes), L.ptr(mids), L.ptr(counts),
                                                   self.n_max, self.code_stride, lists, self.bin_num, L.ptr(vals_out),
                                                   L.stream()), "skml_zipml_unpack_scatter")
        L.count_launches(lists)

    def roundtrip(self, vals: torch.Tensor, n: torch.Tensor) -> None:
        """In place on vals[:n]: every value is replaced by the midpoint of its bucket."""
        self.pack(vals, n)
        self.unpack(None, self.codes, self.mids, n, 1, vals_out=vals)

    def wire_bytes(self, n: int) -> int:
        """Bytes one rank contributes for n non-zeros: raw keys, codes, the midpoint table and the count."""
        return 4 * n + n * self.code_bytes + 4 * self.table_len + 8
