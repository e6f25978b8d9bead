"""Device versions of the two baseline value quantizers.

FixedPoint: `FixedPointCodec` wraps the pack / unpack kernels (csrc/cuda/baseline_kernels.cu):
the b-bit codes are what travels between ranks (4 + b/8 bytes per non-zero), keys raw as in
the reference (ml/gradient/FixedPointGradient.scala:27-30). `fixed_point_roundtrip` is the
same arithmetic in torch ops, kept for the dense gradient kind.

Zip: `zipml_roundtrip` (torch ops) turns the values into the values the reference's ZipML
compressor would decode to (keys raw, ml/gradient/ZipGradient.scala:27-30); the values are
exchanged dequantized (fp32) through the raw key/value all-gather path, so the byte saving of
its packed codes is not realised on the wire.

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


def zipml_roundtrip(vals: torch.Tensor, n: torch.Tensor, bin_num: int) -> None:
    """In place on vals[:n]: every value is replaced by the midpoint of its ZipML bucket."""
    cnt = int(n.item())  # the halving loop is data dependent: this baseline synchronises
    if cnt == 0:
        return
    v = vals[:cnt].double()
    s, _ = torch.sort(v)
    r = torch.cumsum(s, 0)
    t = torch.cumsum(s * s, 0)
    idx = torch.arange(cnt, device=v.device)
    split_num = cnt
    while split_num > bin_num:
        pairs = split_num // 2
        L = idx[0:2 * pairs:2]
        nxt = torch.cat([idx[2:2 * pairs:2], idx.new_tensor([cnt])]) if 2 * pairs >= split_num else idx[2:2 * pairs + 1:2]
        R = nxt[:pairs] - 1
        rl = torch.where(L > 0, r[(L - 1).clamp_min(0)], torch.zeros_like(r[L]))
        tl = torch.where(L > 0, t[(L - 1).clamp_min(0)], torch.zeros_like(t[L]))
        l1, l2 = r[R] - rl, t[R] - tl
        m = (R - L + 1).double()
        mean = l1 / m
        err = l2 + mean * mean * m - 2 * mean * l1
        odd = split_num % 2
        thr_num = min(max(1, bin_num // 2 - odd), pairs)
        thr = torch.topk(err, thr_num).values[-1]
        keep_second = err >= thr
        # keep at most thr_num second halves (ties at the threshold are cut in index order)
        over = torch.cumsum(keep_second.long(), 0) > thr_num
        keep_second = keep_second & ~over
        firsts = idx[0:2 * pairs:2]
        seconds = idx[1:2 * pairs:2][keep_second]
        new = torch.sort(torch.cat([firsts, seconds] + ([idx[split_num - 1:split_num]] if odd else []))).values
        if new.numel() >= split_num:
            break
        idx = torch.cat([new, idx[new.numel():]])
        split_num = new.numel()
    splits = torch.unique_consecutive(s[idx[1:split_num]]) if split_num > 1 else s[:1]
    lo, hi = s[0], s[-1]
    edges = torch.cat([lo.view(1), splits, hi.view(1)])
    mids = 0.5 * (edges[:-1] + edges[1:])
    bins = torch.searchsorted(splits, v, right=True)
    vals[:cnt] = mids[bins].float()
