"""Device versions of the two baseline value quantizers (torch ops on the GPU).

They turn the values of a sparse gradient into the values the reference's baseline
compressors would decode to, so that `compressor=FixedPoint` and `compressor=Zip` train on
GPUs with the same numerics as on the host engine. Keys travel raw, as in the reference
(ml/gradient/FixedPointGradient.scala:27-30, ml/gradient/ZipGradient.scala:27-30); the
values are exchanged dequantized (fp32) through the raw key/value all-gather path, so the
byte saving of the packed codes is not realised on the wire here.

Reference: ml/gradient/FixedPointGradient.scala:39-75 (sign + (b-1)-bit magnitude of
floor(|v| / ||v||_2 * max) + Bernoulli(1/2)), ml/gradient/ZipGradient.scala:70-129 (sorted
values, prefix sums of v and v^2, repeated halving of the split candidates keeping the
bin_num/2 adjacent pairs with the largest squared error, bucket midpoints as decode values).
"""
from __future__ import annotations

import torch


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
