"""Shadow check of the fused compress kernel: recompute a payload on the CPU oracle from the same
keys, values and split points and compare it with the bytes the GPU produced.

The GPU's quantile summary is its own design (only its rank-error behaviour is specified), so the
split points are taken from the launch being checked; everything downstream of them (bucket
values, zero bucket, group edges, hash choice, sketch tables, key flags and deltas, restart
points) must then match the oracle bit for bit. Used by `GpuEngine` when
`extras={"shadow_every": k}` is set, and by the tests.
"""
from __future__ import annotations

from typing import List

import numpy as np

HEADER_FIELDS = ("kind", "step", "rank", "world", "dim", "nnz", "bin_num", "zero_idx", "group_num", "row_num",
                 "col_ratio", "key_encoder", "cell_bits", "seed", "restart_interval")


class ShadowMismatch(RuntimeError):
    pass


def _group_fields(g):
    if not g["n"]:
        return (0,)
    return (g["n"], g["col_num"], tuple(g["hash_ids"]), g["table"].tolist(), g["keys"]["flag_words"].tolist(),
            g["keys"]["delta_words"].tolist(), g["restart_raw"].tolist())


_GROUP_FIELD_NAMES = ("n", "col_num", "hash_ids", "table", "flag_words", "delta_words", "restart")


def compare_payload(payload: bytes, keys: np.ndarray, vals: np.ndarray, dim: int, splits: np.ndarray,
                    group_num: int, row_num: int, col_ratio: float, seed: int) -> List[str]:
    """Returns the list of differences (empty = the payload equals the oracle's)."""
    from ..compress import oracle
    got = oracle.parse(payload)
    if got["kind"] != 1:
        return [] if len(keys) == 0 or got["kind"] == 2 else [f"kind {got['kind']} for {len(keys)} non-zeros"]
    opts = dict(bin_num=int(len(splits) + 1), group_num=int(group_num), row_num=int(row_num), col_ratio=float(col_ratio),
                seed=int(seed), step=int(got["step"]), rank=int(got["rank"]), world=int(got["world"]), tie_mode=1)
    ref_bytes = oracle.compress_sparse(np.ascontiguousarray(keys, dtype=np.int32), np.ascontiguousarray(vals, dtype=np.float32),
                                       int(dim), opts, np.ascontiguousarray(splits, dtype=np.float32),
                                       float(got["min_value"]), float(got["max_value"]))
    ref = oracle.parse(ref_bytes)
    diffs = [f"header field {k}: {got[k]} != {ref[k]}" for k in HEADER_FIELDS if got[k] != ref[k]]
    if not np.array_equal(got["bucket_values"], ref["bucket_values"]):
        diffs.append("bucket values differ")
    for gi, (a, b) in enumerate(zip(got["groups"], ref["groups"])):
        for name, x, y in zip(_GROUP_FIELD_NAMES, _group_fields(a), _group_fields(b)):
            if x != y:
                diffs.append(f"group {gi}: {name} differs")
    _, k2, _ = oracle.decompress(payload)
    if not np.array_equal(k2, keys):
        diffs.append("decoded keys differ from the gradient's keys")
    return diffs


def check_payload(*args, **kw) -> None:
    diffs = compare_payload(*args, **kw)
    if diffs:
        raise ShadowMismatch("GPU payload differs from the CPU oracle: " + "; ".join(diffs[:8]))
