"""Stand-alone demo of the compression library: a dense and a sparse vector are
compressed, decompressed and compared, printing error quantiles, RMSE and compression
rate against 8 B per dense value and 12 B per sparse non-zero.

Reference: sample/App.java:25-117 (``dense()``: 1M values of which 90 % are N(0,1) draws,
256 buckets; ``sparse()``: about 10 % of the dimensions non-zero, 256 buckets, 8 groups,
2 rows, column ratio 0.3)."""
from __future__ import annotations

import numpy as np

from .api import DenseVectorCompressor, HeapQuantileSketch, Parallel, QuantizationType, SparseVectorCompressor


def _report(name, before, after, raw_bytes, comp_bytes):
    err = np.abs(before - after)
    sk = HeapQuantileSketch()
    sk.update(err)
    q = sk.get_quantiles(10)
    rmse = float(np.sqrt(np.mean((before - after) ** 2)))
    print(f"[{name}] first values before: {np.array2string(before[:10], precision=5)}")
    print(f"[{name}] first values after : {np.array2string(after[:10], precision=5)}")
    print(f"[{name}] error deciles: {np.array2string(q, precision=6)}")
    print(f"[{name}] RMSE {rmse:.6g}; {raw_bytes} -> {comp_bytes} bytes, compression rate {raw_bytes / comp_bytes:.3f}")
    return {"rmse": rmse, "rate": raw_bytes / comp_bytes}


def dense(size: int = 1_000_000, seed: int = 0):
    rng = np.random.default_rng(seed)
    v = np.where(rng.random(size) < 0.9, rng.normal(size=size), 0.0)
    c = DenseVectorCompressor(QuantizationType.QUANTILE, 256, seed=seed)
    c.parallel_compress_dense(v)
    return _report("dense", v, c.decompress_dense(), 8 * size, c.memory_bytes())


def sparse(dim: int = 100_000, seed: int = 0):
    rng = np.random.default_rng(seed + 1)
    mask = rng.random(dim) < 0.1
    keys = np.nonzero(mask)[0].astype(np.int32)
    vals = rng.normal(size=len(keys))
    c = SparseVectorCompressor(QuantizationType.QUANTILE, 256, 8, 2, 0.3, seed=seed)
    c.parallel_compress_sparse(keys, vals)
    k2, v2 = c.decompress_sparse()
    if not np.array_equal(k2, keys):
        print("ERROR: decoded keys differ from the input keys")
    return _report("sparse", vals, v2, 12 * len(keys), c.memory_bytes())


def main(size: int = 1_000_000, seed: int = 0):
    Parallel.set_parallelism(4)
    d = dense(size, seed)
    s = sparse(max(size // 10, 1000), seed)
    Parallel.shutdown()
    return d, s


if __name__ == "__main__":
    main()
