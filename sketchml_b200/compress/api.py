"""Object API over the C++ oracle, shaped like the reference's public classes.

Reference: base/VectorCompressor.java:9-27, base/Quantizer.java:21-152,
base/QuantileSketch.java:22-32, base/BinaryEncoder.java:6-10,
sample/SparseVectorCompressor.java:52-147, sample/DenseVectorCompressor.java:34-116,
sketch/frequency/GroupedMinMaxSketch.java:35-146, common/Constants.java:9-42,
util/Utils.java:6-15.
"""
from __future__ import annotations

import enum
from typing import Optional, Sequence

import numpy as np

from . import oracle


def sizeof(obj) -> int:
    """Wire size in bytes (the reference measures Java-serialized length, Utils.java:6-15)."""
    if isinstance(obj, (bytes, bytearray)):
        return len(obj)
    if hasattr(obj, "nbytes_wire"):
        return obj.nbytes_wire()
    raise TypeError("object has no wire form")


class Parallel:
    """Process-wide parallelism of the CPU library (common/Constants.java:9-42): the number of
    threads the ``parallel_*`` methods hand to the C++ library, which then summarises the values in
    per-thread quantile sketches that are merged (quantization/QuantileQuantizer.java:53-92), looks
    the buckets up slice by slice, and builds the groups' sketches and key codes on a thread per
    share of groups (sketch/frequency/GroupedMinMaxSketch.java:72-101). On a GPU the parallel
    decomposition is the kernel grid instead."""
    _parallelism = 1

    @classmethod
    def set_parallelism(cls, n: int) -> None:
        if n < 1:
            raise oracle.SketchMLError("parallelism must be positive")
        cls._parallelism = int(n)

    @classmethod
    def get_parallelism(cls) -> int:
        return cls._parallelism

    @classmethod
    def shutdown(cls) -> None:
        cls._parallelism = 1


class QuantizationType(enum.Enum):
    UNIFORM = "uniform"
    QUANTILE = "quantile"
    ZIPML = "zipml"


class Quantizer:
    DEFAULT_BIN_NUM = 256
    quantization_type = None

    def __init__(self, bin_num: int = DEFAULT_BIN_NUM):
        self.bin_num = int(bin_num)
        self.n = 0
        self.splits = None
        self.zero_idx = 0
        self.min = 0.0
        self.max = 0.0
        self.bins = None
        self._values = None

    def _take(self, q: dict, n: int) -> None:
        self.bin_num, self.zero_idx = q["bin_num"], q["zero_idx"]
        self.min, self.max = q["min"], q["max"]
        self.splits, self.bins, self._values = q["splits"], q["bins"], q["values"]
        self.n = n

    def quantize(self, values) -> None:
        raise NotImplementedError

    def parallel_quantize(self, values) -> None:
        self.quantize(values)

    def get_values(self) -> np.ndarray:
        return self._values

    def get_bins(self) -> np.ndarray:
        return self.bins

    def get_zero_idx(self) -> int:
        return self.zero_idx

    def get_bin_num(self) -> int:
        return self.bin_num

    def index_of(self, x: float) -> int:
        return int(np.searchsorted(self.splits, x, side="right"))

    def times_by(self, x: float) -> None:
        self.min *= x
        self.max *= x
        self.splits = self.splits * x
        self._values = self._values * x

    def nbytes_wire(self) -> int:
        code = 1 if self.bin_num <= 256 else (2 if self.bin_num <= 65536 else 4)
        return 4 + 4 + 8 * (self.bin_num - 1) + 4 + 16 + 4 + code * len(self.bins)

    def to_java_stream(self) -> bytes:
        return oracle.export_java_quantizer(np.asarray(self.splits, np.float64), self.min, self.max,
                                            np.asarray(self._source, np.float64))

    @staticmethod
    def new_quantizer(kind: QuantizationType, bin_num: int) -> "Quantizer":
        return {QuantizationType.QUANTILE: QuantileQuantizer, QuantizationType.UNIFORM: UniformQuantizer,
                QuantizationType.ZIPML: ZipMLQuantizer}[kind](bin_num)


class QuantileQuantizer(Quantizer):
    quantization_type = QuantizationType.QUANTILE

    def __init__(self, bin_num=Quantizer.DEFAULT_BIN_NUM, k: int = 128, seed: int = 0, offset_mode: int = 2,
                 java_compat_max: bool = False):
        super().__init__(bin_num)
        self.k, self.seed, self.offset_mode, self.java_compat_max = k, seed, offset_mode, java_compat_max

    def quantize(self, values) -> None:
        v = np.ascontiguousarray(values)
        self._source = v
        self._take(oracle.quantile_quantize(v, self.bin_num, self.k, self.seed, self.offset_mode,
                                            self.java_compat_max), len(v))

    def parallel_quantize(self, values) -> None:
        """One sketch per thread over a slice of the values, merged before the splits are queried;
        the buckets are looked up in parallel (QuantileQuantizer.java:53-92)."""
        v = np.ascontiguousarray(values)
        self._source = v
        self._take(oracle.quantile_quantize(v, self.bin_num, self.k, self.seed, self.offset_mode,
                                            self.java_compat_max, Parallel.get_parallelism()), len(v))


class UniformQuantizer(Quantizer):
    quantization_type = QuantizationType.UNIFORM

    def quantize(self, values) -> None:
        v = np.ascontiguousarray(values, dtype=np.float64)
        self._source = v
        self._take(oracle.uniform_quantize(v, self.bin_num), len(v))


class ZipMLQuantizer(Quantizer):
    quantization_type = QuantizationType.ZIPML

    def quantize(self, values) -> None:
        v = np.ascontiguousarray(values, dtype=np.float64)
        self._source = v
        self._take(oracle.zipml_quantize(v, self.bin_num), len(v))


class HeapQuantileSketch:
    DEFAULT_K = 128

    def __init__(self, k: int = DEFAULT_K, seed: int = 0, offset_mode: int = 2, java_compat_max: bool = False):
        self._s = oracle.QuantileSketch(k, seed, offset_mode, java_compat_max)

    def reset(self):
        self._s.reset()

    def update(self, value) -> None:
        self._s.update(np.atleast_1d(np.asarray(value, dtype=np.float64)))

    def merge(self, other: "HeapQuantileSketch") -> None:
        self._s.merge(other._s)

    def get_quantiles(self, even_partition: int) -> np.ndarray:
        return self._s.quantiles(int(even_partition))

    def get_quantile(self, fraction: float) -> float:
        if not (0.0 <= fraction <= 1.0):
            raise oracle.SketchMLError("Fraction should be in range [0.0, 1.0]")
        if self.n == 0:
            return float("nan")
        if fraction == 0.0:
            return self.min_value
        if fraction == 1.0:
            return self.max_value
        samples, cum = self._s.summary()
        rank = min(int(self.n * fraction), self.n - 1)
        return float(samples[np.searchsorted(cum, rank, side="right") - 1])

    n = property(lambda self: self._s.n)
    min_value = property(lambda self: self._s.min)
    max_value = property(lambda self: self._s.max)
    k = property(lambda self: self._s.k)
    is_empty = property(lambda self: self._s.n == 0)


class MinMaxSketch:
    DEFAULT_ROW_NUM = 2

    def __init__(self, row_num: int, col_num: int, zero_value: int, hash_ids: Optional[Sequence[int]] = None,
                 seed: int = 0, tie_mode: int = 0):
        ids = list(hash_ids) if hash_ids is not None else oracle.pick_hashes(seed, 0, 0, 0, row_num)
        self._s = oracle.MinMaxSketch(row_num, col_num, zero_value, ids, tie_mode)
        self.row_num, self.col_num, self.zero_value, self.hash_ids = row_num, col_num, zero_value, ids

    def insert(self, key, value) -> None:
        self._s.insert(np.atleast_1d(np.asarray(key, np.int32)), np.atleast_1d(np.asarray(value, np.int32)))

    def query(self, key):
        r = self._s.query(np.atleast_1d(np.asarray(key, np.int32)))
        return int(r[0]) if np.isscalar(key) else r

    @property
    def table(self) -> np.ndarray:
        return self._s.table


class _Encoder:
    def __init__(self):
        self.code = None

    def decode(self) -> np.ndarray:
        raise NotImplementedError

    def nbytes_wire(self) -> int:
        return 4 + 4 + 8 * len(self.code["flag_words"]) + 4 + 8 * len(self.code["delta_words"])


class DeltaBinaryEncoder(_Encoder):
    def encode(self, values) -> None:
        self.code = oracle.delta_binary_encode(np.asarray(values, np.int32))

    def decode(self):
        return oracle.delta_binary_decode(self.code)


class DeltaAdaptiveEncoder(_Encoder):
    def encode(self, values) -> None:
        self.code = oracle.delta_adaptive_encode(np.asarray(values, np.int32))

    def decode(self):
        return oracle.delta_adaptive_decode(self.code)

    def nbytes_wire(self):
        return super().nbytes_wire() + 5


class HuffmanEncoder(_Encoder):
    def encode(self, values) -> None:
        self.code = oracle.huffman_encode(np.asarray(values, np.int32))

    def decode(self):
        return oracle.huffman_decode(self.code)

    def nbytes_wire(self):
        return 4 + 12 * len(self.code["items"]) + 4 + 8 * len(self.code["words"]) + 4


class GroupedMinMaxSketch:
    DEFAULT_GROUP_NUM = 8
    DEFAULT_COL_RATIO = 0.3

    def __init__(self, group_num=DEFAULT_GROUP_NUM, row_num=MinMaxSketch.DEFAULT_ROW_NUM,
                 col_ratio=DEFAULT_COL_RATIO, bin_num=256, zero_value=0, key_encoder="delta_adaptive",
                 seed: int = 0, cell_bits: int = -1):
        self.opts = dict(group_num=group_num, row_num=row_num, col_ratio=col_ratio, bin_num=bin_num,
                         key_encoder=0 if key_encoder == "delta_binary" else 1, seed=seed, cell_bits=cell_bits)
        self.bin_num, self.zero_value = bin_num, zero_value
        self.payload = None

    def create(self, keys, bins, threads: int = 1) -> None:
        """Builds the per-group sketches and key codes from (key, bucket) pairs. The
        buckets are passed through a quantizer whose splits are the integers
        0.5, 1.5, ... so that bucket b decodes to b."""
        keys = np.asarray(keys, np.int32)
        bins = np.asarray(bins, np.float64)
        splits = np.arange(self.bin_num - 1, dtype=np.float64) + 0.5
        self._splits = splits
        self.payload = self._build(keys, bins, splits, threads)

    def _build(self, keys, bins, splits, threads: int = 1):
        # zero_idx is derived from the splits by the oracle: shift so that bucket
        # `zero_value` is the first with split >= 0.
        shift = self.zero_value
        return oracle.compress_sparse(keys, bins - shift, int(keys.max()) + 1 if len(keys) else 1,
                                      dict(self.opts, threads=int(threads)),
                                      splits - shift, float(-shift - 0.5), float(self.bin_num - shift - 0.5))

    def parallel_create(self, keys, bins) -> None:
        """The same payload, with the groups' sketches and key codes built on `Parallel.get_parallelism()`
        threads (GroupedMinMaxSketch.java:72-101)."""
        self.create(keys, bins, threads=Parallel.get_parallelism())

    def restore(self):
        p = oracle.parse(self.payload)
        ks, bs = [], []
        for g in p["groups"]:
            if g["n"] == 0:
                continue
            dec = oracle.delta_binary_decode if p["key_encoder"] == 0 else oracle.delta_adaptive_decode
            k = dec(g["keys"])
            sk = oracle.MinMaxSketch(p["row_num"], g["col_num"], p["zero_idx"], g["hash_ids"][:p["row_num"]], 1)
            # rebuild from the stored table
            t = g["table"]
            b = np.full(len(k), p["zero_idx"], np.int32)
            for r in range(p["row_num"]):
                c = t[r * g["col_num"] + oracle.hash(g["hash_ids"][r], k, g["col_num"])]
                far = np.abs(c - p["zero_idx"]) > np.abs(b - p["zero_idx"])
                b = np.where(far, c, b).astype(np.int32)
            ks.append(list(k))
            bs.append(list(b))
        return oracle.kway_merge(ks, bs)

    def nbytes_wire(self):
        return len(self.payload)


class VectorCompressor:
    """base/VectorCompressor.java:9-27."""

    def compress_dense(self, values) -> None:
        raise NotImplementedError

    def compress_sparse(self, keys, values) -> None:
        raise NotImplementedError

    def parallel_compress_dense(self, values) -> None:
        self.compress_dense(values)

    def parallel_compress_sparse(self, keys, values) -> None:
        self.compress_sparse(keys, values)

    def decompress_dense(self) -> np.ndarray:
        raise NotImplementedError

    def decompress_sparse(self):
        raise NotImplementedError

    def times_by(self, x: float) -> None:
        raise NotImplementedError

    def size(self) -> int:
        raise NotImplementedError

    def memory_bytes(self) -> int:
        raise NotImplementedError


class SparseVectorCompressor(VectorCompressor):
    def __init__(self, quant_type=QuantizationType.QUANTILE, quant_bin_num=256, group_num=8, row_num=2,
                 col_ratio=0.3, key_encoder="delta_adaptive", cell_bits=0, seed=0, dtype=np.float64):
        if quant_type is not QuantizationType.QUANTILE:
            raise oracle.SketchMLError("the sketch compressor uses the quantile quantizer")
        self.opts = dict(bin_num=quant_bin_num, group_num=group_num, row_num=row_num, col_ratio=col_ratio,
                         key_encoder=0 if key_encoder == "delta_binary" else 1, cell_bits=cell_bits, seed=seed)
        self.dtype = dtype
        self.payload = None
        self._size = 0

    def compress_sparse(self, keys, values) -> None:
        keys = np.asarray(keys, np.int32)
        values = np.asarray(values, self.dtype)
        if len(keys) != len(values):
            raise oracle.SketchMLError(
                f"Lengths of key array and value array do not match: {len(keys)}, {len(values)}")
        self._size = len(keys)
        dim = int(keys.max()) + 1 if len(keys) else 1
        self.payload = oracle.compress_sparse(keys, values, dim, dict(self.opts, threads=self._threads))

    _threads = 1

    def parallel_compress_sparse(self, keys, values) -> None:
        """Per-thread quantile sketches merged into one, buckets looked up in parallel, one thread per
        share of bucket groups (sample/SparseVectorCompressor.java parallelCompressSparse)."""
        self._threads = Parallel.get_parallelism()
        try:
            self.compress_sparse(keys, values)
        finally:
            self._threads = 1

    def parallel_compress_dense(self, values) -> None:
        values = np.asarray(values, self.dtype)
        self.parallel_compress_sparse(np.arange(len(values), dtype=np.int32), values)

    def compress_dense(self, values) -> None:
        values = np.asarray(values, self.dtype)
        self.compress_sparse(np.arange(len(values), dtype=np.int32), values)

    def decompress_sparse(self):
        _, k, v = oracle.decompress(self.payload)
        return k, v

    def decompress_dense(self) -> np.ndarray:
        return self.decompress_sparse()[1]

    def times_by(self, x):
        self.payload = oracle.payload_times_by(self.payload, float(x))

    def size(self):
        return self._size

    def memory_bytes(self):
        return len(self.payload)

    def to_java_stream(self) -> bytes:
        return oracle.export_java_fields(self.payload)


class DenseVectorCompressor(VectorCompressor):
    def __init__(self, quant_type=QuantizationType.QUANTILE, quant_bin_num=256, seed=0):
        self.quant_type, self.bin_num, self.seed = quant_type, quant_bin_num, seed
        self.q = None
        self._size = 0
        self._keys = None

    def compress_dense(self, values, parallel: bool = False) -> None:
        self.q = Quantizer.new_quantizer(self.quant_type, self.bin_num)
        if isinstance(self.q, QuantileQuantizer):
            self.q.seed = self.seed
        (self.q.parallel_quantize if parallel else self.q.quantize)(np.asarray(values, np.float64))
        self._size = len(values)
        self._keys = None

    def parallel_compress_dense(self, values) -> None:
        """sample/DenseVectorCompressor.java parallelCompressDense: the quantizer's parallel form."""
        self.compress_dense(values, parallel=True)

    def parallel_compress_sparse(self, keys, values) -> None:
        keys = np.asarray(keys, np.int32)
        dense = np.zeros(int(keys.max()) + 1 if len(keys) else 0)
        dense[keys] = values
        self.compress_dense(dense, parallel=True)

    def compress_sparse(self, keys, values) -> None:
        keys = np.asarray(keys, np.int32)
        dense = np.zeros(int(keys.max()) + 1 if len(keys) else 0)  # the reference allocates maxKey (one short)
        dense[keys] = values
        self.compress_dense(dense)

    def decompress_dense(self) -> np.ndarray:
        return self.q.get_values()[self.q.get_bins()]

    def decompress_sparse(self):
        v = self.decompress_dense()
        return np.arange(len(v), dtype=np.int32), v

    def times_by(self, x):
        self.q.times_by(x)

    def size(self):
        return self._size

    def memory_bytes(self):
        return 12 + self.q.nbytes_wire()
