"""Run configuration: one dataclass, an argparse CLI with the reference's option
names, and a parser for verbatim ``spark.sketchml.*=value`` pairs.

Reference: ml/conf/MLConf.scala:10-81 (keys, defaults, validation) and
ml/common/Constants.scala:4-14 (enumerations). Options without a counterpart
there are marked "new".
"""
from __future__ import annotations

import argparse
import dataclasses
import math
from dataclasses import dataclass, field
from typing import Iterable, Optional

# ml/common/Constants.scala:4-14
ML_LOGISTIC_REGRESSION = "LogisticRegression"
ML_SUPPORT_VECTOR_MACHINE = "SupportVectorMachine"
ML_LINEAR_REGRESSION = "LinearRegression"
ALGOS = (ML_LOGISTIC_REGRESSION, ML_SUPPORT_VECTOR_MACHINE, ML_LINEAR_REGRESSION)
ALGO_ALIASES = {
    "lr": ML_LOGISTIC_REGRESSION, "logistic": ML_LOGISTIC_REGRESSION,
    "svm": ML_SUPPORT_VECTOR_MACHINE, "linreg": ML_LINEAR_REGRESSION,
    "linear": ML_LINEAR_REGRESSION, "leastsquares": ML_LINEAR_REGRESSION,
}
FORMAT_LIBSVM, FORMAT_CSV, FORMAT_DUMMY, FORMAT_SYNTHETIC = "libsvm", "csv", "dummy", "synthetic"
FORMATS = (FORMAT_LIBSVM, FORMAT_CSV, FORMAT_DUMMY, FORMAT_SYNTHETIC)
COMPRESSOR_SKETCH, COMPRESSOR_FIXED_POINT, COMPRESSOR_ZIP = "Sketch", "FixedPoint", "Zip"
COMPRESSOR_FLOAT, COMPRESSOR_NONE = "Float", "None"
COMPRESSORS = (COMPRESSOR_SKETCH, COMPRESSOR_FIXED_POINT, COMPRESSOR_ZIP, COMPRESSOR_FLOAT, COMPRESSOR_NONE)

# spark.sketchml.<key> -> field name (ml/conf/MLConf.scala:10-45)
SPARK_KEYS = {
    "algo": "algo", "input.path": "input", "input.format": "format", "worker.num": "worker_num",
    "feature.num": "feature_num", "valid.ratio": "valid_ratio", "epoch.num": "epoch_num",
    "batch.sample.ratio": "batch_sample_ratio", "learn.rate": "learn_rate", "learn.decay": "learn_decay",
    "reg.l1": "l1_reg", "reg.l2": "l2_reg", "gradient.compressor": "compressor",
    "quantization.bin.num": "quant_bin_num", "minmaxsketch.group.num": "sketch_group_num",
    "minmaxsketch.row.num": "sketch_row_num", "minmaxsketch.col.ratio": "sketch_col_ratio",
    "fixed.point.bit.num": "fixed_point_bit_num",
}


@dataclass
class MLConf:
    # required in the reference
    algo: str = ML_LOGISTIC_REGRESSION
    input: str = ""
    format: str = FORMAT_LIBSVM
    worker_num: int = 1
    feature_num: int = 0
    # defaults of the reference
    valid_ratio: float = 0.25
    epoch_num: int = 100
    batch_sample_ratio: float = 0.1
    learn_rate: float = 0.1
    learn_decay: float = 0.9
    l1_reg: float = 0.1
    l2_reg: float = 0.1
    compressor: str = COMPRESSOR_SKETCH
    quant_bin_num: int = 256
    sketch_group_num: int = 8
    sketch_row_num: int = 2
    sketch_col_ratio: float = 0.3
    fixed_point_bit_num: int = 8
    # new options
    optimizer: str = "sgd"              # "sgd" | "adam" (the reference always builds Adam)
    key_encoder: str = "delta_binary"   # "delta_binary" | "delta_adaptive"
    cell_bits: int = -1                 # -1 auto (8/16), 32 raw ints, 0 Huffman-coded tables
    sketch_k: int = 128
    seed: int = 0
    dtype: str = "float32"              # "float32" on GPUs, "float64" for the CPU plumbing run
    device: str = "auto"                # "auto" | "cpu" | "cuda"
    pipeline_depth: int = 0             # 0 = exact synchronous steps, 1 = gradient one step stale
    recompress_sum: bool = False        # CPU only: second lossy step on the summed gradient
    neg_y: Optional[bool] = None        # None: +-1 labels for LR/SVM, raw targets for regression
    hot_columns: int = 8192             # columns [0, hot) accumulate in shared memory
    log_every: int = 0                  # batches between host-side loss reads (0 = once per epoch)
    checkpoint_dir: str = ""
    checkpoint_every: int = 0           # epochs between checkpoints (0 = never)
    resume: str = ""
    export_path: str = ""
    metrics_path: str = ""
    exchange: str = "auto"              # "auto" | "p2p" | "nccl" | "gloo"
    step_timeout_s: float = 1.0         # bound of every device-side wait
    # synthetic data (format == "synthetic")
    syn_rows: int = 100000
    syn_nnz_per_row: int = 20
    syn_zipf_s: float = 1.1
    syn_values: str = "binary"          # "binary" | "uniform_l2" | "normal"
    syn_wstar_density: float = 0.1
    syn_noise: float = 0.0
    extras: dict = field(default_factory=dict)

    def __post_init__(self):
        self.algo = ALGO_ALIASES.get(str(self.algo).lower(), self.algo)
        self.validate()

    # ml/conf/MLConf.scala:75-81
    def validate(self) -> None:
        if self.algo not in ALGOS:
            raise ValueError(f"Unrecognizable algorithm: {self.algo}")
        if self.format not in FORMATS:
            raise ValueError(f"Unrecognizable file format: {self.format}")
        if self.compressor not in COMPRESSORS:
            raise ValueError(f"Unrecognizable gradient compressor: {self.compressor}")
        if self.optimizer not in ("sgd", "adam"):
            raise ValueError(f"Unrecognizable optimizer: {self.optimizer}")
        if self.key_encoder not in ("delta_binary", "delta_adaptive"):
            raise ValueError(f"Unrecognizable key encoder: {self.key_encoder}")
        if not (0.0 <= self.valid_ratio < 1.0):
            raise ValueError("valid ratio must be in [0, 1)")
        if not (0.0 < self.batch_sample_ratio <= 1.0):
            raise ValueError("batch sample ratio must be in (0, 1]")
        if not (1 <= self.sketch_row_num <= 8):
            raise ValueError("Currently only 8 hash functions are available")
        if not (1 <= self.sketch_group_num <= 32):
            raise ValueError("minmaxsketch group num must be in [1, 32]")
        if not (2 <= self.quant_bin_num <= 65536):
            raise ValueError("quantization bin num must be in [2, 65536]")
        if self.sketch_col_ratio <= 0:
            raise ValueError("minmaxsketch col ratio must be positive")
        if self.fixed_point_bit_num >= 30 or self.fixed_point_bit_num < 2:
            raise ValueError(f"Bit num out of range: {self.fixed_point_bit_num}")
        if self.sketch_k < 1 or self.sketch_k >= 65535 or self.sketch_k & (self.sketch_k - 1):
            raise ValueError("sketch k must be a power of two below 65535")
        if self.pipeline_depth not in (0, 1):
            raise ValueError("pipeline depth must be 0 or 1")
        if self.dtype not in ("float32", "float64"):
            raise ValueError("dtype must be float32 or float64")

    @property
    def batch_num(self) -> int:
        """Batches per epoch (ml/objective/GradientDescent.scala:21)."""
        return int(math.ceil(1.0 / self.batch_sample_ratio))

    @property
    def use_neg_y(self) -> bool:
        if self.neg_y is not None:
            return self.neg_y
        return self.algo != ML_LINEAR_REGRESSION

    def sketch_options(self, step: int = 0, rank: int = 0, world: int = 1) -> dict:
        return dict(
            bin_num=self.quant_bin_num, group_num=self.sketch_group_num, row_num=self.sketch_row_num,
            col_ratio=self.sketch_col_ratio, key_encoder=0 if self.key_encoder == "delta_binary" else 1,
            cell_bits=self.cell_bits, sketch_k=self.sketch_k, seed=self.seed, step=step, rank=rank,
            world=world,
        )

    def to_dict(self) -> dict:
        return dataclasses.asdict(self)

    @classmethod
    def from_dict(cls, d: dict) -> "MLConf":
        names = {f.name for f in dataclasses.fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in names})

    @classmethod
    def from_spark_pairs(cls, pairs: Iterable[str], **overrides) -> "MLConf":
        """Accepts ``spark.sketchml.key=value`` strings as given to spark-submit --conf."""
        kw = {}
        types = {f.name: f.type for f in dataclasses.fields(cls)}
        for p in pairs:
            if "=" not in p:
                raise ValueError(f"expected key=value, got {p!r}")
            k, v = p.split("=", 1)
            k = k.strip()
            if k.startswith("spark.sketchml."):
                k = k[len("spark.sketchml."):]
            if k not in SPARK_KEYS:
                raise KeyError(f"unknown option spark.sketchml.{k}")
            name = SPARK_KEYS[k]
            kw[name] = _coerce(types[name], v.strip())
        kw.update(overrides)
        return cls(**kw)


def _coerce(tp, v: str):
    tp = str(tp)
    if "int" in tp:
        return int(v)
    if "float" in tp:
        return float(v)
    if "bool" in tp:
        return v.lower() in ("1", "true", "yes")
    return v


def add_arguments(p: argparse.ArgumentParser) -> None:
    d = MLConf()
    p.add_argument("--conf", action="append", default=[], metavar="spark.sketchml.K=V",
                   help="reference-style option, may be repeated")
    for f in dataclasses.fields(MLConf):
        if f.name == "extras":
            continue
        flag = "--" + f.name.replace("_", "-")
        default = getattr(d, f.name)
        if isinstance(default, bool) or f.name == "neg_y":
            p.add_argument(flag, type=lambda s: s.lower() in ("1", "true", "yes"), default=None)
        else:
            p.add_argument(flag, type=type(default), default=None)
    # aliases with the reference's dotted names spelled with dashes
    p.add_argument("--input-path", dest="input", default=None)
    p.add_argument("--input-format", dest="format", default=None)
    p.add_argument("--batch-sp-ratio", dest="batch_sample_ratio", type=float, default=None)
    p.add_argument("--quantization-bin-num", dest="quant_bin_num", type=int, default=None)
    p.add_argument("--minmaxsketch-group-num", dest="sketch_group_num", type=int, default=None)
    p.add_argument("--minmaxsketch-row-num", dest="sketch_row_num", type=int, default=None)
    p.add_argument("--minmaxsketch-col-ratio", dest="sketch_col_ratio", type=float, default=None)
    p.add_argument("--gradient-compressor", dest="compressor", default=None)
    p.add_argument("--reg-l1", dest="l1_reg", type=float, default=None)
    p.add_argument("--reg-l2", dest="l2_reg", type=float, default=None)


def conf_from_args(ns: argparse.Namespace) -> MLConf:
    names = {f.name for f in dataclasses.fields(MLConf)}
    over = {k: v for k, v in vars(ns).items() if k in names and v is not None}
    return MLConf.from_spark_pairs(getattr(ns, "conf", []) or [], **over)
