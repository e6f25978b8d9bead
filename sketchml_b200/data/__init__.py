"""Data layer: text parsers, the CSR row store with its cyclic minibatch cursor,
deterministic sharding / validation split, and synthetic generators."""
from .dataset import CSRMatrix, DataSet, split_train_valid, shard_rows  # noqa: F401
from .parser import load_data, parse_lines, parse_text_native, parse_libsvm, parse_csv, parse_dummy  # noqa: F401
from .synthetic import SyntheticSpec, generate_cpu  # noqa: F401
from .feeder import HostBatchFeeder, PinnedBatch  # noqa: F401
