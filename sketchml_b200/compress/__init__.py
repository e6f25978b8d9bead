"""Stand-alone compression library (the counterpart of the reference's Spark-free
``sketch`` module): quantizers, quantile sketch, MinMaxSketch, key encoders, Huffman
coder and the two ``VectorCompressor`` implementations."""
from . import oracle  # noqa: F401
from .api import (QuantizationType, Quantizer, QuantileQuantizer, UniformQuantizer, ZipMLQuantizer,  # noqa: F401
                  HeapQuantileSketch, MinMaxSketch, GroupedMinMaxSketch, DeltaBinaryEncoder,
                  DeltaAdaptiveEncoder, HuffmanEncoder, VectorCompressor, SparseVectorCompressor,
                  DenseVectorCompressor, Parallel, sizeof)
