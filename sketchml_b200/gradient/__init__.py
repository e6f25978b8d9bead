"""Gradient containers and the compressor factory."""
from .kinds import (Kind, Gradient, ZeroGradient, DenseDoubleGradient, SparseDoubleGradient,  # noqa: F401
                    DenseFloatGradient, SparseFloatGradient, SketchGradient, FixedPointGradient,
                    ZipGradient, compress, sum_gradients, evaluate_compression)
