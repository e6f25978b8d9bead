"""sketchml_b200: distributed minibatch training of sparse linear models with
sketch-compressed gradient exchange, written for NVIDIA B200 (sm_100a)."""

__version__ = "0.1.0"
