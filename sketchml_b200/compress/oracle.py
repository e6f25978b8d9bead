"""Loads (building on first use) the C++ CPU oracle and re-exports its functions."""
from __future__ import annotations

from .. import build as _build

_build.build_oracle()
from .._oracle import *  # noqa: F401,F403,E402
from .. import _oracle as _mod  # noqa: E402

SketchMLError = _mod.SketchMLError
KIND_EMPTY, KIND_SPARSE, KIND_DENSE = 0, 1, 2
