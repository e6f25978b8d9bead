"""sm_100a kernels (libskml_cuda.so) and their Python wrappers."""
from . import lib  # noqa: F401
from .glm import DeviceCSR, GlmState, glm_grad, glm_validate, compact_gradient, update_dense, update_gathered, update_sparse  # noqa: F401
from .codec import GpuCompressor, GpuDecoder, ExchangeRegionView, read_status  # noqa: F401
from .datagen import generate_gpu  # noqa: F401
