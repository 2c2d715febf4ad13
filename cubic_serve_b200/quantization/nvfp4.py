"""NVFP4 helpers (thin alias module so call sites read ``nvfp4.quantize``)."""
from .formats import nvfp4_activation_quantize as activation_quantize  # noqa: F401
from .formats import nvfp4_dense as dense  # noqa: F401
from .formats import nvfp4_quantize as quantize  # noqa: F401
