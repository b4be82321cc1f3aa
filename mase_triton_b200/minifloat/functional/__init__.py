from .cast import compose_minifloat_component, extract_minifloat_component, quantize_dequantize  # noqa: F401
from .linear import minifloat_linear  # noqa: F401
from .matmul import minifloat_matmul  # noqa: F401
