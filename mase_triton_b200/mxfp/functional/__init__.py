from .cast import (  # noqa: F401
    compose_mxfp_tensor,
    extract_mxfp_components,
    extract_mxfp_tensor,
    flatten_for_quantize,
    permute_for_dequantize,
    quantize_dequantize,
)
from .linear import mxfp_linear, parse_mxfp_linear_type  # noqa: F401
from .matmul import mxfp_matmul  # noqa: F401
