from .cast import (compose_mxfp_tensor, compose_mxfp_tensor_strided, extract_mxfp_components,  # noqa: F401
                   extract_mxfp_components_strided, quantize_dequantize, quantize_dequantize_strided)
