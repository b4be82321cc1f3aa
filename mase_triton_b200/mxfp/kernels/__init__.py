from .cast import compose_mxfp_tensor, extract_mxfp_components, quantize_dequantize  # noqa: F401
