from .cast import compose_minifloat_component, extract_minifloat_component, quantize_dequantize  # noqa: F401
