from . import functional, helpers, kernels, layers, meta  # noqa: F401
