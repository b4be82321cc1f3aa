from . import functional, kernels, layers, meta  # noqa: F401
