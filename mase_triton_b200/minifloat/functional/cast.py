"""Public minifloat casts (reference: ``src/mase_triton/minifloat/functional/cast.py:10-90``)."""

from __future__ import annotations

import torch
from torch import Tensor

from .. import kernels
from ..meta import MinifloatMeta, MinifloatTensorMeta


def extract_minifloat_component(tensor: Tensor, minifloat_meta: MinifloatMeta) -> tuple[Tensor, MinifloatTensorMeta]:
    """Quantise ``tensor`` to minifloat codes.

    Returns ``(element, tensor_meta)``: ``element`` is a uint16 tensor shaped like the input,
    ``tensor_meta`` records the input's device, dtype and shape together with the format.
    """
    element = kernels.extract_minifloat_component(tensor, minifloat_meta)
    tensor_meta = MinifloatTensorMeta(device=tensor.device, dtype=tensor.dtype, shape=tensor.shape, meta=minifloat_meta)
    return element, tensor_meta


def compose_minifloat_component(element: Tensor, tensor_meta: MinifloatTensorMeta,
                                output_dtype: torch.dtype | None = None) -> Tensor:
    """Dequantise codes; ``output_dtype`` defaults to the dtype recorded in ``tensor_meta``."""
    if output_dtype is None:
        output_dtype = getattr(torch, tensor_meta.dtype)
    return kernels.compose_minifloat_component(element, tensor_meta.meta, output_dtype=output_dtype)


def quantize_dequantize(tensor: Tensor, minifloat_meta: MinifloatMeta, output_dtype: torch.dtype | None = None) -> Tensor:
    """``compose(extract(tensor))`` as a single fused kernel (8 B/element for fp32 instead of 12)."""
    return kernels.quantize_dequantize(tensor, minifloat_meta, tensor.dtype if output_dtype is None else output_dtype)
