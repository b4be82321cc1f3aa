"""``minifloat_linear`` (reference: ``src/mase_triton/minifloat/functional/linear.py:108-171``).

Per-tensor (un-blocked) fake quantisation of activation, weight and bias followed by a
dense linear.  ``layer_type`` names what is quantised (``Xq``/``X``, ``Wq``/``W``, ``Bq``/``B``).
Both backends give the same values: ``"separate"`` mirrors the reference's op sequence,
``"fused"`` (a stub in the reference) is accepted and runs the same kernels.
"""

from __future__ import annotations

from typing import Literal

import torch
from torch import Tensor

from ..._linear_common import check_backend, parse_layer_type
from ..meta import MinifloatMeta, MinifloatTensorMeta
from .cast import compose_minifloat_component, quantize_dequantize


def minifloat_linear(
    x: Tensor,
    x_meta: MinifloatMeta | None,
    w: Tensor | None,
    w_element: Tensor | None,
    w_tensor_meta: MinifloatTensorMeta | None,
    b: Tensor | None,
    b_element: Tensor | None,
    b_tensor_meta: MinifloatTensorMeta | None,
    layer_type: Literal["XWB", "XWBq", "XWqB", "XWqBq", "XqWB", "XqWBq", "XqWqB", "XqWqBq"],
    backend: Literal["separate", "fused"],
) -> Tensor:
    kind = parse_layer_type(layer_type)
    check_backend(backend)
    if kind.x_quantised:
        x = quantize_dequantize(x, x_meta)                      # same bits as extract + compose
    weight = compose_minifloat_component(w_element, w_tensor_meta) if kind.w_quantised else w
    if kind.b_quantised:
        # a quantised-bias layer ignores a plain bias unless codes for it exist
        bias = compose_minifloat_component(b_element, b_tensor_meta) if b is not None else None
    else:
        bias = b
    return torch.nn.functional.linear(x, weight, bias)
