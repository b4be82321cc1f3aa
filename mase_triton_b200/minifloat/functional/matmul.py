"""``minifloat_matmul`` (reference: ``src/mase_triton/minifloat/functional/matmul.py:10-35``)."""

from __future__ import annotations

from typing import Literal

import torch
from torch import Tensor

from ..._linear_common import check_backend
from ..meta import MinifloatMeta
from .cast import quantize_dequantize


def minifloat_matmul(
    input: Tensor,
    other: Tensor,
    input_meta: MinifloatMeta | None,
    other_meta: MinifloatMeta | None,
    func_type: Literal["XW", "XqW", "XWq", "XqWq"],
    backend: Literal["separate", "fused"],
) -> Tensor:
    """``torch.matmul`` on operands fake-quantised per ``func_type`` (batched operands allowed)."""
    check_backend(backend)
    if "Xq" in func_type:
        assert input_meta is not None
        input = quantize_dequantize(input, input_meta)
    if "Wq" in func_type:
        assert other_meta is not None
        other = quantize_dequantize(other, other_meta)
    return torch.matmul(input, other)
