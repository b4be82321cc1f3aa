"""``mxfp_matmul`` (reference: ``src/mase_triton/mxfp/functional/matmul.py:10-35``)."""

from __future__ import annotations

from typing import Literal

import torch
from torch import Tensor

from ..._linear_common import check_backend
from ..meta import MXFPMeta
from .cast import quantize_dequantize


def mxfp_matmul(
    input: Tensor,
    other: Tensor,
    input_meta: MXFPMeta | None,
    other_meta: MXFPMeta | None,
    func_type: Literal["XW", "XqW", "XWq", "XqWq"],
    backend: Literal["separate", "fused"],
) -> Tensor:
    """``torch.matmul`` with ``input`` blocked along its last dim and ``other`` along its
    second-to-last dim (the contraction dim of both); batched operands are allowed."""
    check_backend(backend)
    if "Xq" in func_type:
        assert input_meta is not None
        input = quantize_dequantize(input, block_dim=-1, mxfp_meta=input_meta)
    if "Wq" in func_type:
        assert other_meta is not None
        other = quantize_dequantize(other, block_dim=-2, mxfp_meta=other_meta)
    return torch.matmul(input, other)
