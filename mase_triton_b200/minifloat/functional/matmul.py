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
    """``torch.matmul`` on operands fake-quantised per ``func_type`` (batched operands allowed).
    ``backend="fused"``: the fake-quantised operands (bf16 / fp16) are multiplied by this library's
    ``kind::f16`` tensor-core GEMM, one launch per batch entry, with ``other`` transposed once to the
    ``[N, K]`` order its loader reads; other dtypes raise ``NotImplementedError`` like the reference's
    ``fused`` (matmul.py:33-34)."""
    check_backend(backend)
    if "Xq" in func_type:
        assert input_meta is not None
        input = quantize_dequantize(input, input_meta)
    if "Wq" in func_type:
        assert other_meta is not None
        other = quantize_dequantize(other, other_meta)
    if backend == "fused":
        from ... import tc_linear

        if input.ndim < 2 or other.ndim < 2 or input.shape[-1] != other.shape[-2] or input.dtype != other.dtype:
            raise NotImplementedError("backend='fused' needs matrix operands of one dtype whose inner dimensions agree")
        K, N = other.shape[-2], other.shape[-1]
        reason = tc_linear.why_not(input, K) or tc_linear.why_not(other, K)
        if reason is not None:
            raise NotImplementedError(f"backend='fused' is not implemented for this call: {reason}; use backend='separate'")
        wt = other.transpose(-1, -2).contiguous()
        if other.ndim == 2:
            return tc_linear.dense_linear(input, wt)
        batch = torch.broadcast_shapes(input.shape[:-2], other.shape[:-2])
        rows = input.shape[-2]
        x3 = input.expand(*batch, rows, K).reshape(-1, rows, K)
        w3 = wt.expand(*batch, N, K).reshape(-1, N, K)
        out = torch.empty((x3.shape[0], rows, N), dtype=input.dtype, device=input.device)
        for i in range(x3.shape[0]):
            out[i] = tc_linear.dense_linear(x3[i], w3[i])
        return out.reshape(*batch, rows, N)
    return torch.matmul(input, other)
