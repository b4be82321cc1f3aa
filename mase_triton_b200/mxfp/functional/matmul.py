"""``mxfp_matmul`` (reference: ``src/mase_triton/mxfp/functional/matmul.py:10-35``)."""

from __future__ import annotations

from typing import Literal

import torch
from torch import Tensor

from ..._linear_common import check_backend
from .. import gemm as _gemm
from ..meta import MXFPMeta
from .cast import quantize_dequantize


def _fused_matmul(input: Tensor, other: Tensor, input_meta: MXFPMeta, other_meta: MXFPMeta) -> Tensor:
    """Both operands stay quantised: ``other`` is transposed to ``[N, K]`` so that its blocks (along its
    second-to-last dim, the contraction dim) run along the contiguous dim, and every batch entry is one
    block-scaled tensor-core GEMM."""
    K, N = other.shape[-2], other.shape[-1]
    if other.ndim == 2:                                  # shared right operand: one GEMM over all rows
        a = _gemm.quantize_pack_fused(input.reshape(-1, K), input_meta) if input_meta.element_exp_bits >= 4 \
            else _gemm.quantize_pack(input.reshape(-1, K), input_meta)
        b = _gemm.quantize_pack(other.t().contiguous(), other_meta, _gemm.OPERAND_B)
        return _gemm.mx_gemm(a, b, input.dtype).reshape(*input.shape[:-1], N)
    batch = torch.broadcast_shapes(input.shape[:-2], other.shape[:-2])
    x = input.expand(*batch, *input.shape[-2:]).reshape(-1, input.shape[-2], K)
    w = other.expand(*batch, K, N).reshape(-1, K, N)
    out = torch.empty((x.shape[0], x.shape[1], N), dtype=input.dtype, device=input.device)
    for i in range(x.shape[0]):
        a = _gemm.quantize_pack(x[i], input_meta)
        b = _gemm.quantize_pack(w[i].t().contiguous(), other_meta, _gemm.OPERAND_B)
        _gemm.mx_gemm(a, b, input.dtype, out=out[i])
    return out.reshape(*batch, input.shape[-2], N)


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
    if (backend == "fused" and "Xq" in func_type and "Wq" in func_type and input.is_cuda and other.is_cuda
            and _gemm.supported(input_meta) and _gemm.supported(other_meta) and input.ndim >= 2 and other.ndim >= 2
            and input.dtype == other.dtype and input.dtype in (torch.bfloat16, torch.float16, torch.float32)
            and input.shape[-1] == other.shape[-2] and input.shape[-1] % 32 == 0 and input.numel() > 0 and other.numel() > 0):
        return _fused_matmul(input, other, input_meta, other_meta)
    if "Xq" in func_type:
        assert input_meta is not None
        input = quantize_dequantize(input, block_dim=-1, mxfp_meta=input_meta)
    if "Wq" in func_type:
        assert other_meta is not None
        other = quantize_dequantize(other, block_dim=-2, mxfp_meta=other_meta)
    return torch.matmul(input, other)
