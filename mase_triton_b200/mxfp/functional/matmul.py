"""``mxfp_matmul`` (reference: ``src/mase_triton/mxfp/functional/matmul.py:10-35``)."""

from __future__ import annotations

from typing import Literal

import torch
from torch import Tensor

from ... import tc_linear
from ..._linear_common import check_backend
from .. import gemm as _gemm
from ..meta import MXFPMeta
from .cast import extract_mxfp_components, quantize_dequantize


def _fused_matmul(input: Tensor, other: Tensor, input_meta: MXFPMeta, other_meta: MXFPMeta) -> Tensor:
    """Both operands stay quantised.  ``other`` (blocks along its second-to-last dim, the contraction
    dim) is quantised by the strided-block kernel, whose output order is already the ``[N, K]`` layout
    the right GEMM operand needs, so no transposed copy is made; both operands are quantised with one
    kernel each over all batch entries, and every batch entry is one block-scaled tensor-core GEMM."""
    K, N = other.shape[-2], other.shape[-1]
    w_scales, w_elements, _ = extract_mxfp_components(other, -2, other_meta)       # [..., N, K] order
    if other.ndim == 2:                                  # shared right operand: one GEMM over all rows
        a = _gemm.pack_activation(input.reshape(-1, K), input_meta)
        b = _gemm.pack_operand(w_scales, w_elements, N, K, other_meta, _gemm.OPERAND_B)
        return _gemm.mx_gemm(a, b, input.dtype).reshape(*input.shape[:-1], N)
    batch = torch.broadcast_shapes(input.shape[:-2], other.shape[:-2])
    rows = input.shape[-2]
    x_scales, x_elements, _ = extract_mxfp_components(input, -1, input_meta)
    nb_x, nb_w = input.numel() // (rows * K), other.numel() // (K * N)
    x_scales, x_elements = x_scales.view(nb_x, rows * K // 32), x_elements.view(nb_x, rows * K)
    w_scales, w_elements = w_scales.view(nb_w, N * K // 32), w_elements.view(nb_w, N * K)
    # batch entry i of the broadcast result reads entry ix[i] of input and iw[i] of other
    ix = torch.arange(nb_x).view(*input.shape[:-2]).expand(batch).reshape(-1).tolist()
    iw = torch.arange(nb_w).view(*other.shape[:-2]).expand(batch).reshape(-1).tolist()
    packed_x: dict[int, _gemm.PackedOperand] = {}
    packed_w: dict[int, _gemm.PackedOperand] = {}
    out = torch.empty((len(ix), rows, N), dtype=input.dtype, device=input.device)
    for i, (jx, jw) in enumerate(zip(ix, iw)):
        if jx not in packed_x:
            packed_x[jx] = _gemm.pack_operand(x_scales[jx], x_elements[jx], rows, K, input_meta, _gemm.OPERAND_A)
        if jw not in packed_w:
            packed_w[jw] = _gemm.pack_operand(w_scales[jw], w_elements[jw], N, K, other_meta, _gemm.OPERAND_B)
        _gemm.mx_gemm(packed_x[jx], packed_w[jw], input.dtype, out=out[i])
    return out.reshape(*batch, rows, N)


def _tc_matmul(input: Tensor, other: Tensor, input_meta: MXFPMeta | None, other_meta: MXFPMeta | None, func_type: str) -> Tensor:
    """``backend="fused"`` for the forms whose operands are not both block-quantised codes (bf16 / fp16): the
    left operand is fake-quantised by one kernel when ``Xq``; a ``Wq`` right operand is quantised by the
    strided-block kernel, whose ``[N, K]`` code order is what the GEMM's loader expands on the fly; a dense
    right operand is transposed once to ``[N, K]``.  Each batch entry is one ``kind::f16`` tensor-core GEMM."""
    K, N = other.shape[-2], other.shape[-1]
    if "Xq" in func_type:
        input = quantize_dequantize(input, block_dim=-1, mxfp_meta=input_meta)
    batch = torch.broadcast_shapes(input.shape[:-2], other.shape[:-2]) if other.ndim > 2 else None
    rows = input.shape[-2]
    quantised_w = "Wq" in func_type and _gemm.supported(other_meta) and K % 32 == 0
    if quantised_w:
        w_scales, w_elements, _ = extract_mxfp_components(other, -2, other_meta)           # [..., N, K] order
        nb_w = other.numel() // (K * N)
        w_scales, w_elements = w_scales.view(nb_w, N * K // 32), w_elements.view(nb_w, N * K)
        run = lambda x2, j: tc_linear.mxfp_weight_linear(x2, w_scales[j], w_elements[j], (N, K), other_meta)     # noqa: E731
    else:
        if "Wq" in func_type:
            other = quantize_dequantize(other, block_dim=-2, mxfp_meta=other_meta)
        wt = other.transpose(-1, -2).contiguous().view(-1, N, K)
        run = lambda x2, j: tc_linear.dense_linear(x2, wt[j])                                                    # noqa: E731
    if batch is None:
        return run(input.reshape(-1, K), 0).reshape(*input.shape[:-1], N)
    nb_x = input.numel() // (rows * K)
    x3 = input.reshape(nb_x, rows, K)
    ix = torch.arange(nb_x).view(*input.shape[:-2]).expand(batch).reshape(-1).tolist()
    iw = torch.arange(other.numel() // (K * N)).view(*other.shape[:-2]).expand(batch).reshape(-1).tolist()
    out = torch.empty((len(ix), rows, N), dtype=input.dtype, device=input.device)
    for i, (jx, jw) in enumerate(zip(ix, iw)):
        out[i] = run(x3[jx], jw)
    return out.reshape(*batch, rows, N)


def mxfp_matmul(
    input: Tensor,
    other: Tensor,
    input_meta: MXFPMeta | None,
    other_meta: MXFPMeta | None,
    func_type: Literal["XW", "XqW", "XWq", "XqWq"],
    backend: Literal["separate", "fused"],
) -> Tensor:
    """``torch.matmul`` with ``input`` blocked along its last dim and ``other`` along its
    second-to-last dim (the contraction dim of both); batched operands are allowed.
    ``backend="fused"`` runs this library's tensor-core GEMMs and raises ``NotImplementedError`` for what
    they do not take (the reference raises it for every ``fused`` call, matmul.py:31-32)."""
    check_backend(backend)
    if "Xq" in func_type:
        assert input_meta is not None
    if "Wq" in func_type:
        assert other_meta is not None
    if backend == "fused":
        if input.ndim < 2 or other.ndim < 2 or input.shape[-1] != other.shape[-2] or input.dtype != other.dtype:
            raise NotImplementedError("backend='fused' needs matrix operands of one dtype whose inner dimensions agree")
        if (func_type == "XqWq" and input.is_cuda and other.is_cuda and _gemm.supported(input_meta) and _gemm.supported(other_meta)
                and input.dtype in (torch.bfloat16, torch.float16, torch.float32) and input.shape[-1] % 32 == 0
                and input.numel() > 0 and other.numel() > 0):
            return _fused_matmul(input, other, input_meta, other_meta)
        reason = tc_linear.why_not(input, input.shape[-1]) or tc_linear.why_not(other, input.shape[-1])
        if reason is not None:
            raise NotImplementedError(f"backend='fused' is not implemented for this call: {reason}; use backend='separate'")
        return _tc_matmul(input, other, input_meta, other_meta, func_type)
    if "Xq" in func_type:
        input = quantize_dequantize(input, block_dim=-1, mxfp_meta=input_meta)
    if "Wq" in func_type:
        other = quantize_dequantize(other, block_dim=-2, mxfp_meta=other_meta)
    return torch.matmul(input, other)
