"""``mxfp_linear`` (reference: ``src/mase_triton/mxfp/functional/linear.py:118-210``).

``layer_type`` names what is fake-quantised: activation (``Xq``, blocks along the last dim),
weight (``Wq``, blocks along ``in_features``) and bias (``Bq``).  ``backend="separate"`` follows
the reference's op sequence (dequantise, then a dense linear in the operand dtype);
``backend="fused"`` is a stub in the reference; here it runs the tensor-core GEMMs of this library
(``csrc/mxq_gemm.cu``, ``csrc/mxq_dq_gemm.cu``) and raises ``NotImplementedError`` for what they do not take.
"""

from __future__ import annotations

from typing import Literal

import torch
from torch import Tensor

from ... import _lib, tc_linear
from ..._linear_common import check_backend, parse_layer_type
from ..meta import MXFPMeta, MXFPTensorMeta
from .. import gemm as _gemm
from .cast import compose_mxfp_tensor, quantize_dequantize

LayerType = Literal["XWB", "XWBq", "XWqB", "XWqBq", "XqWB", "XqWBq", "XqWqB", "XqWqBq"]


def parse_mxfp_linear_type(x_meta: MXFPMeta | None, w_tensor_meta: MXFPTensorMeta | None,
                           b_tensor_meta: MXFPTensorMeta | None) -> str:
    """Layer-type string for the given metas: a ``q`` after X / W / B when that operand has a meta."""
    return "".join(name + ("" if meta is None else "q")
                   for name, meta in (("X", x_meta), ("W", w_tensor_meta), ("B", b_tensor_meta)))


def block_scaled_ok(x: Tensor, x_meta: MXFPMeta | None, w_tensor_meta: MXFPTensorMeta | None) -> bool:
    """True when ``x`` and a weight described by ``w_tensor_meta`` can both stay quantised on the block-scaled
    tensor-core GEMM: 32-element blocks along ``in_features``, is_finite elements, CUDA, a kernel dtype."""
    if x_meta is None or w_tensor_meta is None:
        return False
    shape = tuple(w_tensor_meta.shape)
    return (len(shape) == 2 and w_tensor_meta.block_dim in (1, -1) and _gemm.supported(w_tensor_meta.meta) and _gemm.supported(x_meta)
            and x.is_cuda and x.dtype in _lib.DTYPE_ID and x.shape[-1] == shape[1] and shape[1] % 32 == 0 and x.numel() > 0)


def _fused_linear(x: Tensor, x_meta: MXFPMeta | None, w: Tensor | None, w_scales: Tensor | None, w_elements: Tensor | None,
                  w_tensor_meta: MXFPTensorMeta | None, bias: Tensor | None, kind, bias_q=None) -> Tensor:
    """``backend="fused"``: every layer type runs a hand-written tensor-core GEMM of this library.

    * ``XqWq`` with 32-element blocks and is_finite elements: both operands stay quantised, block-scaled
      ``tcgen05.mma.kind::mxf8f6f4`` GEMM (fp32 / bf16 / fp16 activations); MXFP4 activation x MXFP4 weight with
      ``in_features`` a multiple of 256 stay packed nibbles and run on ``kind::mxf4`` at twice the rate;
    * every other combination on bf16 / fp16 activations: ``tcgen05.mma.kind::f16`` GEMM; an ``Xq``
      activation is fake-quantised by one bandwidth-bound kernel first, a ``Wq`` weight is expanded from
      its codes inside the GEMM's operand loader while the activation is short, and once by the compose
      kernel otherwise (``tc_linear.expand_in_loader``; also for block layouts that loader does not read);
    * anything else raises ``NotImplementedError`` as the reference's ``fused`` does -- nothing falls back to
      a library GEMM silently.
    """
    w_shape = tuple(w_tensor_meta.shape) if kind.w_quantised else tuple(w.shape)
    K = x.shape[-1]
    w_blocks_along_k = kind.w_quantised and len(w_shape) == 2 and w_tensor_meta.block_dim in (1, -1) and _gemm.supported(w_tensor_meta.meta)
    if kind.x_quantised and kind.w_quantised and block_scaled_ok(x, x_meta, w_tensor_meta):
        wq = _gemm.packed_weight(w_scales, w_elements, w_shape, w_tensor_meta.meta, rows=x.numel() // K,
                                 nibbles=_gemm.fp4_pair(x_meta, w_tensor_meta.meta, K))
        if bias_q is not None and _gemm.bias_codes_ok(bias_q[0], bias_q[1], bias_q[2].meta, w_shape[0], getattr(torch, bias_q[2].dtype), x.dtype):
            # the bias stays quantised too: its codes are decoded in the GEMM's epilogue
            return _gemm.mx_linear(x, x_meta, wq, None, bias_q=(bias_q[0], bias_q[1], bias_q[2].meta))
        if bias_q is not None:
            bias = compose_mxfp_tensor(*bias_q)
        return _gemm.mx_linear(x, x_meta, wq, bias)
    if bias_q is not None:
        bias = compose_mxfp_tensor(*bias_q)
    reason = tc_linear.why_not(x, K)
    if reason is not None:
        raise NotImplementedError(f"backend='fused' is not implemented for this call: {reason}; use backend='separate'")
    if kind.x_quantised:
        x = quantize_dequantize(x, block_dim=-1, mxfp_meta=x_meta)       # same bits as extract + compose
    if not kind.w_quantised:
        return tc_linear.dense_linear(x, w, bias)
    if getattr(torch, w_tensor_meta.dtype) != x.dtype:
        raise RuntimeError(f"the weight dequantises to {w_tensor_meta.dtype}, the input is {x.dtype}")
    if w_blocks_along_k and K % 32 == 0 and tc_linear.expand_in_loader(x.numel() // K, w_shape[0]):
        return tc_linear.mxfp_weight_linear(x, w_scales, w_elements, w_shape, w_tensor_meta.meta, bias)
    return tc_linear.dense_linear(x, compose_mxfp_tensor(w_scales, w_elements, w_tensor_meta).contiguous(), bias)


def mxfp_linear(
    x: Tensor,
    x_meta: MXFPMeta | None,
    w: Tensor | None,
    w_scales: Tensor | None,
    w_elements: Tensor | None,
    w_tensor_meta: MXFPTensorMeta | None,
    b: Tensor | None,
    b_scales: Tensor | None,
    b_elements: Tensor | None,
    b_tensor_meta: MXFPTensorMeta | None,
    layer_type: LayerType,
    backend: Literal["separate", "fused"],
) -> Tensor:
    kind = parse_layer_type(layer_type)
    check_backend(backend)
    if backend == "fused":
        # the reference only uses bias codes when a plain bias is passed as well (then the codes win); the fused route
        # hands them on as codes so that the block-scaled GEMM can decode them in its epilogue
        bias_q = (b_scales, b_elements, b_tensor_meta) if (kind.b_quantised and b is not None) else None
        return _fused_linear(x, x_meta, w, w_scales, w_elements, w_tensor_meta, None if kind.b_quantised else b, kind, bias_q)
    if kind.b_quantised:
        # the reference only dequantises bias codes when a plain bias is passed as well
        bias = compose_mxfp_tensor(b_scales, b_elements, b_tensor_meta) if b is not None else None
    else:
        bias = b
    if kind.x_quantised:
        x = quantize_dequantize(x, block_dim=-1, mxfp_meta=x_meta)       # same bits as extract + compose
    weight = compose_mxfp_tensor(w_scales, w_elements, w_tensor_meta) if kind.w_quantised else w
    return torch.nn.functional.linear(x, weight, bias)
