"""``mxfp_linear`` (reference: ``src/mase_triton/mxfp/functional/linear.py:118-210``).

``layer_type`` names what is fake-quantised: activation (``Xq``, blocks along the last dim),
weight (``Wq``, blocks along ``in_features``) and bias (``Bq``).  ``backend="separate"`` follows
the reference's op sequence (dequantise, then a dense linear in the operand dtype);
``backend="fused"`` is a stub in the reference and is implemented here.
"""

from __future__ import annotations

from typing import Literal

import torch
from torch import Tensor

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
    if kind.b_quantised:
        # the reference only dequantises bias codes when a plain bias is passed as well
        bias = compose_mxfp_tensor(b_scales, b_elements, b_tensor_meta) if b is not None else None
    else:
        bias = b
    if (backend == "fused" and kind.x_quantised and kind.w_quantised and x.is_cuda and x.dtype in (torch.bfloat16, torch.float16, torch.float32)
            and _gemm.supported(x_meta) and _gemm.supported(w_tensor_meta.meta) and w_tensor_meta.block_dim in (1, -1)
            and len(w_tensor_meta.shape) == 2 and x.shape[-1] % 32 == 0 and x.numel() > 0):
        # both operands stay quantised: block-scaled tensor-core GEMM, fp32 accumulation
        wq = _gemm.packed_weight(w_scales, w_elements, w_tensor_meta.shape, w_tensor_meta.meta)
        return _gemm.mx_linear(x, x_meta, wq, bias)
    if kind.x_quantised:
        x = quantize_dequantize(x, block_dim=-1, mxfp_meta=x_meta)       # same bits as extract + compose
    weight = compose_mxfp_tensor(w_scales, w_elements, w_tensor_meta) if kind.w_quantised else w
    return torch.nn.functional.linear(x, weight, bias)
