"""``minifloat_linear`` (reference: ``src/mase_triton/minifloat/functional/linear.py:108-171``).

Per-tensor (un-blocked) fake quantisation of activation, weight and bias followed by a
dense linear.  ``layer_type`` names what is quantised (``Xq``/``X``, ``Wq``/``W``, ``Bq``/``B``).
Both backends give the same values: ``"separate"`` mirrors the reference's op sequence,
``"fused"`` (a stub in the reference) keeps activation and weight as 8-bit codes and multiplies them
on the tensor cores (the block-scaled GEMM with every block scale at 2^0) when both are quantised to a
finite format of at most 8 bits and ``in_features`` is a multiple of 32; otherwise it runs the same
kernels as ``"separate"``.
"""

from __future__ import annotations

from typing import Literal

import torch
from torch import Tensor

from ..._linear_common import check_backend, parse_layer_type
from ..meta import MinifloatMeta, MinifloatTensorMeta
from .. import kernels
from .cast import compose_minifloat_component, quantize_dequantize


def _narrow(meta: MinifloatMeta | None) -> bool:
    return meta is not None and meta.is_finite and meta.exp_bits + meta.frac_bits <= 7


def _tensor_core_ok(x: Tensor, x_meta, w_element, w_tensor_meta) -> bool:
    if not (x.is_cuda and w_element is not None and w_tensor_meta is not None and _narrow(x_meta) and _narrow(w_tensor_meta.meta)):
        return False
    shape = tuple(w_tensor_meta.shape)
    return (len(shape) == 2 and x.shape[-1] == shape[1] and shape[1] % 32 == 0 and x.numel() > 0
            and x.dtype in (torch.bfloat16, torch.float16, torch.float32))


def _packed_weight(w_element: Tensor, w_tensor_meta: MinifloatTensorMeta):
    """Tensor-core form of the weight codes, kept on the code tensor itself and rebuilt when it changes."""
    from ...mxfp import gemm as _gemm
    tag = (w_element._version, tuple(w_tensor_meta.shape), w_tensor_meta.meta)
    cached = getattr(w_element, "_mxq_packed", None)
    if cached is None or cached[0] != tag:
        n, k = w_tensor_meta.shape
        cached = (tag, _gemm.pack_codes(None, w_element.reshape(n, k).to(torch.uint8), n, k, w_tensor_meta.meta.exp_bits,
                                        w_tensor_meta.meta.frac_bits, _gemm.OPERAND_B))
        w_element._mxq_packed = cached
    return cached[1]


def _fused_linear(x: Tensor, x_meta: MinifloatMeta, w_element: Tensor, w_tensor_meta: MinifloatTensorMeta, bias: Tensor | None) -> Tensor:
    from ...mxfp import gemm as _gemm
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    a = _gemm.minifloat_quantize_pack(x2, x_meta.exp_bits, x_meta.frac_bits, x_meta.round_mode)    # FP8: one kernel
    if a is None:
        codes = kernels.extract_minifloat_component(x2, x_meta).to(torch.uint8)      # the sign sits below bit 8
        a = _gemm.pack_codes(None, codes, x2.shape[0], k, x_meta.exp_bits, x_meta.frac_bits, _gemm.OPERAND_A)
    out = _gemm.mx_gemm(a, _packed_weight(w_element, w_tensor_meta), x.dtype, bias=bias)
    return out.reshape(*x.shape[:-1], out.shape[-1])


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
    if backend == "fused" and kind.x_quantised and kind.w_quantised and _tensor_core_ok(x, x_meta, w_element, w_tensor_meta):
        if kind.b_quantised:
            bias = compose_minifloat_component(b_element, b_tensor_meta) if b is not None else None
        else:
            bias = b
        return _fused_linear(x, x_meta, w_element, w_tensor_meta, bias)
    if kind.x_quantised:
        x = quantize_dequantize(x, x_meta)                      # same bits as extract + compose
    weight = compose_minifloat_component(w_element, w_tensor_meta) if kind.w_quantised else w
    if kind.b_quantised:
        # a quantised-bias layer ignores a plain bias unless codes for it exist
        bias = compose_minifloat_component(b_element, b_tensor_meta) if b is not None else None
    else:
        bias = b
    return torch.nn.functional.linear(x, weight, bias)
