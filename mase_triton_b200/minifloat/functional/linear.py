"""``minifloat_linear`` (reference: ``src/mase_triton/minifloat/functional/linear.py:108-171``).

Per-tensor (un-blocked) fake quantisation of activation, weight and bias followed by a
dense linear.  ``layer_type`` names what is quantised (``Xq``/``X``, ``Wq``/``W``, ``Bq``/``B``).
``"separate"`` mirrors the reference's op sequence (dequantise, then a library linear).  ``"fused"`` (a stub
in the reference) runs this library's tensor-core GEMMs: with both operands quantised to E4M3, E5M2 or one
of the narrower OCP formats and ``in_features`` a multiple of 32, activation and weight stay 8-bit codes
(the block-scaled GEMM with every block scale at 2^0; FP4 x FP4 with ``in_features`` a multiple of 256 stays packed
nibbles on the 4-bit tensor-core kind); every other layer type on bf16 / fp16 activations
takes the ``kind::f16`` GEMM that expands weight codes in its operand loader; what neither takes raises
``NotImplementedError``.
"""

from __future__ import annotations

from typing import Literal

import torch
from torch import Tensor

from ..._linear_common import check_backend, parse_layer_type
from ..meta import MinifloatMeta, MinifloatTensorMeta
from .. import kernels
from .cast import compose_minifloat_component, quantize_dequantize


# element formats whose every value has an exact 8-bit tensor-core encoding (the pack tables of
# mxq_mx_pack_operand): E4M3, E5M2 and the three narrower OCP formats
_TENSOR_CORE_FORMATS = frozenset({(4, 3), (5, 2), (2, 3), (3, 2), (2, 1)})


def _narrow(meta: MinifloatMeta | None) -> bool:
    return meta is not None and meta.is_finite and (meta.exp_bits, meta.frac_bits) in _TENSOR_CORE_FORMATS


def _tensor_core_ok(x: Tensor, x_meta, w_element, w_tensor_meta) -> bool:
    if not (x.is_cuda and w_element is not None and w_tensor_meta is not None and _narrow(x_meta) and _narrow(w_tensor_meta.meta)):
        return False
    shape = tuple(w_tensor_meta.shape)
    return (len(shape) == 2 and x.shape[-1] == shape[1] and shape[1] % 32 == 0 and x.numel() > 0
            and x.dtype in (torch.bfloat16, torch.float16, torch.float32))


def _fp4_pair(x_meta: MinifloatMeta, w_meta: MinifloatMeta, k: int) -> bool:
    """FP4 (E2M1) activation and weight with whole 256-element stages: both stay packed nibbles and the GEMM runs on
    the 4-bit x 4-bit tensor-core kind (every block scale 2^0), at twice the rate of the 8-bit kinds."""
    return (x_meta.exp_bits, x_meta.frac_bits) == (2, 1) and (w_meta.exp_bits, w_meta.frac_bits) == (2, 1) and k % 256 == 0


def _packed_weight(w_element: Tensor, w_tensor_meta: MinifloatTensorMeta, nibbles: bool = False):
    """Tensor-core form of the weight codes, kept on the code tensor itself and rebuilt when it changes."""
    from ...mxfp import gemm as _gemm
    tag = (w_element._version, tuple(w_tensor_meta.shape), w_tensor_meta.meta, nibbles)
    cached = getattr(w_element, "_mxq_packed", None)
    if cached is None or cached[0] != tag:
        n, k = w_tensor_meta.shape
        cached = (tag, _gemm.pack_codes(None, w_element.reshape(n, k).to(torch.uint8), n, k, w_tensor_meta.meta.exp_bits,
                                        w_tensor_meta.meta.frac_bits, _gemm.OPERAND_B, native=nibbles))
        w_element._mxq_packed = cached
    return cached[1]


def _fused_linear(x: Tensor, x_meta: MinifloatMeta, w_element: Tensor, w_tensor_meta: MinifloatTensorMeta, bias: Tensor | None) -> Tensor:
    from ...mxfp import gemm as _gemm
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    nibbles = _fp4_pair(x_meta, w_tensor_meta.meta, k)
    a = None if nibbles else _gemm.minifloat_quantize_pack(x2, x_meta.exp_bits, x_meta.frac_bits, x_meta.round_mode)    # FP8: one kernel
    if a is None:
        codes = kernels.extract_minifloat_component(x2, x_meta).to(torch.uint8)      # the sign sits below bit 8
        a = _gemm.pack_codes(None, codes, x2.shape[0], k, x_meta.exp_bits, x_meta.frac_bits, _gemm.OPERAND_A, native=nibbles)
    out = _gemm.mx_gemm(a, _packed_weight(w_element, w_tensor_meta, nibbles), x.dtype, bias=bias)
    return out.reshape(*x.shape[:-1], out.shape[-1])


def _tc_linear(x: Tensor, x_meta, w: Tensor | None, w_element: Tensor | None, w_tensor_meta, bias: Tensor | None, kind) -> Tensor:
    """``backend="fused"`` for the layer types that are not "both operands as 8-bit tensor-core codes":
    ``tcgen05.mma.kind::f16`` GEMM on bf16 / fp16 activations; an ``Xq`` activation is fake-quantised by
    one kernel first, ``Wq`` codes are expanded inside the GEMM's operand loader while the activation is short and
    once by the compose kernel otherwise (``tc_linear.expand_in_loader``)."""
    from ... import tc_linear

    reason = tc_linear.why_not(x, x.shape[-1])
    if reason is not None:
        raise NotImplementedError(f"backend='fused' is not implemented for this call: {reason}; use backend='separate'")
    if kind.x_quantised:
        x = quantize_dequantize(x, x_meta)
    if not kind.w_quantised:
        return tc_linear.dense_linear(x, w, bias)
    if getattr(torch, w_tensor_meta.dtype) != x.dtype:
        raise RuntimeError(f"the weight dequantises to {w_tensor_meta.dtype}, the input is {x.dtype}")
    shape = tuple(w_tensor_meta.shape)
    if (len(shape) == 2 and w_tensor_meta.meta.exp_bits <= 8 and w_element.dtype == torch.uint16
            and tc_linear.expand_in_loader(x.numel() // x.shape[-1], shape[0])):
        return tc_linear.minifloat_weight_linear(x, w_element, shape, w_tensor_meta.meta, bias)
    return tc_linear.dense_linear(x, compose_minifloat_component(w_element, w_tensor_meta).contiguous(), bias)


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
    if kind.b_quantised:
        # a quantised-bias layer ignores a plain bias unless codes for it exist
        bias = compose_minifloat_component(b_element, b_tensor_meta) if b is not None else None
    else:
        bias = b
    if backend == "fused":
        if kind.x_quantised and kind.w_quantised and _tensor_core_ok(x, x_meta, w_element, w_tensor_meta):
            return _fused_linear(x, x_meta, w_element, w_tensor_meta, bias)
        return _tc_linear(x, x_meta, w, w_element, w_tensor_meta, bias, kind)
    if kind.x_quantised:
        x = quantize_dequantize(x, x_meta)                      # same bits as extract + compose
    weight = compose_minifloat_component(w_element, w_tensor_meta) if kind.w_quantised else w
    return torch.nn.functional.linear(x, weight, bias)
