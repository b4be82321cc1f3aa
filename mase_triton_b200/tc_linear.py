"""Host side of the dequantise-in-the-loader tensor-core GEMM (``csrc/mxq_dq_gemm.cu``).

``backend="fused"`` of the linear / matmul functions lands here for every layer type whose operands
are not both block-quantised: the activation is bf16 / fp16 (fake-quantised first when the layer type
says ``Xq``) and the weight is dense, MXFP codes + scales, or per-tensor minifloat codes that the
kernel expands while it loads them.  The reference implements none of this: its ``backend="fused"``
raises ``NotImplementedError`` (``src/mase_triton/mxfp/functional/linear.py:31-32``).
"""

from __future__ import annotations

import torch
from torch import Tensor

from . import _lib
from .mxfp.gemm import _raise_if_failed, status_word

TC_DTYPES = (torch.bfloat16, torch.float16)


def why_not(x: Tensor, K: int, multiple: int = 8) -> str | None:
    """``None`` when ``x [..., K]`` can be the left operand of these kernels, else the reason."""
    if not x.is_cuda:
        return "tensors are not on a CUDA device"
    if x.dtype not in TC_DTYPES:
        return f"operand dtype {x.dtype} (the tensor-core path of this layer type takes bfloat16 / float16)"
    if x.numel() == 0:
        return "empty input"
    if K % multiple != 0:
        return f"in_features={K} is not a multiple of {multiple}"
    return None


def _prep(x: Tensor, N: int, bias: Tensor | None):
    K = x.shape[-1]
    x2 = x.reshape(-1, K).contiguous()
    out = torch.empty((x2.shape[0], N), dtype=x.dtype, device=x.device)
    if bias is not None:
        assert bias.numel() == N
        bias = bias.to(x.dtype).contiguous()
    _raise_if_failed(x.device)
    return x2, out, bias


def dense_linear(x: Tensor, w: Tensor, bias: Tensor | None = None) -> Tensor:
    """``x [..., K] @ w[N, K]^T (+ bias)`` with both operands dense bf16 / fp16."""
    if w.dtype != x.dtype:
        raise RuntimeError(f"expected the weight to have the input's dtype {x.dtype}, got {w.dtype}")
    N, K = w.shape
    assert x.shape[-1] == K
    x2, out, bias = _prep(x, N, bias)
    w = w.contiguous()
    dev = x.device
    with torch.cuda.device(dev):
        rc = _lib.load().mxq_dense_linear(x2.data_ptr(), w.data_ptr(), _lib.DTYPE_ID[x.dtype], out.data_ptr(),
                                          None if bias is None else bias.data_ptr(), x2.shape[0], N, K,
                                          status_word(dev).data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc, "mxq_dense_linear")
    return out.reshape(*x.shape[:-1], N)


def mxfp_weight_linear(x: Tensor, w_scales: Tensor, w_elements: Tensor, shape: tuple[int, int], w_meta, bias: Tensor | None = None) -> Tensor:
    """``x @ dequant(W)^T (+ bias)`` with ``W`` left as MXFP codes + scales (32-element blocks along
    ``in_features``, is_finite elements) and expanded inside the GEMM's operand loader."""
    N, K = shape
    assert x.shape[-1] == K and w_meta.block_size == 32 and w_meta.element_is_finite
    assert w_scales.dtype == torch.uint8 and w_elements.dtype == torch.uint8
    assert w_elements.numel() == N * K and w_scales.numel() == N * K // 32
    x2, out, bias = _prep(x, N, bias)
    w_scales, w_elements = w_scales.contiguous(), w_elements.contiguous()
    dev = x.device
    with torch.cuda.device(dev):
        rc = _lib.load().mxq_mxfp_weight_linear(x2.data_ptr(), _lib.DTYPE_ID[x.dtype], w_scales.data_ptr(), w_elements.data_ptr(),
                                                w_meta.element_exp_bits, w_meta.element_frac_bits, out.data_ptr(),
                                                None if bias is None else bias.data_ptr(), x2.shape[0], N, K,
                                                status_word(dev).data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc, "mxq_mxfp_weight_linear")
    return out.reshape(*x.shape[:-1], N)


def minifloat_weight_linear(x: Tensor, w_element: Tensor, shape: tuple[int, int], w_meta, bias: Tensor | None = None) -> Tensor:
    """``x @ dequant(W)^T (+ bias)`` with ``W`` left as per-tensor minifloat uint16 codes."""
    N, K = shape
    assert x.shape[-1] == K and w_element.dtype == torch.uint16 and w_element.numel() == N * K
    x2, out, bias = _prep(x, N, bias)
    w_element = w_element.contiguous()
    dev = x.device
    with torch.cuda.device(dev):
        rc = _lib.load().mxq_minifloat_weight_linear(x2.data_ptr(), _lib.DTYPE_ID[x.dtype], w_element.data_ptr(), w_meta.exp_bits,
                                                     w_meta.frac_bits, int(bool(w_meta.is_finite)), out.data_ptr(),
                                                     None if bias is None else bias.data_ptr(), x2.shape[0], N, K,
                                                     status_word(dev).data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc, "mxq_minifloat_weight_linear")
    return out.reshape(*x.shape[:-1], N)


def expand_in_loader(rows: int, out_features: int) -> bool:
    """Where a weight-only-quantised linear expands its codes.  Inside the GEMM's loader every 256-row tile of
    the activation expands the weight again, so that route pays while the activation is at most two tiles tall and
    the weight has enough column tiles to occupy the GPU (then the dense weight never exists in memory and the
    codes are read once).  Taller activations expand the weight once with the compose kernel (same values bit
    for bit) and run the same GEMM on dense operands: measured on B200 with a 14336 x 4096 MXFP8 weight,
    0.080 / 0.155 / 0.98 ms in the loader against 0.085 / 0.128 / 0.65 ms expanded once at 512 / 1024 / 8192 rows."""
    return rows <= 512 and out_features >= 8192

