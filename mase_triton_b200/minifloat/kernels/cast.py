"""Host side of the minifloat CUDA kernels.

Same seam as the reference's Triton hosts (``src/mase_triton/minifloat/kernels/cast.py:148-170``
and ``:263-288``): a contiguous tensor in, a freshly allocated tensor out, launched on the
current stream of the tensor's device.  The arithmetic matches the reference's PyTorch path
(``src/mase_triton/minifloat/fake.py``) bit for bit.
"""

from __future__ import annotations

import torch
from torch import Tensor

from .. import meta as _meta
from ... import _lib


def _codes_u16(elements: Tensor) -> Tensor:
    assert elements.dtype == torch.uint16
    return elements.contiguous()


def extract_minifloat_component(x: Tensor, minifloat_meta: "_meta.MinifloatMeta") -> Tensor:
    """Floating tensor (fp32 / bf16 / fp16) -> uint16 codes of the same shape."""
    _lib.require_cuda(x, "extract_minifloat_component")
    if x.dtype not in _lib.DTYPE_ID:
        x = x.to(torch.float32)
    x = x.contiguous()
    codes = torch.empty(x.shape, dtype=torch.uint16, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.load().mxq_minifloat_extract(x.data_ptr(), _lib.DTYPE_ID[x.dtype], codes.data_ptr(), x.numel(),
                                               *_lib.fmt_args(minifloat_meta), _lib.stream_ptr(x.device))
    _lib.check(rc, "mxq_minifloat_extract")
    return codes


def compose_minifloat_component(elements: Tensor, minifloat_meta: "_meta.MinifloatMeta", output_dtype: torch.dtype) -> Tensor:
    """uint16 codes -> tensor of ``output_dtype`` with the same shape."""
    _lib.require_cuda(elements, "compose_minifloat_component")
    elements = _codes_u16(elements)
    kernel_dtype = output_dtype if output_dtype in _lib.DTYPE_ID else torch.float32
    out = torch.empty(elements.shape, dtype=kernel_dtype, device=elements.device)
    eb, fb, fin, _ = _lib.fmt_args(minifloat_meta)
    with torch.cuda.device(elements.device):
        rc = _lib.load().mxq_minifloat_compose(elements.data_ptr(), out.data_ptr(), _lib.DTYPE_ID[kernel_dtype],
                                               elements.numel(), eb, fb, fin, _lib.stream_ptr(elements.device))
    _lib.check(rc, "mxq_minifloat_compose")
    return out if kernel_dtype == output_dtype else out.to(output_dtype)


def quantize_dequantize(x: Tensor, minifloat_meta: "_meta.MinifloatMeta", output_dtype: torch.dtype,
                        out: Tensor | None = None) -> Tensor:
    """extract + compose in one pass, without the uint16 intermediate. ``out`` (contiguous, same
    number of elements, a kernel dtype) receives the result when given."""
    _lib.require_cuda(x, "quantize_dequantize")
    if x.dtype not in _lib.DTYPE_ID:
        x = x.to(torch.float32)
    x = x.contiguous()
    kernel_dtype = output_dtype if output_dtype in _lib.DTYPE_ID else torch.float32
    if out is None:
        out = torch.empty(x.shape, dtype=kernel_dtype, device=x.device)
    else:
        assert out.is_contiguous() and out.numel() == x.numel() and out.dtype == kernel_dtype == output_dtype
    with torch.cuda.device(x.device):
        rc = _lib.load().mxq_minifloat_qdq(x.data_ptr(), _lib.DTYPE_ID[x.dtype], out.data_ptr(), _lib.DTYPE_ID[kernel_dtype],
                                           x.numel(), *_lib.fmt_args(minifloat_meta), _lib.stream_ptr(x.device))
    _lib.check(rc, "mxq_minifloat_qdq")
    return out if kernel_dtype == output_dtype else out.to(output_dtype)
