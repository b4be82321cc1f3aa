"""Host side of the MXFP CUDA kernels.

Same seam as the reference's Triton hosts (``src/mase_triton/mxfp/kernels/cast.py:126-160`` and
``:237-272``): a flat tensor in, freshly allocated tensors out, launched on the current stream of
the tensor's device.  The block maximum is reduced inside the kernel (the reference runs a
separate ``_find_block_max`` pass, ``:15-21``).  Results match the reference's PyTorch path
(``src/mase_triton/mxfp/fake.py``) bit for bit.
"""

from __future__ import annotations

import torch
from torch import Tensor

from ... import _lib
from ..meta import MXFPMeta


def _fmt(mxfp_meta: MXFPMeta):
    return (mxfp_meta.block_size, mxfp_meta.element_exp_bits, mxfp_meta.element_frac_bits,
            int(bool(mxfp_meta.element_is_finite)), _lib.ROUND_ID[mxfp_meta.round_mode])


def _as_kernel_input(x: Tensor) -> Tensor:
    if x.dtype not in _lib.DTYPE_ID:
        x = x.float()
    return x.contiguous()


def extract_mxfp_components(x: Tensor, mxfp_meta: MXFPMeta) -> tuple[Tensor, Tensor]:
    """1-D floating tensor -> ``(scales uint8 [n_blocks, 1], elements uint8 [n_blocks, block_size])``."""
    _lib.require_cuda(x, "extract_mxfp_components")
    assert x.ndim == 1, "x must be a 1D tensor"
    x = _as_kernel_input(x)
    B, eb, fb, fin, rm = _fmt(mxfp_meta)
    n = x.numel()
    assert n % B == 0, "Number of elements must be a multiple of block size"
    scales = torch.empty((n // B, 1), dtype=torch.uint8, device=x.device)
    elements = torch.empty((n // B, B), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.load().mxq_mxfp_extract(x.data_ptr(), _lib.DTYPE_ID[x.dtype], scales.data_ptr(), elements.data_ptr(),
                                          n, B, eb, fb, fin, rm, _lib.stream_ptr(x.device))
    _lib.check(rc, "mxq_mxfp_extract")
    return scales, elements


def compose_mxfp_tensor(scales: Tensor, elements: Tensor, mxfp_meta: MXFPMeta, output_dtype: torch.dtype) -> Tensor:
    """``(scales, elements)`` -> flat tensor of ``output_dtype``."""
    _lib.require_cuda(elements, "compose_mxfp_tensor")
    assert scales.dtype == torch.uint8
    assert elements.dtype == torch.uint8
    scales, elements = scales.contiguous(), elements.contiguous()
    B, eb, fb, fin, _ = _fmt(mxfp_meta)
    n = elements.numel()
    assert n == scales.numel() * B, "elements and scales disagree on the number of blocks"
    kernel_dtype = output_dtype if output_dtype in _lib.DTYPE_ID else torch.float32
    out = torch.empty((n,), dtype=kernel_dtype, device=elements.device)
    with torch.cuda.device(elements.device):
        rc = _lib.load().mxq_mxfp_compose(scales.data_ptr(), elements.data_ptr(), out.data_ptr(),
                                          _lib.DTYPE_ID[kernel_dtype], n, B, eb, fb, fin, _lib.stream_ptr(elements.device))
    _lib.check(rc, "mxq_mxfp_compose")
    return out if kernel_dtype == output_dtype else out.to(output_dtype)


def quantize_dequantize(x: Tensor, mxfp_meta: MXFPMeta, output_dtype: torch.dtype, out: Tensor | None = None) -> Tensor:
    """Fused extract + compose of a flat tensor: no scales or elements are written. ``out``
    (contiguous, same number of elements, a kernel dtype) receives the result when given."""
    _lib.require_cuda(x, "quantize_dequantize")
    assert x.ndim == 1, "x must be a 1D tensor"
    x = _as_kernel_input(x)
    B, eb, fb, fin, rm = _fmt(mxfp_meta)
    n = x.numel()
    assert n % B == 0, "Number of elements must be a multiple of block size"
    kernel_dtype = output_dtype if output_dtype in _lib.DTYPE_ID else torch.float32
    if out is None:
        out = torch.empty((n,), dtype=kernel_dtype, device=x.device)
    else:
        assert out.is_contiguous() and out.numel() == n and out.dtype == kernel_dtype == output_dtype
    with torch.cuda.device(x.device):
        rc = _lib.load().mxq_mxfp_qdq(x.data_ptr(), _lib.DTYPE_ID[x.dtype], out.data_ptr(), _lib.DTYPE_ID[kernel_dtype],
                                      n, B, eb, fb, fin, rm, _lib.stream_ptr(x.device))
    _lib.check(rc, "mxq_mxfp_qdq")
    return out if kernel_dtype == output_dtype else out.to(output_dtype)


# --- blocks along a dimension that is not the contiguous one -------------------------------------------
# The tensor is seen as [outer, D, inner]; the kernels read / write that layout directly and produce the
# bytes the permute + flat route would.  Each function returns None when the library does not cover the
# case (MXQ_ESIZE), and the caller then takes that route.
_ESIZE = -3


def _split(shape: tuple[int, ...], block_dim: int) -> tuple[int, int, int]:
    outer = 1
    for s in shape[:block_dim]:
        outer *= s
    inner = 1
    for s in shape[block_dim + 1:]:
        inner *= s
    return outer, shape[block_dim], inner


def extract_mxfp_components_strided(x: Tensor, block_dim: int, mxfp_meta: MXFPMeta) -> tuple[Tensor, Tensor] | None:
    """Contiguous N-D tensor, blocks along ``block_dim`` (non-negative) -> ``(scales, elements)`` in the
    order ``flatten_for_quantize`` would give them."""
    _lib.require_cuda(x, "extract_mxfp_components")
    x = _as_kernel_input(x)
    B, eb, fb, fin, rm = _fmt(mxfp_meta)
    outer, D, inner = _split(tuple(x.shape), block_dim)
    n = x.numel()
    if n == 0 or n % B != 0:
        return None
    scales = torch.empty((n // B, 1), dtype=torch.uint8, device=x.device)
    elements = torch.empty((n // B, B), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.load().mxq_mxfp_extract_strided(x.data_ptr(), _lib.DTYPE_ID[x.dtype], scales.data_ptr(), elements.data_ptr(),
                                                  outer, D, inner, B, eb, fb, fin, rm, _lib.stream_ptr(x.device))
    if rc == _ESIZE:
        return None
    _lib.check(rc, "mxq_mxfp_extract_strided")
    return scales, elements


def compose_mxfp_tensor_strided(scales: Tensor, elements: Tensor, shape: tuple[int, ...], block_dim: int,
                                mxfp_meta: MXFPMeta, output_dtype: torch.dtype) -> Tensor | None:
    """``(scales, elements)`` -> contiguous tensor of ``shape`` whose blocks run along ``block_dim``."""
    _lib.require_cuda(elements, "compose_mxfp_tensor")
    assert scales.dtype == torch.uint8
    assert elements.dtype == torch.uint8
    if output_dtype not in _lib.DTYPE_ID:
        return None
    scales, elements = scales.contiguous(), elements.contiguous()
    B, eb, fb, fin, _ = _fmt(mxfp_meta)
    outer, D, inner = _split(tuple(shape), block_dim)
    n = elements.numel()
    assert n == scales.numel() * B and n == outer * D * inner, "elements, scales and shape disagree"
    if n == 0:
        return None
    out = torch.empty(tuple(shape), dtype=output_dtype, device=elements.device)
    with torch.cuda.device(elements.device):
        rc = _lib.load().mxq_mxfp_compose_strided(scales.data_ptr(), elements.data_ptr(), out.data_ptr(), _lib.DTYPE_ID[output_dtype],
                                                  outer, D, inner, B, eb, fb, fin, _lib.stream_ptr(elements.device))
    if rc == _ESIZE:
        return None
    _lib.check(rc, "mxq_mxfp_compose_strided")
    return out


def quantize_dequantize_strided(x: Tensor, block_dim: int, mxfp_meta: MXFPMeta, output_dtype: torch.dtype) -> Tensor | None:
    """Fused extract + compose with blocks along ``block_dim``; the result keeps the layout of ``x``."""
    _lib.require_cuda(x, "quantize_dequantize")
    if x.dtype not in _lib.DTYPE_ID or output_dtype != x.dtype or x.numel() == 0:
        return None
    x = x.contiguous()
    B, eb, fb, fin, rm = _fmt(mxfp_meta)
    outer, D, inner = _split(tuple(x.shape), block_dim)
    out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        rc = _lib.load().mxq_mxfp_qdq_strided(x.data_ptr(), _lib.DTYPE_ID[x.dtype], out.data_ptr(), _lib.DTYPE_ID[x.dtype],
                                              outer, D, inner, B, eb, fb, fin, rm, _lib.stream_ptr(x.device))
    if rc == _ESIZE:
        return None
    _lib.check(rc, "mxq_mxfp_qdq_strided")
    return out
