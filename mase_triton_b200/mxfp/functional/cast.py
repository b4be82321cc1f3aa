"""Public MXFP casts (reference: ``src/mase_triton/mxfp/functional/cast.py:11-129``)."""

from __future__ import annotations

import torch
from torch import Tensor

from .. import kernels
from ..helpers import flatten_for_quantize, permute_for_dequantize
from ..meta import MXFPMeta, MXFPTensorMeta


def _blocks_are_strided(shape, block_dim: int) -> bool:
    """True when some dimension after ``block_dim`` has more than one entry, i.e. the reference would
    need a permuted copy to make the blocks contiguous."""
    d = block_dim % len(shape)
    return any(s != 1 for s in tuple(shape)[d + 1:])


def extract_mxfp_components(tensor: Tensor, block_dim: int, mxfp_meta: MXFPMeta) -> tuple[Tensor, Tensor, MXFPTensorMeta]:
    """Quantise ``tensor`` with 1-D blocks running along ``block_dim``.

    Returns ``(scales, elements, tensor_meta)``: uint8 ``scales`` of shape ``[n_blocks, 1]``, uint8
    ``elements`` of shape ``[n_blocks, block_size]`` (one code per byte) and the record needed to
    restore the original shape, dtype and layout.
    """
    ndim = tensor.ndim
    assert -ndim <= block_dim < ndim
    pair = None
    if _blocks_are_strided(tensor.shape, block_dim) and tensor.is_cuda:
        pair = kernels.extract_mxfp_components_strided(tensor, block_dim % ndim, mxfp_meta)
    if pair is None:
        pair = kernels.extract_mxfp_components(flatten_for_quantize(tensor, block_dim), mxfp_meta=mxfp_meta)
    scales, elements = pair
    tensor_meta = MXFPTensorMeta(device=tensor.device, dtype=tensor.dtype, shape=tensor.shape,
                                 block_dim=block_dim, meta=mxfp_meta)
    return scales, elements, tensor_meta


# name used by the reference's README for the same function
extract_mxfp_tensor = extract_mxfp_components


def compose_mxfp_tensor(scales: Tensor, elements: Tensor, tensor_meta: MXFPTensorMeta,
                        output_dtype: torch.dtype | None = None) -> Tensor:
    """Dequantise to the original shape; ``output_dtype`` defaults to the recorded source dtype."""
    if output_dtype is None:
        output_dtype = getattr(torch, tensor_meta.dtype)
    shape = tuple(tensor_meta.shape)
    if _blocks_are_strided(shape, tensor_meta.block_dim) and elements.is_cuda:
        out = kernels.compose_mxfp_tensor_strided(scales, elements, shape, tensor_meta.block_dim % len(shape),
                                                  tensor_meta.meta, output_dtype)
        if out is not None:
            return out
    flat = kernels.compose_mxfp_tensor(scales=scales, elements=elements, mxfp_meta=tensor_meta.meta, output_dtype=output_dtype)
    return permute_for_dequantize(flat, ori_shape=tensor_meta.shape, block_dim=tensor_meta.block_dim)


def quantize_dequantize(tensor: Tensor, block_dim: int, mxfp_meta: MXFPMeta, output_dtype: torch.dtype | None = None) -> Tensor:
    """``compose(extract(tensor))`` in one fused kernel (no codes written to memory)."""
    ndim = tensor.ndim
    assert -ndim <= block_dim < ndim
    if _blocks_are_strided(tensor.shape, block_dim) and tensor.is_cuda:
        out = kernels.quantize_dequantize_strided(tensor, block_dim % ndim, mxfp_meta,
                                                  tensor.dtype if output_dtype is None else output_dtype)
        if out is not None:
            return out
    flat = kernels.quantize_dequantize(flatten_for_quantize(tensor, block_dim), mxfp_meta,
                                       tensor.dtype if output_dtype is None else output_dtype)
    return permute_for_dequantize(flat, ori_shape=tuple(tensor.shape), block_dim=block_dim)
