"""Layout helpers: blocks always run along the last axis of a flattened tensor
(reference: ``src/mase_triton/mxfp/helpers.py:4-47``)."""

from __future__ import annotations

from torch import Tensor


def flatten_for_quantize(tensor: Tensor, block_dim: int) -> Tensor:
    """Move ``block_dim`` to the end and flatten (a view when it already is the last axis)."""
    return tensor.movedim(block_dim % tensor.ndim, -1).flatten()


def permute_for_dequantize(flatten_tensor: Tensor, ori_shape: tuple[int, ...], block_dim: int) -> Tensor:
    """Inverse of :func:`flatten_for_quantize`: back to ``ori_shape`` (possibly a permuted view)."""
    ndim = len(ori_shape)
    block_dim %= ndim
    moved = list(ori_shape)
    moved.append(moved.pop(block_dim))
    return flatten_tensor.reshape(moved).movedim(-1, block_dim)
