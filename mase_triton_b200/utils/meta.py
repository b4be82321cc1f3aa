"""String/tuple normalisers used by the tensor-meta records.

Counterpart of the reference's ``src/mase_triton/utils/meta.py:4-25``: metas store the
device and dtype as plain strings and the shape as a plain tuple so they can be
printed, compared and pickled without holding torch objects.
"""

from __future__ import annotations

import torch


def device_str(device) -> str:
    """``torch.device('cuda:0')`` -> ``'cuda:0'``; strings pass through."""
    return device if isinstance(device, str) else str(device)


def dtype_str(dtype) -> str:
    """``torch.bfloat16`` -> ``'bfloat16'``; strings pass through."""
    return dtype if isinstance(dtype, str) else str(dtype).removeprefix("torch.")


def shape_tuple(shape) -> tuple[int, ...]:
    """``torch.Size`` -> ``tuple``; anything else passes through."""
    return tuple(shape) if isinstance(shape, torch.Size) else shape
