"""Small helpers shared by the PTQ layers (reference: ``src/mase_triton/utils/qlayer.py:4-21``)."""

from __future__ import annotations

import torch


class ChangeDtypeError(Exception):
    """Raised when ``.to()`` / ``.half()`` etc. would re-type a tensor of integer codes."""

    def __init__(self, message: str = "Changing dtype is not allowed."):
        self.message = message
        super().__init__(message)


def _canonical(device) -> torch.device:
    d = torch.device(device)
    return torch.device("cuda", 0) if d.type == "cuda" and d.index is None else d


def devices_equal(device1, device2) -> bool:
    """True when both name the same device; a bare ``cuda`` means ``cuda:0``."""
    return _canonical(device1) == _canonical(device2)
