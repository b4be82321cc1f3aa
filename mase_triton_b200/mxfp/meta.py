"""MXFP (OCP microscaling) format descriptors (reference: ``src/mase_triton/mxfp/meta.py:11-126``).

A block of ``block_size`` consecutive values shares one 8-bit power-of-two scale (E8M0);
each value is a minifloat element of one of five exponent/fraction splits.
"""

from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Literal

from ..minifloat.meta import MinifloatMeta
from ..utils.meta import device_str, dtype_str, shape_tuple

_SCALE_EXP_BITS = (8,)
_ELEMENT_SPLITS = ((4, 3), (5, 2), (2, 3), (3, 2), (2, 1))


@dataclass(frozen=True)
class MXFPMeta:
    block_size: int
    scale_exp_bits: int
    element_exp_bits: int
    element_frac_bits: int
    element_is_finite: bool
    round_mode: Literal["rn", "ru", "rd", "rz"]
    tag: str = ""

    def __post_init__(self):
        assert self.scale_exp_bits in _SCALE_EXP_BITS, (
            f"Invalid exponent bits: {self.scale_exp_bits}. Legal values are: {_SCALE_EXP_BITS}.")
        split = (self.element_exp_bits, self.element_frac_bits)
        assert split in _ELEMENT_SPLITS, (
            f"Invalid element exponent and fraction bits: {split[0]}, {split[1]}. Legal values are: {_ELEMENT_SPLITS}.")

    @property
    def element_meta(self) -> MinifloatMeta:
        """The minifloat format of one element."""
        return MinifloatMeta(exp_bits=self.element_exp_bits, frac_bits=self.element_frac_bits,
                             is_finite=self.element_is_finite, round_mode=self.round_mode)


@dataclass(frozen=True)
class MXFPTensorMeta:
    """Origin of a quantised tensor: device / dtype / shape of the source, the blocked dim, the format."""

    device: str
    dtype: str
    shape: tuple[int, ...]
    block_dim: int
    meta: MXFPMeta

    def __post_init__(self):
        object.__setattr__(self, "device", device_str(self.device))
        object.__setattr__(self, "dtype", dtype_str(self.dtype))
        object.__setattr__(self, "shape", shape_tuple(self.shape))

    def create(self, device=None, dtype=None, shape=None, block_dim: int | None = None,
               meta: MXFPMeta | None = None) -> "MXFPTensorMeta":
        """Copy with some fields replaced (``None`` keeps the current value)."""
        given = dict(device=device, dtype=dtype, shape=shape, block_dim=block_dim, meta=meta)
        return replace(self, **{k: v for k, v in given.items() if v is not None})


def _mx(e: int, m: int, tag: str) -> MXFPMeta:
    return MXFPMeta(block_size=32, scale_exp_bits=8, element_exp_bits=e, element_frac_bits=m,
                    element_is_finite=True, round_mode="rn", tag=tag)


MXFP8_E4M3_fn = _mx(4, 3, "MXFP8_E4M3_fn")
MXFP8_E5M2_fn = _mx(5, 2, "MXFP8_E5M2_fn")
OCP_MXFP6_E2M3 = _mx(2, 3, "OCP_MXFP6_E2M3")
OCP_MXFP6_E3M2 = _mx(3, 2, "OCP_MXFP6_E3M2")
OCP_MXFP4_E2M1 = _mx(2, 1, "OCP_MXFP4_E2M1")
