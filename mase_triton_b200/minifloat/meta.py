"""Minifloat format descriptors (reference: ``src/mase_triton/minifloat/meta.py:48-124``).

A minifloat is sign + ``exp_bits`` + ``frac_bits`` (fewer than 16 bits in total, so a
code fits a uint16).  ``is_finite=True`` means the all-ones exponent encodes ordinary
numbers; otherwise it is reserved for Inf/NaN.
"""

from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Literal

from ..utils.meta import device_str, dtype_str, shape_tuple


@dataclass(frozen=True)
class MinifloatMeta:
    exp_bits: int
    frac_bits: int
    is_finite: bool
    round_mode: Literal["rn", "rd", "ru", "rz"]
    tag: str = ""

    def __post_init__(self):
        assert self.exp_bits > 0
        assert self.frac_bits > 0
        assert self.exp_bits + self.frac_bits < 16

    # -- derived quantities; each mirrors a `_calc_*` helper of the reference (meta.py:10-45) --
    @property
    def exp_bias(self) -> int:
        return 2 ** (self.exp_bits - 1) - 1

    @property
    def n_bits(self) -> int:
        return 1 + self.exp_bits + self.frac_bits

    @property
    def max_normal(self) -> float:
        top = 2**self.exp_bits - (1 if self.is_finite else 2)
        return 2.0 ** (top - self.exp_bias) * (2.0 - 2.0**-self.frac_bits)

    @property
    def min_normal(self) -> float:
        return 2.0 ** (1 - self.exp_bias)

    @property
    def max_subnormal(self) -> float:
        return self.min_normal * (1.0 - 2.0**-self.frac_bits)

    @property
    def min_subnormal(self) -> float:
        return self.min_normal * 2.0**-self.frac_bits


def _preset(e: int, m: int, tag: str) -> MinifloatMeta:
    return MinifloatMeta(exp_bits=e, frac_bits=m, is_finite=True, round_mode="rn", tag=tag)


FP8_E4M3_fn = _preset(4, 3, "FP8_E4M3_fn")
FP8_E5M2_fn = _preset(5, 2, "FP8_E5M2_fn")
FP6_E2M3_fn = _preset(2, 3, "FP6_E2M3_fn")
FP6_E3M2_fn = _preset(3, 2, "FP6_E3M2_fn")
FP4_E2M1_fn = _preset(2, 1, "FP4_E2M1_fn")


@dataclass
class MinifloatTensorMeta:
    """Where a quantised tensor came from: device, dtype and shape of the original plus its format."""

    device: str
    dtype: str
    shape: tuple[int, ...]
    meta: MinifloatMeta

    def __post_init__(self):
        self.device = device_str(self.device)
        self.dtype = dtype_str(self.dtype)
        self.shape = shape_tuple(self.shape)

    def create(self, device=None, dtype=None, shape=None, meta: MinifloatMeta | None = None) -> "MinifloatTensorMeta":
        """Copy with some fields replaced (``None`` keeps the current value)."""
        changes = {k: v for k, v in dict(device=device, dtype=dtype, shape=shape, meta=meta).items() if v is not None}
        return replace(self, **changes)
