"""Pieces shared by ``minifloat_linear`` and ``mxfp_linear``."""

from __future__ import annotations

import re
from typing import NamedTuple

_LAYER_RE = re.compile(r"X(q?)W(q?)")


class LinearKind(NamedTuple):
    x_quantised: bool
    w_quantised: bool
    b_quantised: bool


def parse_layer_type(layer_type: str) -> LinearKind:
    """``'XqWqB'`` -> which of activation / weight / bias are quantised.

    The layer type is one of XWB, XWBq, XWqB, XWqBq, XqWB, XqWBq, XqWqB, XqWqBq; anything
    that names no X?W? pair raises ``NotImplementedError`` like the reference's dispatchers.
    """
    m = _LAYER_RE.search(layer_type)
    if m is None:
        raise NotImplementedError(f"Layer type {layer_type} not implemented")
    return LinearKind(bool(m.group(1)), bool(m.group(2)), "Bq" in layer_type)


def check_backend(backend: str) -> None:
    if backend not in ("separate", "fused"):
        raise NotImplementedError(f"backend {backend!r} not implemented")
