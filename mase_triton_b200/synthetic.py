"""Seeded synthetic inputs with the shapes and value distributions of the five benchmark
configurations.  Everything is generated on the CPU with ``torch.Generator`` so the CUDA path and
the CPU oracle see identical bits; callers move the tensors to a device themselves.

``rows`` lets a caller generate a row slice of a configuration (row sharding across GPUs, or a
bounded CPU sample): the slice is cut from the full tensor, so values do not depend on how the
work is split.
"""

from __future__ import annotations

import torch


def _rows(x: torch.Tensor, rows: slice | None) -> torch.Tensor:
    return x if rows is None else x[rows].contiguous()


def cfg1_mxfp8_fp32(shape=(4096, 4096), seed: int = 0, rows: slice | None = None) -> torch.Tensor:
    """fp32 N(0,1) with 0.1% of the entries multiplied by 2^12 (outliers)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g)
    mask = torch.rand(shape, generator=g) < 1e-3
    x[mask] *= 2.0**12
    return _rows(x, rows)


def cfg2_minifloat_fp32(shape=(8192, 8192), seed: int = 0, rows: slice | None = None) -> torch.Tensor:
    """fp32 magnitudes log-uniform over 2^-24 .. 2^20 with random sign; 0.01% each of the entries
    are zeros (random sign), infinities (random sign) and NaN."""
    g = torch.Generator().manual_seed(seed)
    e = torch.rand(shape, generator=g) * 44.0 - 24.0
    x = torch.exp2(e)
    sign = torch.randint(0, 2, shape, generator=g, dtype=torch.int8)
    x = torch.where(sign.bool(), -x, x)
    pick = torch.rand(shape, generator=g)
    x[pick < 1e-4] = 0.0
    x[(pick >= 1e-4) & (pick < 2e-4)] = float("inf")
    x[(pick >= 2e-4) & (pick < 3e-4)] = float("nan")
    flip = (pick < 2e-4) & sign.bool()          # -0.0 and -inf for about half of them
    x[flip] = -x[flip]
    return _rows(x, rows)


def cfg3_mxfp4_bf16(shape=(16384, 8192), seed: int = 0, rows: slice | None = None) -> torch.Tensor:
    """bf16 activation-like tensor: N(0,1) times a per-column lognormal(0, 1.5) channel scale."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(shape, generator=g)
    ch = torch.exp(1.5 * torch.randn(shape[1], generator=g))
    return _rows((x * ch).to(torch.bfloat16), rows)


def cfg4_linear_operands(m: int = 8192, n: int = 14336, k: int = 4096, seed: int = 0):
    """bf16 x [m,k] ~ N(0,1) and W [n,k] ~ N(0, 0.02)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16)
    w = (0.02 * torch.randn(n, k, generator=g)).to(torch.bfloat16)
    return x, w


# (name, out_features, in_features) of one Llama-3-8B-shaped decoder layer
CFG5_PROJECTIONS = (("q", 4096, 4096), ("k", 1024, 4096), ("v", 1024, 4096), ("o", 4096, 4096),
                    ("gate", 14336, 4096), ("up", 14336, 4096), ("down", 4096, 14336))


def cfg5_weight(name: str, seed: int = 0) -> torch.Tensor:
    """bf16 N(0, 0.02) weight of one projection."""
    idx = [p[0] for p in CFG5_PROJECTIONS].index(name)
    _, n, k = CFG5_PROJECTIONS[idx]
    g = torch.Generator().manual_seed(seed * 100 + idx + 1)
    return (0.02 * torch.randn(n, k, generator=g)).to(torch.bfloat16)


def cfg5_input(in_features: int, batch: int = 16, seq: int = 2048, seed: int = 0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed * 100 + 99 + in_features)
    return torch.randn(batch, seq, in_features, generator=g).to(torch.bfloat16)
