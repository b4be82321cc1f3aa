"""Shared input generators and comparison helpers for the parity tests."""

from __future__ import annotations

from types import SimpleNamespace

import torch

PRESETS = {"E4M3": (4, 3), "E5M2": (5, 2), "E2M3": (2, 3), "E3M2": (3, 2), "E2M1": (2, 1)}
ROUND_MODES = ("rn", "ru", "rd", "rz")


def mf_meta(eb, fb, is_finite=True, round_mode="rn"):
    """Duck-typed MinifloatMeta for the oracle."""
    return SimpleNamespace(exp_bits=eb, frac_bits=fb, is_finite=is_finite, round_mode=round_mode)


def mx_meta(eb, fb, block_size=32, is_finite=True, round_mode="rn"):
    """Duck-typed MXFPMeta for the oracle."""
    return SimpleNamespace(block_size=block_size, scale_exp_bits=8, element_exp_bits=eb, element_frac_bits=fb,
                           element_is_finite=is_finite, round_mode=round_mode)


def int_bits(x: torch.Tensor) -> torch.Tensor:
    """Integer view of a tensor's storage, widened to int64 for comparison."""
    if x.dtype == torch.float32:
        return x.view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    if x.dtype in (torch.bfloat16, torch.float16):
        return x.view(torch.int16).to(torch.int64) & 0xFFFF
    return x.to(torch.int64)


def assert_bits_equal(got: torch.Tensor, want: torch.Tensor, what: str = "", nan_any_payload_16bit: bool = True):
    """Bit-exact comparison. fp32 compares every bit, NaNs included. For 16-bit floats the
    NaN encoding produced by the host's float conversion is platform-defined, so NaNs only
    have to sit at the same places."""
    got, want = got.cpu(), want.cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} != {tuple(want.shape)}"
    assert got.dtype == want.dtype, f"{what}: dtype {got.dtype} != {want.dtype}"
    g, w = int_bits(got), int_bits(want)
    if nan_any_payload_16bit and got.dtype in (torch.bfloat16, torch.float16):
        gn, wn = got.isnan(), want.isnan()
        assert torch.equal(gn, wn), f"{what}: NaN positions differ"
        g, w = g.masked_fill(gn, 0), w.masked_fill(wn, 0)
    neq = g != w
    if neq.any():
        idx = neq.flatten().nonzero().flatten()[:8].tolist()
        gv = [hex(int(g.flatten()[i])) for i in idx]
        wv = [hex(int(w.flatten()[i])) for i in idx]
        raise AssertionError(f"{what}: {int(neq.sum())} of {neq.numel()} differ; first at {idx}: got {gv} want {wv}")


def from_bits32(bits: torch.Tensor) -> torch.Tensor:
    """int64 tensor of 32-bit patterns -> float32 tensor."""
    b = bits.to(torch.int64) & 0xFFFFFFFF
    b = torch.where(b >= (1 << 31), b - (1 << 32), b)
    return b.to(torch.int32).view(torch.float32)


SPECIALS = [0.0, -0.0, float("inf"), float("-inf"), float("nan"), 1e-45, -1e-40, 2.0**-126, 2.0**-127, 1.9375, 1.875,
            3.875, 3.75, 1.125, 1.375, 1.625, 63488.0, 65536.0, 114688.0, 1e6, 3.4e38, -3.4e38, 448.0, 480.0, 500.0,
            2.0**-14, 1.5 * 2.0**-15, 1.75 * 2.0**-15, 1.25 * 2.0**-15, 2.0**-15, 2.0**-16, 2.0**-17, 0.5, 0.625, 0.75,
            6.0, 7.0, 7.5, 8.0, 28.0, 30.0, 32.0, -6.0, -0.5, 0.25, 0.1875, 0.0625, 2.0**-9, 2.0**-6]


def adversarial_fp32(n: int, seed: int = 1234) -> torch.Tensor:
    """Random bit patterns mixed with in-range normals, carry/tie cases, specials and signalling NaNs."""
    g = torch.Generator().manual_seed(seed)
    x = from_bits32(torch.randint(0, 1 << 32, (n,), generator=g, dtype=torch.int64)).clone()
    k = n // 8
    x[:k] = torch.randn(k, generator=g) * torch.exp2(torch.randint(-20, 20, (k,), generator=g).float())
    e = torch.randint(1, 255, (k,), generator=g, dtype=torch.int64)
    s = torch.randint(0, 2, (k,), generator=g, dtype=torch.int64) << 31
    m = 0x7FFFFF - torch.randint(0, 1 << 16, (k,), generator=g, dtype=torch.int64)
    x[k:2 * k] = from_bits32(s | (e << 23) | m)
    tie = torch.randint(0, 1 << 10, (k,), generator=g, dtype=torch.int64) << 13
    x[2 * k:3 * k] = from_bits32(s | (e << 23) | tie)
    near_tie = tie + torch.randint(-3, 4, (k,), generator=g, dtype=torch.int64).clamp(0)
    x[3 * k:4 * k] = from_bits32(s | (e << 23) | near_tie)
    sp = torch.tensor(SPECIALS, dtype=torch.float32)
    x[4 * k:4 * k + sp.numel()] = sp
    snan = 0x7F800001 + torch.randint(0, 0x3FFFFF, (32,), generator=g, dtype=torch.int64)
    x[5 * k:5 * k + 32] = from_bits32(snan)
    x[5 * k + 32:5 * k + 64] = from_bits32(snan | (1 << 31))
    return x


def adversarial_mx_blocks(n_blocks: int, B: int, seed: int = 99) -> torch.Tensor:
    """[n_blocks, B] fp32: wide dynamic range, block maxima just below powers of two, zero /
    subnormal / Inf / NaN blocks, huge in-block ratios."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n_blocks, B, generator=g) * torch.exp2(torch.randint(-130, 128, (n_blocks, 1), generator=g).float())
    e = torch.randint(1, 255, (n_blocks,), generator=g, dtype=torch.int64)
    m = 0x7FFFFF - torch.randint(0, 64, (n_blocks,), generator=g, dtype=torch.int64)
    top = from_bits32((e << 23) | m)
    x[::2, 0] = top[::2]
    if n_blocks >= 24:
        x[1] = 0.0
        x[3] = 1e-40
        x[5, 0] = float("inf")
        x[7, min(1, B - 1)] = float("-inf")
        x[9, min(2, B - 1)] = float("nan")
        x[11] = 3e38
        x[11, 1:3] = torch.tensor([1.0, -1e30])[: max(0, min(2, B - 1))]
        x[13, :3] = torch.tensor([2.0**-126, 1.5 * 2.0**-126, 2.0**-120])[: min(3, B)]
        x[15, :3] = torch.tensor([-0.0, 1e-45, -1e-39])[: min(3, B)]
        x[17, 0] = 2.0**120
        x[17, 1:5] = torch.tensor([-(2.0**-37), -1.5 * 2.0**-38, -(2.0**-38), -(2.0**-40)])[: max(0, min(4, B - 1))]
        x[19] = 0.0
        x[19, 0] = -0.0
        x[21, :6] = torch.tensor([1, -0.3, 0.01, 448, 480, 500.0])[: min(6, B)]
        x[23] = -1e-39
    return x
