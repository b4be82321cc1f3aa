"""Pin the C oracle against the reference's own fake path, bit for bit.

Run where the reference checkout is available:

    python oracle/validate_against_reference.py path/to/mase-triton/src

It imports ``mase_triton.minifloat.fake`` / ``mase_triton.mxfp.fake`` from the
reference and compares them with ``oracle`` on random and adversarial inputs.
Exit code 0 means every comparison was bit-exact.  Not used at run time by the
product, the tests or the benchmark.
"""

from __future__ import annotations

import os
import sys
from pathlib import Path
from types import SimpleNamespace

import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
if len(sys.argv) < 2 and "MASE_TRITON_SRC" not in os.environ:
    raise SystemExit("usage: python " + sys.argv[0] + " <path to the src/ folder of a mase-triton checkout> (or set MASE_TRITON_SRC)")
REF_SRC = sys.argv[1] if len(sys.argv) > 1 else os.environ["MASE_TRITON_SRC"]
sys.path.insert(0, REF_SRC)

import oracle  # noqa: E402
from mase_triton.minifloat import fake as ref_mf  # noqa: E402
from mase_triton.minifloat.meta import MinifloatMeta  # noqa: E402
from mase_triton.mxfp import fake as ref_mx  # noqa: E402
from mase_triton.mxfp.meta import MXFPMeta  # noqa: E402

FORMATS = [(4, 3), (5, 2), (2, 3), (3, 2), (2, 1), (8, 7), (5, 10), (3, 4), (1, 1), (7, 8), (10, 5)]
MX_FORMATS = [(4, 3), (5, 2), (2, 3), (3, 2), (2, 1)]
failures = 0


def bits(t: torch.Tensor) -> torch.Tensor:
    if t.dtype == torch.float32:
        return t.view(torch.int32)
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.view(torch.int16)
    return t


def check(name: str, a: torch.Tensor, b: torch.Tensor):
    global failures
    a, b = bits(a), bits(b)
    if a.shape != b.shape or a.dtype != b.dtype:
        print(f"FAIL {name}: shape/dtype {a.shape}/{a.dtype} vs {b.shape}/{b.dtype}")
        failures += 1
        return
    neq = (a.to(torch.int64) != b.to(torch.int64))
    if neq.any():
        idx = neq.flatten().nonzero()[:5].flatten().tolist()
        print(f"FAIL {name}: {int(neq.sum())} mismatches, first at {idx}: "
              f"{[hex(int(a.flatten()[i]) & 0xFFFFFFFF) for i in idx]} vs {[hex(int(b.flatten()[i]) & 0xFFFFFFFF) for i in idx]}")
        failures += 1


def adversarial_fp32(n: int, g: torch.Generator) -> torch.Tensor:
    """Random bit patterns mixed with values near binade edges, specials and subnormals."""
    raw = torch.randint(-(2**31), 2**31, (n,), generator=g, dtype=torch.int64).to(torch.int32)
    x = raw.view(torch.float32).clone()
    k = n // 8
    # moderate-range normals so every format sees in-range values
    x[:k] = torch.randn(k, generator=g) * torch.exp2(torch.randint(-20, 20, (k,), generator=g).float())
    # values with all-ones / near all-ones mantissas (carry cases) and exact ties
    e = torch.randint(1, 255, (k,), generator=g, dtype=torch.int64)
    m = (0x7FFFFF - torch.randint(0, 1 << 16, (k,), generator=g, dtype=torch.int64))
    s = torch.randint(0, 2, (k,), generator=g, dtype=torch.int64) << 31
    x[k:2 * k] = ((s | (e << 23) | m) & 0xFFFFFFFF).to(torch.int64).apply_(lambda v: v - (1 << 32) if v >= (1 << 31) else v).to(torch.int32).view(torch.float32)
    tie = (torch.randint(0, 1 << 10, (k,), generator=g, dtype=torch.int64) << 13)
    x[2 * k:3 * k] = (((e << 23) | tie)).to(torch.int32).view(torch.float32)
    specials = torch.tensor([0.0, -0.0, float("inf"), float("-inf"), float("nan"), -float("nan"), 1e-45, -1e-40,
                             2.0**-126, 2.0**-127, 1.9375, 1.875, 3.875, 63488.0, 65536.0, 114688.0, 3.4e38, -3.4e38,
                             448.0, 480.0, 500.0, 2.0**-14, 1.5 * 2.0**-15, 2.0**-15, 2.0**-16, 0.5, 0.625, 0.75],
                            dtype=torch.float32)
    x[3 * k:3 * k + specials.numel()] = specials
    # signalling NaNs with random payloads
    snan = (0x7F800001 + torch.randint(0, 0x3FFFFF, (64,), generator=g, dtype=torch.int64)).to(torch.int32)
    x[4 * k:4 * k + 64] = snan.view(torch.float32)
    return x


def main() -> int:
    g = torch.Generator().manual_seed(1234)

    # 1. floor(log2f) round-up table against torch.log2 on this host, for every binade
    top = 96
    for e in range(-126, 128):
        mant = torch.arange(0x7FFFFF - top + 1, 0x7FFFFF + 1, dtype=torch.int64)
        v = (((e + 127) << 23) | mant).to(torch.int32).view(torch.float32)
        # long vector (SIMD body) and one-element tensors (scalar tail) must agree
        l_vec = torch.cat([v, v, v]).log2().floor().to(torch.int32)[:top]
        l_tail = torch.stack([v[i:i + 1].log2().floor().to(torch.int32)[0] for i in range(top - 8, top)])
        cnt = int((l_vec == e + 1).sum())
        if cnt != oracle.log2_roundup_count(e) or not torch.equal(l_vec[top - 8:], l_tail):
            print(f"FAIL log2 table e={e}: torch {cnt} oracle {oracle.log2_roundup_count(e)}")
            global failures
            failures += 1
        # the values that round up must be exactly the topmost ones
        if cnt and not bool((l_vec[top - cnt:] == e + 1).all()):
            print(f"FAIL log2 table e={e}: round-up set is not a suffix")
            failures += 1
    # lower mantissas never round up / down
    for _ in range(4):
        v = torch.randint(1 << 23, 0x7F800000, (1 << 20,), generator=g, dtype=torch.int64).to(torch.int32).view(torch.float32)
        l = v.log2().floor().to(torch.int32)
        vb = v.view(torch.int32)
        e = (vb >> 23) - 127
        near = (0x7FFFFF - (vb & 0x7FFFFF)) < 64
        check("log2 bulk", l[~near], e[~near])
    print("log2 table checked")

    # 2. minifloat extract
    x = adversarial_fp32(1 << 18, g)
    for eb, fb in FORMATS:
        for fin in (True, False):
            for rm in ("rn", "ru", "rd", "rz"):
                meta = MinifloatMeta(exp_bits=eb, frac_bits=fb, is_finite=fin, round_mode=rm)
                check(f"mf extract e{eb}m{fb} fin={fin} {rm}", oracle.extract_minifloat_component(x, meta),
                      ref_mf.extract_minifloat_component(x, meta))
    for dt in (torch.bfloat16, torch.float16):
        allbits = torch.arange(-(2**15), 2**15, dtype=torch.int32).to(torch.int16).view(dt)
        for eb, fb in FORMATS[:7]:
            meta = MinifloatMeta(exp_bits=eb, frac_bits=fb, is_finite=True, round_mode="rn")
            check(f"mf extract all {dt} e{eb}m{fb}", oracle.extract_minifloat_component(allbits, meta),
                  ref_mf.extract_minifloat_component(allbits, meta))
    print("minifloat extract checked")

    # 3. minifloat compose: all 65536 codes
    codes = torch.arange(0, 65536, dtype=torch.int32).to(torch.uint16)
    for eb, fb in FORMATS:
        for fin in (True, False):
            meta = MinifloatMeta(exp_bits=eb, frac_bits=fb, is_finite=fin, round_mode="rn")
            for dt in (torch.float32, torch.bfloat16, torch.float16):
                check(f"mf compose e{eb}m{fb} fin={fin} {dt}", oracle.compose_minifloat_component(codes, meta, dt),
                      ref_mf.compose_minifloat_component(codes, meta, dt))
    print("minifloat compose checked")

    # 4. MXFP extract
    for B in (32, 8, 16, 5):
        nb = 4096
        base = torch.randn(nb, B, generator=g) * torch.exp2(torch.randint(-130, 128, (nb, 1), generator=g).float())
        # near power-of-two block maxima (log2 round-up quirk)
        e = torch.randint(1, 255, (nb,), generator=g, dtype=torch.int64)
        m = 0x7FFFFF - torch.randint(0, 64, (nb,), generator=g, dtype=torch.int64)
        base[::2, 0] = ((e << 23) | m).to(torch.int32).view(torch.float32)[::2]
        # special blocks
        base[1] = 0.0
        base[3] = torch.tensor(1e-40)
        base[5, 0] = float("inf")
        base[7, 1] = float("-inf")
        base[9, 2] = float("nan")
        base[11] = 3e38
        base[11, 1:3] = torch.tensor([1.0, -1e30])
        base[13, :3] = torch.tensor([2.0**-126, 1.5 * 2.0**-126, 2.0**-120])
        base[15, :3] = torch.tensor([-0.0, 1e-45, -1e-39])
        base[17, 0] = 2.0**120
        base[17, 1:5] = torch.tensor([-2.0**-37, -1.5 * 2.0**-38, -2.0**-38, -2.0**-40])
        for dt in (torch.float32, torch.bfloat16, torch.float16):
            xin = base.to(dt).flatten()
            for eb, fb in MX_FORMATS:
                for fin in (True, False):
                    for rm in ("rn", "rz", "ru", "rd"):
                        meta = MXFPMeta(block_size=B, scale_exp_bits=8, element_exp_bits=eb, element_frac_bits=fb,
                                        element_is_finite=fin, round_mode=rm)
                        s_o, e_o = oracle.extract_mxfp_components(xin, meta)
                        s_r, e_r = ref_mx.extract_mxfp_components(xin, meta)
                        tag = f"mx extract B{B} {dt} e{eb}m{fb} fin={fin} {rm}"
                        check(tag + " scales", s_o, s_r)
                        check(tag + " elements", e_o, e_r)
    print("mxfp extract checked")

    # 5. MXFP compose: every (scale, code) pair
    sc = torch.arange(256, dtype=torch.int32).to(torch.uint8).repeat_interleave(8).reshape(-1, 1)   # 2048 blocks
    el = torch.arange(256, dtype=torch.int32).to(torch.uint8).repeat(256).reshape(-1, 32)
    for eb, fb in MX_FORMATS:
        for fin in (True, False):
            meta = MXFPMeta(block_size=32, scale_exp_bits=8, element_exp_bits=eb, element_frac_bits=fb,
                            element_is_finite=fin, round_mode="rn")
            for dt in (torch.float32, torch.bfloat16, torch.float16):
                check(f"mx compose e{eb}m{fb} fin={fin} {dt}", oracle.compose_mxfp_tensor(sc, el, meta, dt),
                      ref_mx.compose_mxfp_tensor(sc, el, meta, dt))
    print("mxfp compose checked")

    print("FAILURES:", failures)
    return 1 if failures else 0


if __name__ == "__main__":
    sys.exit(main())
