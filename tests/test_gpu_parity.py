"""Parity of the CUDA path (through the C ABI and the public Python API) with the CPU oracle,
the golden vectors generated from the reference, and the reference's own known answers."""

from __future__ import annotations

import hashlib
import json
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from helpers import (PRESETS, ROUND_MODES, adversarial_fp32, adversarial_mx_blocks, assert_bits_equal, mf_meta, mx_meta)
from mase_triton_b200 import synthetic
from mase_triton_b200.minifloat import functional as MF
from mase_triton_b200.minifloat import kernels as mf_kernels
from mase_triton_b200.minifloat.meta import (FP4_E2M1_fn, FP6_E2M3_fn, FP6_E3M2_fn, FP8_E4M3_fn, FP8_E5M2_fn, MinifloatMeta)
from mase_triton_b200.mxfp import functional as MX
from mase_triton_b200.mxfp import kernels as mx_kernels
from mase_triton_b200.mxfp.meta import (MXFP8_E4M3_fn, MXFP8_E5M2_fn, OCP_MXFP4_E2M1, OCP_MXFP6_E2M3, OCP_MXFP6_E3M2, MXFPMeta)

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).resolve().parent / "golden"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}
DTYPES = (torch.float32, torch.bfloat16, torch.float16)
MX_PRESETS = [MXFP8_E4M3_fn, MXFP8_E5M2_fn, OCP_MXFP6_E2M3, OCP_MXFP6_E3M2, OCP_MXFP4_E2M1]
MF_PRESETS = [FP8_E4M3_fn, FP8_E5M2_fn, FP6_E2M3_fn, FP6_E3M2_fn, FP4_E2M1_fn]
DEV = "cuda:0"


def mxm(eb, fb, B=32, fin=True, rm="rn"):
    return MXFPMeta(block_size=B, scale_exp_bits=8, element_exp_bits=eb, element_frac_bits=fb, element_is_finite=fin, round_mode=rm)


def sha(t: torch.Tensor) -> str:
    t = t.contiguous().cpu()
    return hashlib.sha256((t if t.dtype == torch.uint8 else t.view(torch.uint8)).numpy().tobytes()).hexdigest()


@pytest.fixture(scope="module")
def small():
    return np.load(GOLD / "golden_small.npz")


@pytest.fixture(scope="module")
def digests():
    return json.loads((GOLD / "golden_digests.json").read_text())


def gold_tensor(arr, dtype_name=None):
    t = torch.from_numpy(arr.copy())
    return t.view(torch.bfloat16) if dtype_name == "bfloat16" else t


# ------------------------------------------------------------------ golden vectors from the reference
def test_golden_minifloat(lib, small):
    x = gold_tensor(small["mf_x"]).to(DEV)
    for k in [k for k in small.files if k.startswith("mf_extract/")]:
        _, name, fin, rm = k.split("/")
        eb, fb = PRESETS[name] if name in PRESETS else tuple(int(v) for v in name[1:].split("m"))
        got = mf_kernels.extract_minifloat_component(x, MinifloatMeta(eb, fb, bool(int(fin)), rm))
        assert_bits_equal(got, gold_tensor(small[k]), k)
    codes = gold_tensor(small["mf_codes"]).to(DEV)
    for k in [k for k in small.files if k.startswith("mf_compose/")]:
        _, name, fin, dn = k.split("/")
        eb, fb = PRESETS[name]
        got = mf_kernels.compose_minifloat_component(codes, MinifloatMeta(eb, fb, bool(int(fin)), "rn"), DT[dn])
        assert_bits_equal(got, gold_tensor(small[k], dn), k)


def test_golden_mxfp(lib, small):
    for k in [k for k in small.files if k.startswith("mx_scales/")]:
        _, B, dn, name, fin, rm = k.split("/")
        eb, fb = PRESETS[name]
        meta = mxm(eb, fb, int(B), bool(int(fin)), rm)
        x = gold_tensor(small[f"mx_x/{B}/{dn}"], dn).to(DEV)
        s, e = mx_kernels.extract_mxfp_components(x, meta)
        tail = k[len("mx_scales/"):]
        assert_bits_equal(s, gold_tensor(small[k]), k)
        assert_bits_equal(e, gold_tensor(small["mx_elements/" + tail]), "elements " + tail)
        if rm == "rn":
            want = gold_tensor(small["mx_composed/" + tail], dn)
            assert_bits_equal(mx_kernels.compose_mxfp_tensor(s, e, meta, DT[dn]), want, "composed " + tail)
            assert_bits_equal(mx_kernels.quantize_dequantize(x, meta, DT[dn]), want, "fused qdq " + tail)
    sc, el = gold_tensor(small["mxc_scales"]).to(DEV), gold_tensor(small["mxc_elements"]).to(DEV)
    for k in [k for k in small.files if k.startswith("mxc_out/")]:
        _, name, fin, dn = k.split("/")
        eb, fb = PRESETS[name]
        got = mx_kernels.compose_mxfp_tensor(sc, el, mxm(eb, fb, 32, bool(int(fin))), DT[dn])
        assert_bits_equal(got, gold_tensor(small[k], dn), k)


# ------------------------------------------------------------------ minifloat vs oracle
@pytest.mark.parametrize("eb,fb", list(PRESETS.values()) + [(8, 7), (5, 10), (3, 4), (1, 1), (7, 8)])
@pytest.mark.parametrize("fin", [True, False])
def test_minifloat_extract_vs_oracle(lib, eb, fb, fin):
    x = adversarial_fp32((1 << 16) + 37)            # odd length: vector body + scalar tail
    xg = x.to(DEV)
    for rm in ROUND_MODES:
        meta = MinifloatMeta(eb, fb, fin, rm)
        assert_bits_equal(mf_kernels.extract_minifloat_component(xg, meta), oracle.extract_minifloat_component(x, meta), f"{meta}")


@pytest.mark.parametrize("meta", MF_PRESETS, ids=lambda m: m.tag)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_minifloat_every_16bit_input(lib, meta, dtype):
    x = torch.arange(-(2**15), 2**15, dtype=torch.int32).to(torch.int16).view(dtype)
    codes, tm = MF.extract_minifloat_component(x.to(DEV), meta)
    assert codes.dtype == torch.uint16 and codes.shape == x.shape and tm.dtype == str(dtype)[6:]
    want_codes = oracle.extract_minifloat_component(x, meta)
    assert_bits_equal(codes, want_codes, "codes")
    assert_bits_equal(MF.compose_minifloat_component(codes, tm), oracle.compose_minifloat_component(want_codes, meta, dtype), "composed")
    assert_bits_equal(MF.quantize_dequantize(x.to(DEV), meta), oracle.quantize_dequantize_minifloat(x, meta), "fused qdq")


@pytest.mark.parametrize("eb,fb", list(PRESETS.values()) + [(8, 7), (5, 10), (3, 4)])
@pytest.mark.parametrize("fin", [True, False])
def test_minifloat_compose_all_codes(lib, eb, fb, fin):
    codes = torch.arange(0, 65536, dtype=torch.int32).to(torch.uint16)
    meta = MinifloatMeta(eb, fb, fin, "rn")
    for dt in DTYPES:
        got = mf_kernels.compose_minifloat_component(codes.to(DEV), meta, dt)
        assert_bits_equal(got, oracle.compose_minifloat_component(codes, meta, dt), f"{meta} {dt}")


@pytest.mark.parametrize("in_dt", DTYPES)
@pytest.mark.parametrize("out_dt", DTYPES)
def test_minifloat_qdq_dtype_matrix(lib, in_dt, out_dt):
    x = adversarial_fp32(1 << 15, seed=3).to(in_dt)
    for meta in (FP8_E5M2_fn, FP4_E2M1_fn, MinifloatMeta(5, 2, False, "rn"), MinifloatMeta(4, 3, True, "ru")):
        got = MF.quantize_dequantize(x.to(DEV), meta, output_dtype=out_dt)
        assert_bits_equal(got, oracle.quantize_dequantize_minifloat(x, meta, out_dt), f"{meta} {in_dt}->{out_dt}")


def test_minifloat_unaligned_and_empty(lib):
    x = adversarial_fp32(4099)
    xg = x.to(DEV)
    for off in (1, 2, 3):      # views that start 4, 8, 12 bytes into the allocation
        got = MF.quantize_dequantize(xg[off:], FP8_E4M3_fn)
        assert_bits_equal(got, oracle.quantize_dequantize_minifloat(x[off:], FP8_E4M3_fn), f"offset {off}")
    e, tm = MF.extract_minifloat_component(torch.empty(0, 5, device=DEV), FP8_E4M3_fn)
    assert e.shape == (0, 5) and MF.compose_minifloat_component(e, tm).shape == (0, 5)
    nc = xg[:4096].reshape(64, 64).t()                       # non-contiguous input
    assert_bits_equal(MF.quantize_dequantize(nc, FP6_E3M2_fn), oracle.quantize_dequantize_minifloat(x[:4096].reshape(64, 64).t(), FP6_E3M2_fn), "transposed")


# reference known answers: test/test_minifloat_fake.py:58-70 and :110-123
def test_fp4_code_table(lib):
    codes = torch.arange(16, dtype=torch.int32).to(torch.uint16).to(DEV)
    got = mf_kernels.compose_minifloat_component(codes, FP4_E2M1_fn, torch.float32).cpu()
    want = torch.tensor([0, 0.5, 1, 1.5, 2, 3, 4, 6, -0.0, -0.5, -1, -1.5, -2, -3, -4, -6])
    assert torch.equal(got, want) and got[8].signbit()


@pytest.mark.parametrize("meta", MF_PRESETS, ids=lambda m: m.tag)
def test_saturation(lib, meta):
    x = torch.ones(8, device=DEV) * meta.max_normal * 2
    assert bool((MF.quantize_dequantize(x, meta) == meta.max_normal).all())
    q, tm = MF.extract_minifloat_component(x, meta)
    assert bool((MF.compose_minifloat_component(q, tm, torch.float32) == meta.max_normal).all())


# ------------------------------------------------------------------ MXFP vs oracle
@pytest.mark.parametrize("name", list(PRESETS))
@pytest.mark.parametrize("B", [32, 8, 16, 5])
def test_mxfp_extract_compose_vs_oracle(lib, name, B):
    eb, fb = PRESETS[name]
    base = adversarial_mx_blocks(4104, B)          # 4104 blocks: not a multiple of the CTA tile
    for dt in DTYPES:
        x = base.to(dt).flatten()
        xg = x.to(DEV)
        for fin in (True, False):
            for rm in (ROUND_MODES if dt == torch.float32 else ("rn",)):
                meta = mxm(eb, fb, B, fin, rm)
                s, e = mx_kernels.extract_mxfp_components(xg, meta)
                s_o, e_o = oracle.extract_mxfp_components(x, mx_meta(eb, fb, B, fin, rm))
                tag = f"{name} B{B} {dt} fin={fin} {rm}"
                assert s.shape == (x.numel() // B, 1) and e.shape == (x.numel() // B, B)
                assert_bits_equal(s, s_o, "scales " + tag)
                assert_bits_equal(e, e_o, "elements " + tag)
                if rm == "rn":
                    y_o = oracle.compose_mxfp_tensor(s_o, e_o, mx_meta(eb, fb, B, fin), dt)
                    assert_bits_equal(mx_kernels.compose_mxfp_tensor(s, e, meta, dt), y_o, "composed " + tag)
                    assert_bits_equal(mx_kernels.quantize_dequantize(xg, meta, dt), y_o, "fused " + tag)


@pytest.mark.parametrize("name", list(PRESETS))
@pytest.mark.parametrize("fin", [True, False])
def test_mxfp_compose_every_scale_code_pair(lib, name, fin):
    eb, fb = PRESETS[name]
    sc = torch.arange(256, dtype=torch.int32).to(torch.uint8).repeat_interleave(8).reshape(-1, 1)
    el = torch.arange(256, dtype=torch.int32).to(torch.uint8).repeat(256).reshape(-1, 32)
    for dt in DTYPES:
        got = mx_kernels.compose_mxfp_tensor(sc.to(DEV), el.to(DEV), mxm(eb, fb, 32, fin), dt)
        assert_bits_equal(got, oracle.compose_mxfp_tensor(sc, el, mx_meta(eb, fb, 32, fin), dt), f"{name} {fin} {dt}")


def test_mxfp_unaligned_views_and_cross_dtype_qdq(lib):
    x = adversarial_mx_blocks(130, 32).flatten()
    xg = torch.cat([torch.zeros(1), x]).to(DEV)[1:]          # 4-byte aligned only
    s, e = mx_kernels.extract_mxfp_components(xg, MXFP8_E4M3_fn)
    s_o, e_o = oracle.extract_mxfp_components(x, mx_meta(4, 3))
    assert_bits_equal(s, s_o, "scales") ; assert_bits_equal(e, e_o, "elements")
    for out_dt in DTYPES:
        got = mx_kernels.quantize_dequantize(x.to(torch.bfloat16).to(DEV), OCP_MXFP6_E3M2, out_dt)
        s2, e2 = oracle.extract_mxfp_components(x.to(torch.bfloat16), mx_meta(3, 2))
        assert_bits_equal(got, oracle.compose_mxfp_tensor(s2, e2, mx_meta(3, 2), out_dt), f"bf16->{out_dt}")
    s0, e0 = mx_kernels.extract_mxfp_components(torch.empty(0, device=DEV), MXFP8_E4M3_fn)
    assert s0.shape == (0, 1) and e0.shape == (0, 32)
    with pytest.raises(AssertionError):
        mx_kernels.extract_mxfp_components(torch.zeros(33, device=DEV), MXFP8_E4M3_fn)
    with pytest.raises(AssertionError):
        mx_kernels.compose_mxfp_tensor(s.to(torch.int32), e, MXFP8_E4M3_fn, torch.float32)


# reference known answers: test/test_mxfp_fake.py:133-216
@pytest.mark.parametrize("meta", MX_PRESETS, ids=lambda m: m.tag)
def test_subnormal_inputs_dequantise_to_zero(lib, meta):
    w = torch.randint(0, 0b0111_1111, (meta.block_size * 16,), dtype=torch.int16).to(torch.int32).view(torch.float32).to(DEV)
    s, e, tm = MX.extract_mxfp_components(w, 0, meta)
    y = MX.compose_mxfp_tensor(s, e, tm, output_dtype=torch.float32)
    assert y.dtype == torch.float32 and bool((y == 0).all()) and bool((s == 0).all())


@pytest.mark.parametrize("dtype", DTYPES)
def test_mxfp4_block8_exact_round_trips(lib, dtype):
    meta = MXFPMeta(block_size=8, scale_exp_bits=8, element_exp_bits=2, element_frac_bits=1, element_is_finite=True, round_mode="rn")
    rows = [[6.0] * 4 + [-6.0] * 4, [1.0] * 4 + [-1.0] * 4, [0.5] * 4 + [-0.5] * 4, [0.0] * 8]
    x = (torch.tensor(rows, dtype=dtype).flatten() * 2.0**-120).to(DEV)
    s, e = mx_kernels.extract_mxfp_components(x, meta)
    assert bool((mx_kernels.compose_mxfp_tensor(s, e, meta, dtype) == x).all())
    x2 = (torch.tensor([[1.0, 0.0, 0.5, 0.5, -0.5, -0.5, -0.5, -0.5], [0.0] * 8]).flatten() * 2.0**-120).to(DEV)
    s, e = mx_kernels.extract_mxfp_components(x2, meta)
    assert bool((mx_kernels.compose_mxfp_tensor(s, e, meta, torch.float32) == x2).all())


@pytest.mark.parametrize("meta", MX_PRESETS, ids=lambda m: m.tag)
@pytest.mark.parametrize("block_dim", [0, 1, -1])
@pytest.mark.parametrize("dtype", DTYPES)
def test_public_api_2d_block_dims(lib, meta, block_dim, dtype):
    g = torch.Generator().manual_seed(11)
    w = (torch.randn(meta.block_size * 16 * 3, generator=g) * 50).to(dtype)
    w = w.reshape(-1, 3) if block_dim % 2 == 0 else w.reshape(3, -1)
    s, e, tm = MX.extract_mxfp_components(w.to(DEV), block_dim, meta)
    assert (tm.device, tm.dtype, tm.shape, tm.block_dim) == (DEV, str(dtype)[6:], tuple(w.shape), block_dim)
    y = MX.compose_mxfp_tensor(s, e, tm, output_dtype=torch.float32)
    assert y.shape == w.shape
    flat = w.movedim(block_dim % 2, -1).flatten()
    s_o, e_o = oracle.extract_mxfp_components(flat, meta)
    assert_bits_equal(s, s_o, "scales") ; assert_bits_equal(e, e_o, "elements")
    y_o = oracle.compose_mxfp_tensor(s_o, e_o, meta, torch.float32).reshape(w.movedim(block_dim % 2, -1).shape).movedim(-1, block_dim % 2)
    assert_bits_equal(y.contiguous(), y_o.contiguous(), "composed")
    assert_bits_equal(MX.quantize_dequantize(w.to(DEV), block_dim, meta, torch.float32).contiguous(), y_o.contiguous(), "fused")
    err = ((w.float() - y.cpu()).abs().mean() / w.float().abs().mean()).item()
    assert err < (0.3 if meta is OCP_MXFP4_E2M1 else 0.1)


# ------------------------------------------------------------------ blocks along a strided dimension
def _strided_case(shape, dim, dtype, seed):
    """Adversarial values (specials, zeros, subnormals, wide binades) laid out so that they form blocks
    along ``dim``; the values come from the same generator as the flat tests."""
    n = int(np.prod(shape))
    moved = list(shape[:dim]) + list(shape[dim + 1:]) + [shape[dim]]
    flat = adversarial_mx_blocks(n // 32, 32, seed=seed).to(dtype)
    return flat.reshape(moved).movedim(-1, dim).contiguous()


@pytest.mark.parametrize("meta", MX_PRESETS, ids=lambda m: m.tag)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape,dim", [((128, 64), 0), ((32, 200), 0), ((160, 33), 0), ((3, 96, 130), 1), ((2, 64, 5, 7), 1),
                                        ((256, 1024), 0)], ids=str)
def test_strided_blocks_match_oracle(lib, meta, dtype, shape, dim):
    """block_dim that is not the contiguous one: the strided kernels give the bytes of the reference's
    permute-then-flatten route (mxfp/helpers.py:4-47; the reference tests it at
    test/test_mxfp_functional.py:127-180)."""
    x = _strided_case(shape, dim, dtype, seed=5 + len(shape))
    flat = x.movedim(dim, -1).flatten()
    s_o, e_o = oracle.extract_mxfp_components(flat, meta)
    pair = mx_kernels.extract_mxfp_components_strided(x.to(DEV), dim, meta)
    assert pair is not None, "the strided kernel must cover this case"
    assert_bits_equal(pair[0], s_o, "scales"); assert_bits_equal(pair[1], e_o, "elements")
    s, e, tm = MX.extract_mxfp_components(x.to(DEV), dim - len(shape), meta)
    assert_bits_equal(s, s_o, "scales (public)"); assert_bits_equal(e, e_o, "elements (public)")
    moved_shape = x.movedim(dim, -1).shape
    for out_dtype in DTYPES:
        y_o = oracle.compose_mxfp_tensor(s_o, e_o, meta, out_dtype).reshape(moved_shape).movedim(-1, dim).contiguous()
        y = mx_kernels.compose_mxfp_tensor_strided(s, e, shape, dim, meta, out_dtype)
        assert y is not None and y.is_contiguous() and tuple(y.shape) == tuple(shape)
        assert_bits_equal(y, y_o, f"composed {out_dtype}")
        assert_bits_equal(MX.compose_mxfp_tensor(s, e, tm, out_dtype).contiguous(), y_o, f"composed {out_dtype} (public)")
    y_o = oracle.compose_mxfp_tensor(s_o, e_o, meta, dtype).reshape(moved_shape).movedim(-1, dim).contiguous()
    q = mx_kernels.quantize_dequantize_strided(x.to(DEV), dim, meta, dtype)
    assert q is not None
    assert_bits_equal(q, y_o, "fused")
    assert_bits_equal(MX.quantize_dequantize(x.to(DEV), dim, meta).contiguous(), y_o, "fused (public)")


def test_strided_blocks_random_shapes(lib):
    """Random (outer, D, inner) splits, all dtypes and presets: the strided kernels against the
    permute-then-flatten order of the oracle."""
    rng = np.random.default_rng(23)
    for trial in range(30):
        outer, D, inner = int(rng.integers(1, 5)), 32 * int(rng.integers(1, 9)), int(rng.integers(2, 150))
        meta = MX_PRESETS[trial % 5]
        dtype = DTYPES[trial % 3]
        shape = (outer, D, inner)
        x = _strided_case(shape, 1, dtype, seed=100 + trial)
        flat = x.movedim(1, -1).flatten()
        s_o, e_o = oracle.extract_mxfp_components(flat, meta)
        pair = mx_kernels.extract_mxfp_components_strided(x.to(DEV), 1, meta)
        assert pair is not None
        assert_bits_equal(pair[0], s_o, f"scales {shape}"); assert_bits_equal(pair[1], e_o, f"elements {shape}")
        y_o = oracle.compose_mxfp_tensor(s_o, e_o, meta, dtype).reshape(outer, inner, D).movedim(-1, 1).contiguous()
        assert_bits_equal(mx_kernels.compose_mxfp_tensor_strided(pair[0], pair[1], shape, 1, meta, dtype), y_o, f"composed {shape}")
        assert_bits_equal(mx_kernels.quantize_dequantize_strided(x.to(DEV), 1, meta, dtype), y_o, f"fused {shape}")


def test_strided_blocks_fall_back_when_not_covered(lib):
    """Blocks that span columns (D % 32 != 0), other block sizes and rounding modes take the
    permute + flat route and still match the oracle."""
    for shape, dim, meta in [((48, 4), 0, mxm(4, 3)), ((64, 6), 0, mxm(4, 3, B=8)), ((64, 6), 0, mxm(2, 1, rm="rz")),
                             ((64, 6), 0, mxm(5, 2, fin=False))]:
        x = torch.randn(shape, generator=torch.Generator().manual_seed(1)) * 7
        flat = x.movedim(dim, -1).flatten()
        s_o, e_o = oracle.extract_mxfp_components(flat, meta)
        s, e, tm = MX.extract_mxfp_components(x.to(DEV), dim, meta)
        assert_bits_equal(s, s_o, "scales"); assert_bits_equal(e, e_o, "elements")
        y_o = oracle.compose_mxfp_tensor(s_o, e_o, meta, torch.float32).reshape(x.movedim(dim, -1).shape).movedim(-1, dim)
        assert_bits_equal(MX.compose_mxfp_tensor(s, e, tm).contiguous(), y_o.contiguous(), "composed")
        assert_bits_equal(MX.quantize_dequantize(x.to(DEV), dim, meta).contiguous(), y_o.contiguous(), "fused")


# ------------------------------------------------------------------ full-size configurations, pinned to the reference by digest
def test_config1_full_size(lib, digests):
    x = synthetic.cfg1_mxfp8_fp32()
    assert sha(x) == digests["cfg1"]["input"]
    xg = x.to(DEV)
    s, e, tm = MX.extract_mxfp_components(xg, -1, MXFP8_E4M3_fn)
    y = MX.compose_mxfp_tensor(s, e, tm)
    assert sha(s) == digests["cfg1"]["scales"] and sha(e) == digests["cfg1"]["elements"] and sha(y) == digests["cfg1"]["composed"]
    assert sha(MX.quantize_dequantize(xg, -1, MXFP8_E4M3_fn)) == digests["cfg1"]["composed"]
    # row sharding does not change results: quantising a row slice gives the matching slice
    s4, e4, _ = MX.extract_mxfp_components(xg[1024:2048], -1, MXFP8_E4M3_fn)
    assert torch.equal(s4, s[1024 * 128:2048 * 128]) and torch.equal(e4, e[1024 * 128:2048 * 128])


def test_config2_full_size(lib, digests):
    x = synthetic.cfg2_minifloat_fp32()
    assert sha(x) == digests["cfg2"]["input"]
    xg = x.to(DEV)
    for fin in (True, False):
        meta = MinifloatMeta(5, 2, fin, "rn")
        assert sha(MF.quantize_dequantize(xg, meta)) == digests["cfg2"][f"qdq_fin{int(fin)}"]
        codes, tm = MF.extract_minifloat_component(xg, meta)
        assert sha(codes) == digests["cfg2"][f"codes_fin{int(fin)}"]
        assert sha(MF.compose_minifloat_component(codes, tm)) == digests["cfg2"][f"qdq_fin{int(fin)}"]


def test_config3_full_size(lib, digests):
    x = synthetic.cfg3_mxfp4_bf16()
    assert sha(x) == digests["cfg3"]["input"]
    xg = x.to(DEV)
    s, e, tm = MX.extract_mxfp_components(xg, -1, OCP_MXFP4_E2M1)
    assert sha(s) == digests["cfg3"]["scales"] and sha(e) == digests["cfg3"]["elements"]
    assert sha(MX.compose_mxfp_tensor(s, e, tm)) == digests["cfg3"]["composed"]
    assert sha(MX.quantize_dequantize(xg, -1, OCP_MXFP4_E2M1)) == digests["cfg3"]["composed"]
