"""The element arithmetic the CUDA kernels use (mase_triton_b200/csrc/mxq_codec.h), compiled for
the host and compared bit-for-bit with the oracle. Needs no GPU."""

from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import pytest
import torch

import oracle
from helpers import (PRESETS, ROUND_MODES, adversarial_fp32, adversarial_mx_blocks, assert_bits_equal, from_bits32,
                     mf_meta, mx_meta)

HERE = Path(__file__).resolve().parent
RM = {"rn": 0, "ru": 1, "rd": 2, "rz": 3}


@pytest.fixture(scope="module")
def hc():
    build = HERE / "_build"
    build.mkdir(exist_ok=True)
    so = build / "libcodec_host.so"
    subprocess.run(["/usr/bin/g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fno-fast-math", "-ffp-contract=off",
                    "-o", str(so), str(HERE / "host_codec" / "codec_host.cpp")], check=True)
    L = ctypes.CDLL(str(so))
    p, i64, i = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int
    L.hc_minifloat_encode.argtypes = [p, p, i64, i, i, i, i, i]
    L.hc_minifloat_decode.argtypes = [p, p, i64, i, i, i, i]
    L.hc_minifloat_qdq.argtypes = [p, p, i64, i, i, i, i, i]
    L.hc_mxfp_extract.argtypes = [p, p, p, i64, i, i, i, i, i, i]
    L.hc_mxfp_compose.argtypes = [p, p, p, i64, i, i, i, i, i]
    L.hc_mxfp_qdq.argtypes = [p, p, i64, i, i, i, i, i]
    L.hc_log2_roundup_count.argtypes = [i]
    return L


def _encode(hc, x, eb, fb, fin, rm, fast):
    x = x.contiguous()
    out = torch.empty(x.shape, dtype=torch.uint16)
    used = hc.hc_minifloat_encode(x.data_ptr(), out.data_ptr(), x.numel(), eb, fb, int(fin), RM[rm], int(fast))
    return out, used


@pytest.mark.parametrize("eb,fb", list(PRESETS.values()) + [(8, 7), (5, 10), (3, 4), (1, 1), (7, 8), (10, 5), (6, 1)])
@pytest.mark.parametrize("fin", [True, False])
def test_minifloat_encode_generic(hc, eb, fb, fin):
    x = adversarial_fp32(1 << 16)
    for rm in ROUND_MODES:
        got, _ = _encode(hc, x, eb, fb, fin, rm, fast=False)
        assert_bits_equal(got, oracle.extract_minifloat_component(x, mf_meta(eb, fb, fin, rm)), f"e{eb}m{fb} {fin} {rm}")


@pytest.mark.parametrize("name", list(PRESETS))
def test_minifloat_encode_fast(hc, name):
    eb, fb = PRESETS[name]
    x = adversarial_fp32(1 << 18, seed=7)
    got, used = _encode(hc, x, eb, fb, True, "rn", fast=True)
    assert used == 1
    assert_bits_equal(got, oracle.extract_minifloat_component(x, mf_meta(eb, fb)), name)
    # every bf16 and fp16 bit pattern
    for dt in (torch.bfloat16, torch.float16):
        allv = torch.arange(-(2**15), 2**15, dtype=torch.int32).to(torch.int16).view(dt).float()
        got, _ = _encode(hc, allv, eb, fb, True, "rn", fast=True)
        assert_bits_equal(got, oracle.extract_minifloat_component(allv, mf_meta(eb, fb)), f"{name} all {dt}")


@pytest.mark.parametrize("name", list(PRESETS))
def test_minifloat_qdq_fast(hc, name):
    eb, fb = PRESETS[name]
    xs = [adversarial_fp32(1 << 18, seed=11)]
    xs += [torch.arange(-(2**15), 2**15, dtype=torch.int32).to(torch.int16).view(dt).float() for dt in (torch.bfloat16, torch.float16)]
    for x in xs:
        x = x.contiguous()
        out = torch.empty(x.numel(), dtype=torch.int32)
        assert hc.hc_minifloat_qdq(x.data_ptr(), out.data_ptr(), x.numel(), eb, fb, 1, 0, 1) == 1
        assert_bits_equal(out.view(torch.float32), oracle.quantize_dequantize_minifloat(x, mf_meta(eb, fb)), name)


@pytest.mark.parametrize("eb,fb", list(PRESETS.values()) + [(8, 7), (5, 10), (3, 4), (1, 1), (7, 8), (10, 5)])
@pytest.mark.parametrize("fin", [True, False])
@pytest.mark.parametrize("fast", [False, True])
def test_minifloat_decode_all_codes(hc, eb, fb, fin, fast):
    codes = torch.arange(0, 65536, dtype=torch.int32).to(torch.uint16)
    out = torch.empty(65536, dtype=torch.int32)
    hc.hc_minifloat_decode(codes.data_ptr(), out.data_ptr(), 65536, eb, fb, int(fin), int(fast))
    want = oracle.compose_minifloat_component(codes, mf_meta(eb, fb, fin), torch.float32)
    assert_bits_equal(out.view(torch.float32), want, f"decode e{eb}m{fb} fin={fin} fast={fast}")


@pytest.mark.parametrize("name", list(PRESETS))
@pytest.mark.parametrize("B", [32, 8, 5])
@pytest.mark.parametrize("fast", [False, True])
def test_mxfp_extract(hc, name, B, fast):
    eb, fb = PRESETS[name]
    base = adversarial_mx_blocks(2048, B)
    for dt in (torch.float32, torch.bfloat16, torch.float16):
        x = base.to(dt).float().flatten().contiguous()
        for fin in (True, False):
            for rm in (("rn",) if fast else ROUND_MODES):
                sc = torch.empty(x.numel() // B, dtype=torch.uint8)
                el = torch.empty(x.numel(), dtype=torch.uint8)
                hc.hc_mxfp_extract(x.data_ptr(), sc.data_ptr(), el.data_ptr(), x.numel(), B, eb, fb, int(fin), RM[rm], int(fast))
                s_o, e_o = oracle.extract_mxfp_components(x, mx_meta(eb, fb, B, fin, rm))
                assert_bits_equal(sc.reshape(-1, 1), s_o, f"scales {name} B{B} {dt} fin={fin} {rm}")
                assert_bits_equal(el.reshape(-1, B), e_o, f"elements {name} B{B} {dt} fin={fin} {rm}")


@pytest.mark.parametrize("name", list(PRESETS))
def test_mxfp_extract_random_normal_data(hc, name):
    eb, fb = PRESETS[name]
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(1 << 20, generator=g) * 100).contiguous()
    sc = torch.empty(x.numel() // 32, dtype=torch.uint8)
    el = torch.empty(x.numel(), dtype=torch.uint8)
    hc.hc_mxfp_extract(x.data_ptr(), sc.data_ptr(), el.data_ptr(), x.numel(), 32, eb, fb, 1, 0, 1)
    s_o, e_o = oracle.extract_mxfp_components(x, mx_meta(eb, fb))
    assert_bits_equal(sc.reshape(-1, 1), s_o, "scales")
    assert_bits_equal(el.reshape(-1, 32), e_o, "elements")


@pytest.mark.parametrize("name", list(PRESETS))
def test_mxfp_fused_qdq(hc, name):
    """The fused quantize-dequantize arithmetic (value built in the fp32 bit domain) against
    compose(extract(x)) of the oracle, fp32 results, for inputs of every kernel dtype."""
    eb, fb = PRESETS[name]
    meta = mx_meta(eb, fb)
    g = torch.Generator().manual_seed(8)
    cases = [adversarial_mx_blocks(4096, 32), adversarial_mx_blocks(4096, 32, seed=3),
             torch.randn(4096, 32, generator=g) * torch.exp(2.0 * torch.randn(4096, 1, generator=g))]
    for base in cases:
        for dt in (torch.float32, torch.bfloat16, torch.float16):
            x = base.to(dt).float().flatten().contiguous()
            out = torch.empty(x.numel(), dtype=torch.int32)
            assert hc.hc_mxfp_qdq(x.data_ptr(), out.data_ptr(), x.numel(), 32, eb, fb, 1, 0) == 1
            s_o, e_o = oracle.extract_mxfp_components(x, meta)
            assert_bits_equal(out.view(torch.float32), oracle.compose_mxfp_tensor(s_o, e_o, meta, torch.float32), f"{name} {dt}")


@pytest.mark.parametrize("name", list(PRESETS))
@pytest.mark.parametrize("fin", [True, False])
@pytest.mark.parametrize("fast", [False, True])
def test_mxfp_compose_all_pairs(hc, name, fin, fast):
    eb, fb = PRESETS[name]
    sc = torch.arange(256, dtype=torch.int32).to(torch.uint8).repeat_interleave(8).contiguous()
    el = torch.arange(256, dtype=torch.int32).to(torch.uint8).repeat(256).contiguous()
    out = torch.empty(el.numel(), dtype=torch.int32)
    hc.hc_mxfp_compose(sc.data_ptr(), el.data_ptr(), out.data_ptr(), el.numel(), 32, eb, fb, int(fin), int(fast))
    want = oracle.compose_mxfp_tensor(sc.reshape(-1, 1), el.reshape(-1, 32), mx_meta(eb, fb, 32, fin), torch.float32)
    assert_bits_equal(out.view(torch.float32), want, f"compose {name} fin={fin} fast={fast}")


def test_log2_roundup_table_matches_host_log2(hc):
    """floor(log2f) of the floats just below every power of two, as this host's torch evaluates
    it, against the closed form the kernels use."""
    top = 64
    for e in range(-126, 128):
        mant = torch.arange(0x7FFFFF - top + 1, 0x7FFFFF + 1, dtype=torch.int64)
        v = from_bits32(((e + 127) << 23) | mant)
        l = torch.cat([v, v]).log2().floor().to(torch.int32)[:top]
        cnt = int((l == e + 1).sum())
        assert cnt == hc.hc_log2_roundup_count(e) == oracle.log2_roundup_count(e), f"binade {e}"
        assert bool((l[top - cnt:] == e + 1).all()) and bool((l[: top - cnt] == e).all())
