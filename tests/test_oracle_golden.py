"""The CPU oracle against vectors generated from the reference's fake path
(tests/golden/make_golden.py). Needs no GPU and does not read the reference."""

from __future__ import annotations

import hashlib
import json
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle
from helpers import PRESETS, assert_bits_equal, mf_meta, mx_meta
from mase_triton_b200 import synthetic

GOLD = Path(__file__).resolve().parent / "golden"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


@pytest.fixture(scope="module")
def small():
    return np.load(GOLD / "golden_small.npz")


@pytest.fixture(scope="module")
def digests():
    return json.loads((GOLD / "golden_digests.json").read_text())


def gold_tensor(arr: np.ndarray, dtype_name: str | None = None) -> torch.Tensor:
    t = torch.from_numpy(arr.copy())
    if dtype_name == "bfloat16":
        t = t.view(torch.bfloat16)
    return t


def sha(t: torch.Tensor) -> str:
    t = t.contiguous()
    return hashlib.sha256((t if t.dtype == torch.uint8 else t.view(torch.uint8)).numpy().tobytes()).hexdigest()


def test_minifloat_extract_golden(small):
    x = gold_tensor(small["mf_x"])
    keys = [k for k in small.files if k.startswith("mf_extract/")]
    assert len(keys) >= 40
    for k in keys:
        _, name, fin, rm = k.split("/")
        eb, fb = PRESETS[name] if name in PRESETS else tuple(int(v) for v in name[1:].split("m"))
        got = oracle.extract_minifloat_component(x, mf_meta(eb, fb, bool(int(fin)), rm))
        assert_bits_equal(got, gold_tensor(small[k]), k)


def test_minifloat_compose_golden(small):
    codes = gold_tensor(small["mf_codes"])
    for k in [k for k in small.files if k.startswith("mf_compose/")]:
        _, name, fin, dn = k.split("/")
        eb, fb = PRESETS[name]
        got = oracle.compose_minifloat_component(codes, mf_meta(eb, fb, bool(int(fin))), DT[dn])
        assert_bits_equal(got, gold_tensor(small[k], dn), k, nan_any_payload_16bit=False)


def test_mxfp_extract_compose_golden(small):
    n = 0
    for k in [k for k in small.files if k.startswith("mx_scales/")]:
        _, B, dn, name, fin, rm = k.split("/")
        eb, fb = PRESETS[name]
        meta = mx_meta(eb, fb, int(B), bool(int(fin)), rm)
        x = gold_tensor(small[f"mx_x/{B}/{dn}"], dn)
        s, e = oracle.extract_mxfp_components(x, meta)
        tail = k[len("mx_scales/"):]
        assert_bits_equal(s, gold_tensor(small[k]), k)
        assert_bits_equal(e, gold_tensor(small["mx_elements/" + tail]), "elements " + tail)
        if rm == "rn":
            y = oracle.compose_mxfp_tensor(s, e, meta, DT[dn])
            assert_bits_equal(y, gold_tensor(small["mx_composed/" + tail], dn), "composed " + tail, nan_any_payload_16bit=False)
        n += 1
    assert n >= 90


def test_mxfp_compose_scale_sweep_golden(small):
    sc, el = gold_tensor(small["mxc_scales"]), gold_tensor(small["mxc_elements"])
    for k in [k for k in small.files if k.startswith("mxc_out/")]:
        _, name, fin, dn = k.split("/")
        eb, fb = PRESETS[name]
        y = oracle.compose_mxfp_tensor(sc, el, mx_meta(eb, fb, 32, bool(int(fin))), DT[dn])
        assert_bits_equal(y, gold_tensor(small[k], dn), k, nan_any_payload_16bit=False)


def test_full_size_config1_digest(digests):
    x = synthetic.cfg1_mxfp8_fp32()
    assert sha(x) == digests["cfg1"]["input"], "the seeded generator no longer reproduces the golden input"
    meta = mx_meta(4, 3)
    s, e = oracle.extract_mxfp_components(x.flatten(), meta)
    assert sha(s) == digests["cfg1"]["scales"]
    assert sha(e) == digests["cfg1"]["elements"]
    assert sha(oracle.compose_mxfp_tensor(s, e, meta, torch.float32)) == digests["cfg1"]["composed"]


def test_full_size_config2_digest(digests):
    x = synthetic.cfg2_minifloat_fp32()
    assert sha(x) == digests["cfg2"]["input"]
    for fin in (True, False):
        meta = mf_meta(5, 2, fin)
        assert sha(oracle.extract_minifloat_component(x, meta)) == digests["cfg2"][f"codes_fin{int(fin)}"]
        assert sha(oracle.quantize_dequantize_minifloat(x, meta)) == digests["cfg2"][f"qdq_fin{int(fin)}"]


def test_full_size_config3_digest(digests):
    x = synthetic.cfg3_mxfp4_bf16()
    assert sha(x) == digests["cfg3"]["input"]
    meta = mx_meta(2, 1)
    s, e = oracle.extract_mxfp_components(x.flatten(), meta)
    assert sha(s) == digests["cfg3"]["scales"]
    assert sha(e) == digests["cfg3"]["elements"]
    assert sha(oracle.compose_mxfp_tensor(s, e, meta, torch.bfloat16)) == digests["cfg3"]["composed"]
