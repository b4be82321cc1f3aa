"""Host-side logic that needs no GPU: metas, layout helpers, layer-type parsing, error behaviour,
and that the C-ABI library loads and exports every symbol its header declares."""

from __future__ import annotations

import ctypes
import re
from pathlib import Path

import pytest
import torch

import mase_triton_b200 as mt
from mase_triton_b200 import _lib
from mase_triton_b200._linear_common import parse_layer_type
from mase_triton_b200.minifloat.meta import (FP4_E2M1_fn, FP6_E2M3_fn, FP6_E3M2_fn, FP8_E4M3_fn, FP8_E5M2_fn, MinifloatMeta,
                                            MinifloatTensorMeta)
from mase_triton_b200.mxfp.functional import (extract_mxfp_components, extract_mxfp_tensor, flatten_for_quantize,
                                             parse_mxfp_linear_type, permute_for_dequantize)
from mase_triton_b200.mxfp.meta import MXFP8_E4M3_fn, OCP_MXFP4_E2M1, MXFPMeta, MXFPTensorMeta
from mase_triton_b200.utils.qlayer import ChangeDtypeError, devices_equal

ROOT = Path(__file__).resolve().parents[1]


def test_header_symbols_exported():
    header = (ROOT / "include" / "mxq.h").read_text()
    declared = set(re.findall(r"\b(mxq_\w+)\s*\(", header))
    assert {"mxq_minifloat_extract", "mxq_minifloat_compose", "mxq_minifloat_qdq", "mxq_mxfp_extract",
            "mxq_mxfp_compose", "mxq_mxfp_qdq", "mxq_version"} <= declared
    L = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in declared:
        assert hasattr(L, name), f"{name} is declared in include/mxq.h but not exported by libmxq.so"
    assert _lib.load().mxq_version() >= 1000
    assert _lib.load().mxq_status_string(-1) == b"invalid argument"


def test_every_bound_symbol_is_declared():
    header = (ROOT / "include" / "mxq.h").read_text()
    for name in list(_lib.SIGNATURES) + list(_lib._STRING_FUNCS) + list(_lib._I64_FUNCS):
        assert re.search(rf"\b{name}\s*\(", header), f"{name} is bound in _lib.py but not declared in include/mxq.h"


# known answers from the reference's tests (test/test_minifloat_fake.py:43-55)
@pytest.mark.parametrize("meta,finfo", [
    (FP4_E2M1_fn, (6.0, 1.0, 0.5, 0.5)),
    (FP6_E2M3_fn, (7.5, 1.0, 0.875, 0.125)),
    (FP6_E3M2_fn, (28.0, 0.25, 0.1875, 0.0625)),
    (FP8_E4M3_fn, (480.0, 2**-6, 2**-6 * 0.875, 2**-9)),
])
def test_builtin_meta(meta, finfo):
    assert (meta.max_normal, meta.min_normal, meta.max_subnormal, meta.min_subnormal) == finfo


def test_meta_validation():
    assert FP8_E5M2_fn.n_bits == 8 and FP8_E5M2_fn.max_normal == 114688.0
    assert MinifloatMeta(5, 2, False, "rn").max_normal == 57344.0
    with pytest.raises(AssertionError):
        MinifloatMeta(exp_bits=0, frac_bits=3, is_finite=True, round_mode="rn")
    with pytest.raises(AssertionError):
        MinifloatMeta(exp_bits=8, frac_bits=8, is_finite=True, round_mode="rn")
    with pytest.raises(AssertionError):
        MXFPMeta(32, 7, 4, 3, True, "rn")
    with pytest.raises(AssertionError):
        MXFPMeta(32, 8, 4, 4, True, "rn")
    assert MXFP8_E4M3_fn.element_meta == MinifloatMeta(4, 3, True, "rn")
    assert hash(MXFP8_E4M3_fn) != hash(OCP_MXFP4_E2M1)
    with pytest.raises(Exception):
        MXFP8_E4M3_fn.block_size = 16          # frozen


def test_tensor_meta_records_strings():
    tm = MXFPTensorMeta(device=torch.device("cpu"), dtype=torch.bfloat16, shape=torch.Size([2, 64]), block_dim=1, meta=MXFP8_E4M3_fn)
    assert (tm.device, tm.dtype, tm.shape) == ("cpu", "bfloat16", (2, 64))
    moved = tm.create(device="cuda:0")
    assert moved.device == "cuda:0" and moved.dtype == "bfloat16" and moved.block_dim == 1 and moved.meta is MXFP8_E4M3_fn
    mm = MinifloatTensorMeta(device="cpu", dtype=torch.float16, shape=(3,), meta=FP8_E4M3_fn)
    assert mm.dtype == "float16" and mm.create(dtype=torch.float32).dtype == "float32"


# reference: test/test_mxfp_functional.py:27-39
@pytest.mark.parametrize("block_dim", [0, 1, 2, -1, -2, -3])
def test_flatten_permute_inverse(block_dim):
    x = torch.arange(24).reshape(2, 3, 4)
    flat = flatten_for_quantize(x, block_dim)
    assert flat.ndim == 1
    # the blocked dim must be the fastest-varying one after flattening
    assert torch.equal(flat[: x.shape[block_dim]], x.movedim(block_dim, -1).reshape(-1, x.shape[block_dim])[0])
    back = permute_for_dequantize(flat, ori_shape=tuple(x.shape), block_dim=block_dim)
    assert back.shape == x.shape and torch.equal(back, x)


def test_layer_type_parsing():
    for lt in ("XWB", "XWBq", "XWqB", "XWqBq", "XqWB", "XqWBq", "XqWqB", "XqWqBq"):
        k = parse_layer_type(lt)
        assert (k.x_quantised, k.w_quantised, k.b_quantised) == ("Xq" in lt, "Wq" in lt, "Bq" in lt)
    with pytest.raises(NotImplementedError):
        parse_layer_type("YZ")
    assert parse_mxfp_linear_type(MXFP8_E4M3_fn, None, None) == "XqWB"
    assert parse_mxfp_linear_type(None, object(), object()) == "XWqBq"
    assert extract_mxfp_tensor is extract_mxfp_components


def test_no_cpu_fallback():
    x = torch.randn(64)
    with pytest.raises(_lib.MXQError):
        mt.mxfp.functional.extract_mxfp_components(x, -1, MXFP8_E4M3_fn)
    with pytest.raises(_lib.MXQError):
        mt.minifloat.functional.quantize_dequantize(x, FP8_E4M3_fn)
    with pytest.raises(AssertionError):
        mt.mxfp.functional.extract_mxfp_components(x, 1, MXFP8_E4M3_fn)      # block_dim out of range


def test_c_abi_rejects_bad_arguments_without_a_gpu():
    L = _lib.load()
    assert L.mxq_mxfp_extract(None, 0, None, None, 33, 32, 4, 3, 1, 0, None) == -1      # n % block_size
    assert L.mxq_mxfp_extract(None, 7, None, None, 32, 32, 4, 3, 1, 0, None) == -1      # dtype id
    assert L.mxq_minifloat_qdq(None, 0, None, 0, 16, 9, 9, 1, 0, None) == -1            # exp+frac >= 16
    assert L.mxq_minifloat_extract(None, 0, None, 16, 4, 3, 1, 0, None) == -1           # null pointers
    assert L.mxq_minifloat_extract(None, 0, None, 0, 4, 3, 1, 0, None) == 0             # empty is a no-op


def test_qlayer_helpers():
    assert devices_equal("cuda", "cuda:0") and not devices_equal("cpu", "cuda:0")
    assert isinstance(ChangeDtypeError(), Exception)
    mt.manager.KernelManager.enable_autotune()
    assert mt.manager.KernelManager.autotune_is_enabled()
    mt.manager.KernelManager.disable_autotune()
    assert not mt.manager.KernelManager.autotune_is_enabled()
