"""Bit-packed storage of element codes, the serialisable layer record, and the tensor-core weight form that a
layer keeps as buffers."""

from __future__ import annotations

import io

import numpy as np
import pytest
import torch

from mase_triton_b200.mxfp import gemm as G
from mase_triton_b200.mxfp import storage
from mase_triton_b200.mxfp.layers import MXFPLinearPTQ
from mase_triton_b200.mxfp.meta import MXFP8_E4M3_fn, MXFP8_E5M2_fn, OCP_MXFP4_E2M1, OCP_MXFP6_E2M3, OCP_MXFP6_E3M2

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def reference_pack(codes: np.ndarray, bits: int) -> np.ndarray:
    """Little-endian bit stream: code i in bits [i * bits, (i + 1) * bits)."""
    n = codes.size
    stream = np.zeros(n * bits, dtype=np.uint8)
    for b in range(bits):
        stream[b::bits] = (codes >> b) & 1
    return np.packbits(stream, bitorder="little")


@pytest.mark.parametrize("bits", [4, 6, 8])
@pytest.mark.parametrize("n", [16, 4096, 16 * 1000 + 16, 1 << 20])
def test_pack_unpack_codes(lib, bits, n):
    g = torch.Generator().manual_seed(n + bits)
    codes = torch.randint(0, 1 << bits, (n,), generator=g, dtype=torch.int32).to(torch.uint8)
    packed = storage.pack_codes(codes.to(DEV), bits)
    assert packed.numel() == n * bits // 8
    assert np.array_equal(packed.cpu().numpy(), reference_pack(codes.numpy(), bits))
    assert torch.equal(storage.unpack_codes(packed, n, bits).cpu(), codes)


@pytest.mark.parametrize("w_meta", [MXFP8_E4M3_fn, MXFP8_E5M2_fn, OCP_MXFP6_E2M3, OCP_MXFP6_E3M2, OCP_MXFP4_E2M1], ids=lambda m: m.tag)
def test_export_import_round_trip(lib, w_meta):
    torch.manual_seed(2)
    fc = torch.nn.Linear(256, 96, bias=True, device=DEV, dtype=torch.bfloat16)
    layer = MXFPLinearPTQ.from_linear(fc, MXFP8_E4M3_fn, w_meta, MXFP8_E4M3_fn, "XqWqBq", "fused")
    rec = layer.export_packed()
    bits = 1 + w_meta.element_exp_bits + w_meta.element_frac_bits
    assert rec["weight"]["packed"].numel() == 96 * 256 * bits // 8 and rec["weight"]["packed"].device.type == "cpu"
    buf = io.BytesIO()
    torch.save(rec, buf)                                   # plain tensors and Python scalars only
    buf.seek(0)
    back = MXFPLinearPTQ.from_packed(torch.load(buf, weights_only=True), DEV)
    assert torch.equal(back.w_elements, layer.w_elements) and torch.equal(back.w_scales, layer.w_scales)
    assert torch.equal(back.b_elements, layer.b_elements) and torch.equal(back.b_scales, layer.b_scales)
    assert back.w_tensor_meta == layer.w_tensor_meta.create(device=back.w_elements.device) and back.layer_type == "XqWqBq"
    x = torch.randn(40, 256, device=DEV).bfloat16()
    assert torch.equal(back(x), layer(x))
    G.check_status(DEV)
    plain = MXFPLinearPTQ.from_linear(fc, None, w_meta, None, "XWqB", "separate")
    again = MXFPLinearPTQ.from_packed(plain.export_packed(), DEV)
    assert torch.equal(again(x), plain(x))


def test_tensor_core_weight_follows_the_module(lib):
    torch.manual_seed(4)
    fc = torch.nn.Linear(512, 320, bias=False, device=DEV, dtype=torch.bfloat16)
    layer = MXFPLinearPTQ.from_linear(fc, MXFP8_E4M3_fn, OCP_MXFP6_E3M2, None, "XqWqB", "fused")
    x = torch.randn(64, 512, device=DEV).bfloat16()
    y = layer(x)
    assert layer._tc_codes is not None and set(layer.state_dict()) == {"w_scales", "w_elements"}      # buffers are not persistent
    first = layer._tc_codes
    assert torch.equal(layer(x), y) and layer._tc_codes is first                  # no re-pack per call
    layer.to("cpu")
    assert layer._tc_codes.device.type == "cpu"
    layer.to(DEV)
    moved = layer._tc_codes
    assert torch.equal(layer(x), y) and torch.equal(moved, first)
    # new codes through load_state_dict: the tensor-core form is rebuilt from them
    other = MXFPLinearPTQ.from_linear(torch.nn.Linear(512, 320, bias=False, device=DEV, dtype=torch.bfloat16), MXFP8_E4M3_fn, OCP_MXFP6_E3M2,
                                      None, "XqWqB", "fused")
    layer.load_state_dict(other.state_dict())
    assert torch.equal(layer(x), other(x)) and not torch.equal(layer(x), y)
    G.check_status(DEV)
