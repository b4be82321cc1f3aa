"""The linear benchmark configurations at their full sizes: configuration 4 (x bf16 [8192, 4096], W [14336, 4096],
both MXFP8 E4M3) and the seven projections of configuration 5 (32768 tokens, W MXFP6 E3M2, x MXFP8 E4M3,
`down` with K = 14336).  The fused layer is compared

* with an fp32 matmul of the operands as the CPU oracle dequantises them, element-wise within
  |y - y32| <= 2^-7 |y32| + 2^-7 rms(y32) (about one bf16 ulp plus accumulation-order slack), in row chunks, and
* with the layer's own ``backend="separate"`` output (the reference's op sequence, an independently
  rounded bf16 result): mean |y - y_sep| / mean |y_sep| < 5e-3.
"""

from __future__ import annotations

import pytest
import torch

import oracle
from mase_triton_b200 import synthetic
from mase_triton_b200.mxfp import gemm as G
from mase_triton_b200.mxfp.layers import MXFPLinearPTQ
from mase_triton_b200.mxfp.meta import MXFP8_E4M3_fn, OCP_MXFP6_E3M2

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
CHUNK = 8192


def oracle_dequant(t: torch.Tensor, meta) -> torch.Tensor:
    """fp32 values of ``t`` after MXFP extract + compose along its last dim, by the CPU oracle."""
    s, e = oracle.extract_mxfp_components(t.reshape(-1), meta)
    return oracle.compose_mxfp_tensor(s, e, meta, torch.float32).reshape(t.shape)


def check_layer(x: torch.Tensor, w: torch.Tensor, x_meta, w_meta, layer_type: str = "XqWqB"):
    n_out, n_in = w.shape
    fc = torch.nn.Linear(n_in, n_out, bias=False, device=DEV, dtype=torch.bfloat16)
    with torch.no_grad():
        fc.weight.copy_(w)
    xm = x_meta if "Xq" in layer_type else None
    fused = MXFPLinearPTQ.from_linear(fc, xm, w_meta, None, layer_type, "fused")
    sep = MXFPLinearPTQ.from_linear(fc, xm, w_meta, None, layer_type, "separate")
    xg = x.to(DEV)
    y = fused(xg)
    G.check_status(DEV)
    assert y.shape == (*x.shape[:-1], n_out) and y.dtype == torch.bfloat16
    y_sep = sep(xg)
    rel = ((y.float() - y_sep.float()).abs().mean() / y_sep.float().abs().mean()).item()
    assert rel < 5e-3, rel
    del y_sep
    x_dq = (oracle_dequant(x, x_meta) if xm is not None else x.float()).reshape(-1, n_in)
    w_dq = oracle_dequant(w, w_meta).to(DEV)
    y2 = y.reshape(-1, n_out)
    worst = 0.0
    for r0 in range(0, x_dq.shape[0], CHUNK):
        y32 = x_dq[r0:r0 + CHUNK].to(DEV) @ w_dq.t()              # true fp32 (TF32 is off by default)
        tol = 2.0**-7 * y32.abs() + 2.0**-7 * y32.pow(2).mean().sqrt()
        excess = ((y2[r0:r0 + CHUNK].float() - y32).abs() - tol).max().item()
        worst = max(worst, excess)
        del y32, tol
    assert worst <= 0.0, f"largest excess over the tolerance: {worst}"


def test_config4_full_size(lib):
    x, w = synthetic.cfg4_linear_operands()
    check_layer(x, w, MXFP8_E4M3_fn, MXFP8_E4M3_fn)


def test_config4_full_size_weight_only(lib):
    """The same shape with only the weight quantised: the weight codes are expanded inside the GEMM's loader."""
    x, w = synthetic.cfg4_linear_operands()
    check_layer(x, w, MXFP8_E4M3_fn, MXFP8_E4M3_fn, "XWqB")


@pytest.mark.parametrize("proj", [p[0] for p in synthetic.CFG5_PROJECTIONS])
def test_config5_projection_full_size(lib, proj):
    _, n_out, n_in = next(p for p in synthetic.CFG5_PROJECTIONS if p[0] == proj)
    w = synthetic.cfg5_weight(proj)
    x = synthetic.cfg5_input(n_in)
    assert w.shape == (n_out, n_in) and x.shape == (16, 2048, n_in)
    check_layer(x, w, MXFP8_E4M3_fn, OCP_MXFP6_E3M2)


def test_config5_shared_activation(lib):
    """q / k / v on one packed activation give the bytes of three independent forward calls."""
    x = synthetic.cfg5_input(4096)[:2].to(DEV)
    layers = {}
    for proj in ("q", "k", "v"):
        w = synthetic.cfg5_weight(proj)
        fc = torch.nn.Linear(w.shape[1], w.shape[0], bias=False, device=DEV, dtype=torch.bfloat16)
        with torch.no_grad():
            fc.weight.copy_(w)
        layers[proj] = MXFPLinearPTQ.from_linear(fc, MXFP8_E4M3_fn, OCP_MXFP6_E3M2, None, "XqWqB", "fused")
    packed = layers["q"].pack_input(x)
    for proj, layer in layers.items():
        y = layer.forward_packed(packed, torch.bfloat16, lead_shape=tuple(x.shape[:-1]))
        assert torch.equal(y, layer(x)), proj
    G.check_status(DEV)
