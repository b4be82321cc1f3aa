"""The dequantise-in-the-loader tensor-core GEMM (layer types whose operands are not both block-quantised).

Two kinds of check: (1) with an identity activation the GEMM output IS the dequantised weight, so the
loader's expansion is compared bit for bit with the oracle's compose; (2) random operands against an
fp32 matmul of the oracle-dequantised operands, with the tolerance used for every linear here:
|y - y32| <= 2^-7 |y32| + 2^-7 rms(y32).
"""

from __future__ import annotations

import pytest
import torch

import oracle
from helpers import mf_meta
from mase_triton_b200 import tc_linear
from mase_triton_b200.minifloat import functional as MF
from mase_triton_b200.minifloat.layers import MinifloatLinearPTQ
from mase_triton_b200.minifloat.meta import FP8_E4M3_fn, MinifloatMeta
from mase_triton_b200.mxfp import functional as MX
from mase_triton_b200.mxfp import gemm as G
from mase_triton_b200.mxfp.layers import MXFPLinearPTQ
from mase_triton_b200.mxfp.meta import MXFP8_E4M3_fn, MXFP8_E5M2_fn, OCP_MXFP4_E2M1, OCP_MXFP6_E2M3, OCP_MXFP6_E3M2

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
MX_ALL = [MXFP8_E4M3_fn, MXFP8_E5M2_fn, OCP_MXFP6_E2M3, OCP_MXFP6_E3M2, OCP_MXFP4_E2M1]
DTYPES = [torch.bfloat16, torch.float16]


def within_tolerance(y: torch.Tensor, y32: torch.Tensor) -> bool:
    tol = 2.0**-7 * y32.abs() + 2.0**-7 * y32.pow(2).mean().sqrt()
    return bool(((y.float() - y32).abs() <= tol).all())


def same_values(got: torch.Tensor, want: torch.Tensor) -> bool:
    """Equal values (a sum of one term and zeros cannot keep the sign of a zero), NaNs at the same places."""
    gn, wn = got.isnan(), want.isnan()
    return bool(torch.equal(gn, wn)) and bool(torch.equal(got.masked_fill(gn, 0), want.masked_fill(wn, 0)))


@pytest.mark.parametrize("shape", [(256, 256, 64), (128, 512, 128), (300, 520, 200), (1, 8, 8), (1000, 2000, 1024), (513, 257, 96),
                                   (2048, 4096, 4096)])
@pytest.mark.parametrize("dtype", DTYPES, ids=["bf16", "f16"])
def test_dense_linear(lib, shape, dtype):
    M, N, K = shape
    torch.manual_seed(M * 7 + N + K)
    x = torch.randn(M, K, device=DEV).to(dtype)
    w = (0.05 * torch.randn(N, K, device=DEV)).to(dtype)
    bias = torch.randn(N, device=DEV).to(dtype)
    y32 = x.float() @ w.float().t()
    y = tc_linear.dense_linear(x, w)
    G.check_status(DEV)
    assert y.shape == (M, N) and y.dtype == dtype
    assert within_tolerance(y, y32), (y.float() - y32).abs().max().item()
    yb = tc_linear.dense_linear(x.reshape(1, M, K), w, bias)
    G.check_status(DEV)
    assert yb.shape == (1, M, N) and within_tolerance(yb.reshape(M, N), y32 + bias.float())


@pytest.mark.parametrize("meta", MX_ALL, ids=lambda m: m.tag)
@pytest.mark.parametrize("dtype", DTYPES, ids=["bf16", "f16"])
def test_mxfp_weight_expansion_is_the_reference_compose(lib, meta, dtype):
    """x = identity: out[i, n] = dequant(W)[n, i] exactly (one non-zero product per output, fp32 accumulate)."""
    K, N = 512, 300
    g = torch.Generator().manual_seed(11)
    w = torch.randn(N, K, generator=g) * torch.exp2(torch.randint(-20, 14, (N, 1), generator=g).float())
    s, e = oracle.extract_mxfp_components(w.flatten(), meta)
    s, e = s.clone(), e.clone()
    nb = K // 32
    # every code of the format, and the scale bytes at the edges: smallest (2^-127), around the range where
    # one bf16 multiply no longer covers scale and re-bias together, and the largest finite one
    e.view(N, K)[0, :256] = torch.arange(256, dtype=torch.uint8) & ((1 << (meta.element_exp_bits + meta.element_frac_bits + 1)) - 1)
    for j, sb in enumerate((0, 1, 2, 126, 127, 128, 134, 135, 142, 143, 200, 253, 254)):
        s.view(N, nb)[1 + j, :] = sb
    want = oracle.compose_mxfp_tensor(s, e, meta, dtype).reshape(N, K)           # what compose(..., output_dtype=dtype) gives
    x = torch.eye(K, dtype=dtype, device=DEV)
    got = tc_linear.mxfp_weight_linear(x, s.to(DEV), e.to(DEV), (N, K), meta)
    G.check_status(DEV)
    # 0 * Inf inside a dot product is NaN for the whole output, as in a dense linear on the composed weight
    ref = torch.nn.functional.linear(x.float(), want.to(DEV).float()).to(dtype)
    assert same_values(got.cpu(), ref.cpu())
    finite_rows = torch.isfinite(want.float()).all(dim=1)
    assert same_values(got.cpu().t()[finite_rows], want[finite_rows])


@pytest.mark.parametrize("fmt", [(4, 3, True), (5, 2, True), (3, 2, True), (2, 1, True), (5, 10, True), (8, 7, True), (4, 3, False), (3, 4, True)],
                         ids=lambda f: f"E{f[0]}M{f[1]}{'' if f[2] else '_inf'}")
@pytest.mark.parametrize("dtype", DTYPES, ids=["bf16", "f16"])
def test_minifloat_weight_expansion_is_the_reference_compose(lib, fmt, dtype):
    eb, fb, fin = fmt
    K, N = 256, 264
    meta = mf_meta(eb, fb, fin)
    g = torch.Generator().manual_seed(5)
    n_codes = 1 << (eb + fb + 1)
    codes = torch.randint(0, n_codes, (N, K), generator=g, dtype=torch.int32)
    codes[0, :] = torch.arange(K) % n_codes
    if not fin:
        # keep the Inf / NaN codes (all-ones exponent) to the first rows so that the others stay comparable
        top = ((codes >> fb) & ((1 << eb) - 1)) == (1 << eb) - 1
        codes[8:] = torch.where(top[8:], codes[8:] & ~(1 << fb), codes[8:])
    codes16 = codes.to(torch.uint16)
    want = oracle.compose_minifloat_component(codes16, meta, dtype)
    x = torch.eye(K, dtype=dtype, device=DEV)
    tm = SimpleMeta(eb, fb, fin)
    got = tc_linear.minifloat_weight_linear(x, codes16.to(DEV), (N, K), tm)
    G.check_status(DEV)
    ref = torch.nn.functional.linear(x.float(), want.to(DEV).float()).to(dtype)
    assert same_values(got.cpu(), ref.cpu())
    finite_rows = torch.isfinite(want.float()).all(dim=1)
    if finite_rows.any():
        assert same_values(got.cpu().t()[finite_rows], want[finite_rows])


class SimpleMeta:
    def __init__(self, eb, fb, fin):
        self.exp_bits, self.frac_bits, self.is_finite = eb, fb, fin


@pytest.mark.parametrize("meta", MX_ALL, ids=lambda m: m.tag)
@pytest.mark.parametrize("shape", [(256, 512, 256), (300, 1000, 160), (64, 256, 4096), (1024, 768, 1056)])
def test_mxfp_weight_linear_random(lib, meta, shape):
    M, N, K = shape
    torch.manual_seed(N + K)
    for dtype in DTYPES:
        x = torch.randn(M, K, device=DEV).to(dtype)
        w = (0.05 * torch.randn(N, K)).to(dtype)
        s, e = oracle.extract_mxfp_components(w.flatten(), meta)
        w_dq = oracle.compose_mxfp_tensor(s, e, meta, torch.float32).reshape(N, K).to(DEV)
        bias = torch.randn(N, device=DEV).to(dtype)
        y = tc_linear.mxfp_weight_linear(x, s.to(DEV), e.to(DEV), (N, K), meta, bias)
        G.check_status(DEV)
        assert within_tolerance(y, x.float() @ w_dq.t() + bias.float()), (meta.tag, dtype)


@pytest.mark.parametrize("layer_type", ["XWB", "XWqB", "XqWB", "XqWqB", "XWBq", "XqWqBq"])
@pytest.mark.parametrize("dtype", DTYPES, ids=["bf16", "f16"])
def test_every_mxfp_layer_type_runs_fused(lib, layer_type, dtype):
    """backend='fused' gives, within tolerance, the fp32 linear of the oracle-dequantised operands for every
    layer type, including block sizes the block-scaled GEMM does not take (then both operands are dequantised
    first and the dense tensor-core GEMM multiplies them)."""
    torch.manual_seed(17)
    M, N, K = 192, 320, 512
    for x_meta, w_meta in ((MXFP8_E4M3_fn, OCP_MXFP6_E3M2), (mx_real(16, 4, 3), mx_real(16, 2, 1))):
        fc = torch.nn.Linear(K, N, bias=True, device=DEV, dtype=dtype)
        xm = x_meta if "Xq" in layer_type else None
        wm = w_meta if "Wq" in layer_type else None
        bm = MXFP8_E4M3_fn if "Bq" in layer_type else None
        layer = MXFPLinearPTQ.from_linear(fc, xm, wm, bm, layer_type, backend="fused")
        x = (torch.randn(M, K, device=DEV) * 2).to(dtype)
        y = layer(x)
        G.check_status(DEV)
        x_dq = oracle_mx(x, xm) if xm else x.float().cpu()
        w_dq = oracle_mx(fc.weight.detach(), wm) if wm else fc.weight.detach().float().cpu()
        b_used = None if bm is not None else fc.bias.detach().float().cpu()      # a quantised bias is dropped, as in the reference
        y32 = torch.nn.functional.linear(x_dq, w_dq, b_used)
        assert y.dtype == dtype and within_tolerance(y.cpu(), y32), layer_type


def mx_real(block, eb, fb):
    from mase_triton_b200.mxfp.meta import MXFPMeta
    return MXFPMeta(block_size=block, scale_exp_bits=8, element_exp_bits=eb, element_frac_bits=fb, element_is_finite=True, round_mode="rn")


def oracle_mx(t: torch.Tensor, meta) -> torch.Tensor:
    s, e = oracle.extract_mxfp_components(t.detach().cpu().flatten(), meta)
    return oracle.compose_mxfp_tensor(s, e, meta, torch.float32).reshape(t.shape)


def test_fused_refuses_what_it_cannot_run(lib):
    """fp32 operands of a mixed layer type have no tensor-core kernel here: the call says so instead of
    running a library GEMM."""
    fc = torch.nn.Linear(64, 32, bias=False, device=DEV, dtype=torch.float32)
    layer = MXFPLinearPTQ.from_linear(fc, None, MXFP8_E4M3_fn, None, "XWqB", backend="fused")
    with pytest.raises(NotImplementedError):
        layer(torch.randn(4, 64, device=DEV))
    with pytest.raises(NotImplementedError):
        MF.minifloat_matmul(torch.randn(4, 64, device=DEV), torch.randn(64, 8, device=DEV), FP8_E4M3_fn, None, "XqW", "fused")
    with pytest.raises(NotImplementedError):
        MX.mxfp_matmul(torch.randn(4, 64, device=DEV), torch.randn(64, 8, device=DEV), None, MXFP8_E4M3_fn, "XWq", "fused")
    # both operands quantised in fp32 stay on the block-scaled kernel
    both = MXFPLinearPTQ.from_linear(fc, MXFP8_E4M3_fn, MXFP8_E4M3_fn, None, "XqWqB", backend="fused")
    assert both(torch.randn(4, 64, device=DEV)).dtype == torch.float32
    G.check_status(DEV)


@pytest.mark.parametrize("fmt", [(3, 4), (4, 2), (5, 1), (4, 3)], ids=lambda f: f"E{f[0]}M{f[1]}")
@pytest.mark.parametrize("layer_type", ["XqWqB", "XWqB", "XqWB"])
def test_minifloat_linear_fused_any_format(lib, fmt, layer_type):
    """Formats without an exact 8-bit tensor-core encoding (E3M4, E4M2, E5M1) take the kind::f16 GEMM."""
    torch.manual_seed(3)
    meta = MinifloatMeta(exp_bits=fmt[0], frac_bits=fmt[1], is_finite=True, round_mode="rn")
    M, N, K = 100, 200, 256
    fc = torch.nn.Linear(K, N, bias=True, device=DEV, dtype=torch.bfloat16)
    xm = meta if "Xq" in layer_type else None
    wm = meta if "Wq" in layer_type else None
    layer = MinifloatLinearPTQ.from_linear(fc, xm, wm, None, layer_type, "fused")
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    y = layer(x)
    G.check_status(DEV)
    x_dq = oracle.quantize_dequantize_minifloat(x.cpu(), xm).float() if xm else x.float().cpu()
    w_dq = oracle.quantize_dequantize_minifloat(fc.weight.detach().cpu(), wm).float() if wm else fc.weight.detach().float().cpu()
    y32 = torch.nn.functional.linear(x_dq, w_dq, fc.bias.detach().float().cpu())
    assert within_tolerance(y.cpu(), y32)


@pytest.mark.parametrize("func_type", ["XW", "XqW", "XWq", "XqWq"])
def test_matmul_fused_all_forms(lib, func_type):
    torch.manual_seed(23)
    a = (torch.randn(2, 3, 64, 256, device=DEV) * 2).to(torch.bfloat16)
    b = torch.randn(3, 256, 96, device=DEV).to(torch.bfloat16)
    xm = MXFP8_E4M3_fn if "Xq" in func_type else None
    wm = OCP_MXFP6_E2M3 if "Wq" in func_type else None
    y = MX.mxfp_matmul(a, b, xm, wm, func_type, "fused")
    G.check_status(DEV)
    y_sep = MX.mxfp_matmul(a.float(), b.float(), xm, wm, func_type, "separate")
    assert y.shape == (2, 3, 64, 96) and within_tolerance(y, y_sep)
    y2 = MX.mxfp_matmul(a, b[0], xm, wm, func_type, "fused")
    assert within_tolerance(y2, MX.mxfp_matmul(a.float(), b[0].float(), xm, wm, func_type, "separate"))
    mm = FP8_E4M3_fn
    z = MF.minifloat_matmul(a, b, mm if "Xq" in func_type else None, mm if "Wq" in func_type else None, func_type, "fused")
    z_sep = MF.minifloat_matmul(a.float(), b.float(), mm if "Xq" in func_type else None, mm if "Wq" in func_type else None, func_type, "separate")
    G.check_status(DEV)
    assert within_tolerance(z, z_sep)


@pytest.mark.parametrize("round_mode", ["rn", "rz", "ru", "rd"])
@pytest.mark.parametrize("fmt", [(4, 3), (5, 2)], ids=["E4M3", "E5M2"])
def test_fused_activation_honours_round_mode(lib, round_mode, fmt):
    """With an identity weight (exact in MXFP8) the fused linear returns the quantised activation itself, so
    the rounding mode of the activation's meta must show bit for bit."""
    from mase_triton_b200.mxfp.meta import MXFPMeta
    K = 256
    g = torch.Generator().manual_seed(9)
    # magnitudes within a factor of four per row: a block that holds the saturated top code is stored with its
    # elements halved, which is exact only while no element is a subnormal code
    x = (torch.rand(96, K, generator=g) * 0.75 + 0.25) * torch.exp2(torch.randint(-8, 8, (96, 1), generator=g).float())
    x = x * (torch.randint(0, 2, (96, K), generator=g).float() * 2 - 1)
    x_meta = MXFPMeta(block_size=32, scale_exp_bits=8, element_exp_bits=fmt[0], element_frac_bits=fmt[1], element_is_finite=True,
                      round_mode=round_mode)
    want = oracle_mx(x, x_meta)
    eye = torch.eye(K, device=DEV)
    ws, we, wtm = MX.extract_mxfp_components(eye, 1, MXFP8_E4M3_fn)
    y = MX.mxfp_linear(x.to(DEV), x_meta, None, ws, we, wtm, None, None, None, None, "XqWqB", "fused")
    G.check_status(DEV)
    assert torch.equal(y.cpu(), want)
    a = G.pack_activation(x.to(DEV), x_meta)
    b = G.quantize_pack(x.to(DEV), x_meta)
    assert torch.equal(a.codes, b.codes) and torch.equal(a.sf, b.sf)


@pytest.mark.parametrize("kind", ["mxfp", "minifloat"])
def test_weight_only_layer_routes_agree(lib, kind):
    """A weight-only-quantised layer expands its codes inside the GEMM's loader for short activations of wide
    layers and once (compose kernel + the same GEMM on dense operands) otherwise: both give the same bytes."""
    torch.manual_seed(23)
    N, K = 8192, 256
    fc = torch.nn.Linear(K, N, bias=True, device=DEV, dtype=torch.bfloat16)
    if kind == "mxfp":
        layer = MXFPLinearPTQ.from_linear(fc, None, OCP_MXFP6_E3M2, None, "XWqB", backend="fused")
    else:
        layer = MinifloatLinearPTQ.from_linear(fc, None, FP8_E4M3_fn, None, "XWqB", backend="fused")
    assert tc_linear.expand_in_loader(512, N) and not tc_linear.expand_in_loader(513, N) and not tc_linear.expand_in_loader(64, 4096)
    x = torch.randn(768, K, device=DEV, dtype=torch.bfloat16)
    tall = layer(x)                       # 768 rows: expanded once
    short = layer(x[:512])                # 512 rows: expanded in the loader
    G.check_status(DEV)
    assert torch.equal(tall[:512], short)
