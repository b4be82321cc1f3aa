"""Linear / matmul functions and the PTQ layers on the GPU: exact agreement with the reference's
"dequantise, then dense linear" semantics, the reference's own error bounds, and the module
invariants (state, .to(), from_quantized)."""

from __future__ import annotations

import pytest
import torch

import oracle
from mase_triton_b200.minifloat import functional as MF
from mase_triton_b200.minifloat.layers import MinifloatLinearPTQ
from mase_triton_b200.mxfp import gemm as G
from mase_triton_b200.minifloat.meta import FP4_E2M1_fn, FP6_E3M2_fn, FP8_E4M3_fn, FP8_E5M2_fn
from mase_triton_b200.mxfp import functional as MX
from mase_triton_b200.mxfp.layers import MXFPLinearPTQ
from mase_triton_b200.mxfp.meta import MXFP8_E4M3_fn, MXFP8_E5M2_fn, OCP_MXFP4_E2M1, OCP_MXFP6_E2M3, OCP_MXFP6_E3M2
from mase_triton_b200.utils.qlayer import ChangeDtypeError, devices_equal

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
MX_METAS = [MXFP8_E4M3_fn, MXFP8_E5M2_fn, OCP_MXFP6_E2M3, OCP_MXFP6_E3M2, OCP_MXFP4_E2M1, None]


def layer_type_of(x_meta, w_meta, b_meta):
    return ("Xq" if x_meta else "X") + ("Wq" if w_meta else "W") + ("Bq" if b_meta else "B")


def oracle_mx_qdq(t: torch.Tensor, meta, block_dim=-1) -> torch.Tensor:
    flat = t.cpu().movedim(block_dim % t.ndim, -1)
    s, e = oracle.extract_mxfp_components(flat.flatten(), meta)
    return oracle.compose_mxfp_tensor(s, e, meta, t.dtype).reshape(flat.shape).movedim(-1, block_dim % t.ndim)


@pytest.mark.parametrize("x_meta", MX_METAS, ids=lambda m: m.tag if m else "None")
@pytest.mark.parametrize("w_meta", [MXFP8_E4M3_fn, OCP_MXFP6_E3M2, OCP_MXFP4_E2M1, None], ids=lambda m: m.tag if m else "None")
@pytest.mark.parametrize("bias", [True, False])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_mxfp_linear_ptq_from_linear(lib, x_meta, w_meta, bias, dtype):
    torch.manual_seed(42)
    M, N, K = 128, 512, 1024
    b_meta = MXFP8_E4M3_fn if bias and w_meta is OCP_MXFP4_E2M1 else None
    lt = layer_type_of(x_meta, w_meta, b_meta)
    fc = torch.nn.Linear(K, N, bias=bias, device=DEV, dtype=dtype)
    q = MXFPLinearPTQ.from_linear(fc, x_meta, w_meta, b_meta, lt, backend="separate")
    x = torch.randn(M, K, device=DEV, dtype=dtype) * 3
    y_ref, y = fc(x), q(x)
    assert y.shape == y_ref.shape and y.dtype == dtype
    err = ((y_ref - y).abs().mean() / y_ref.abs().mean()).item()
    assert err < (0.4 if OCP_MXFP4_E2M1 in (x_meta, w_meta) else 0.25)          # reference bound
    # exact semantics: dequantised operands (oracle) through the same dense linear
    x_dq = oracle_mx_qdq(x, x_meta).to(DEV) if x_meta else x
    w_dq = oracle_mx_qdq(fc.weight.detach(), w_meta, 1).to(DEV) if w_meta else fc.weight
    b_used = None if b_meta is not None else fc.bias            # a quantised bias is dropped, as in the reference
    y_exact = torch.nn.functional.linear(x_dq, w_dq, b_used)
    assert torch.equal(y, y_exact)
    if x_meta is not None and w_meta is not None:
        y_fused = MXFPLinearPTQ.from_linear(fc, x_meta, w_meta, b_meta, lt, backend="fused")(x)
        tol = 2.0**-7 * y_exact.float().abs() + 2.0**-7 * y_exact.float().pow(2).mean().sqrt()
        assert bool(((y_fused.float() - y_exact.float()).abs() <= tol).all())


def test_mxfp_from_quantized_and_state(lib):
    torch.manual_seed(0)
    fc = torch.nn.Linear(256, 64, bias=True, device=DEV, dtype=torch.bfloat16)
    a = MXFPLinearPTQ.from_linear(fc, MXFP8_E4M3_fn, OCP_MXFP6_E3M2, None, "XqWqB", "separate")
    assert a.w_scales.dtype == torch.uint8 and a.w_scales.shape == (64 * 256 // 32, 1)
    assert a.w_elements.shape == (64 * 256 // 32, 32) and a.weight is None
    assert set(a.state_dict()) == {"w_scales", "w_elements", "bias"}
    assert (a.w_tensor_meta.shape, a.w_tensor_meta.block_dim, a.w_tensor_meta.dtype) == ((64, 256), 1, "bfloat16")
    b = MXFPLinearPTQ.from_quantized(a.w_scales, a.w_elements, a.w_tensor_meta, a.bias, None, None, None,
                                     MXFP8_E4M3_fn, "XqWqB", "separate")
    x = torch.randn(8, 256, device=DEV, dtype=torch.bfloat16)
    assert torch.equal(a(x), b(x)) and (b.in_features, b.out_features) == (256, 64)
    with pytest.raises(ValueError):
        MXFPLinearPTQ(None, fc.bias, None, None, None, "XWqBq", "separate", w_scales=a.w_scales, w_elements=a.w_elements,
                      w_tensor_meta=a.w_tensor_meta, b_scales=a.w_scales, b_elements=a.w_elements, b_tensor_meta=a.w_tensor_meta)
    with pytest.raises(NotImplementedError):
        MX.mxfp_linear(x, None, fc.weight, None, None, None, None, None, None, None, "bogus", "separate")
    assert "layer_type=XqWqB" in repr(a)


def test_mxfp_layer_to_invariants(lib):
    fc = torch.nn.Linear(64, 32, bias=True, dtype=torch.float32)
    layer = MXFPLinearPTQ.from_linear(fc.to(DEV), MXFP8_E4M3_fn, MXFP8_E4M3_fn, MXFP8_E4M3_fn, "XqWqBq", "separate")
    assert layer.b_scales is not None and layer.bias is None
    layer.to(torch.float16)                                  # floating casts leave the integer codes alone
    assert layer.w_scales.dtype == torch.uint8 and layer.b_elements.dtype == torch.uint8
    with pytest.raises(ChangeDtypeError):
        layer._apply(lambda t: t.to(torch.float32))          # anything that re-types the codes is refused
    cpu = MXFPLinearPTQ.from_linear(fc.to(DEV), None, MXFP8_E4M3_fn, None, "XWqB", "separate").to("cpu")
    assert cpu.w_tensor_meta.device == "cpu" and cpu.w_scales.device.type == "cpu" and cpu.w_scales.dtype == torch.uint8
    back = cpu.to(DEV)
    assert devices_equal(back.w_tensor_meta.device, DEV) and back.bias.dtype == torch.float32
    y = back(torch.randn(4, 64, device=DEV))
    assert y.shape == (4, 32)


# reference: test/test_mxfp_functional.py:183-265
@pytest.mark.parametrize("x_meta", [None, MXFP8_E4M3_fn, OCP_MXFP4_E2M1], ids=lambda m: m.tag if m else "None")
@pytest.mark.parametrize("y_meta", [None, MXFP8_E5M2_fn, OCP_MXFP6_E2M3], ids=lambda m: m.tag if m else "None")
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_mxfp_matmul(lib, x_meta, y_meta, dtype):
    torch.manual_seed(1)
    ft = ("Xq" if x_meta else "X") + ("Wq" if y_meta else "W")
    a = torch.randn((2, 4, 128, 1024), dtype=dtype, device=DEV) * 5
    b = torch.randn((2, 4, 1024, 512), dtype=dtype, device=DEV) * 3
    y_ref = torch.matmul(a, b)
    y = MX.mxfp_matmul(a, b, input_meta=x_meta, other_meta=y_meta, func_type=ft, backend="separate")
    assert y.shape == y_ref.shape
    err = ((y - y_ref).abs().mean() / y_ref.abs().mean()).item()
    if x_meta is None and y_meta is None:
        assert err == 0
    else:
        assert err < (0.5 if OCP_MXFP4_E2M1 in (x_meta, y_meta) else 0.45 if OCP_MXFP6_E2M3 in (x_meta, y_meta) else 0.25)
    a_dq = oracle_mx_qdq(a, x_meta, -1).to(DEV) if x_meta else a
    b_dq = oracle_mx_qdq(b, y_meta, -2).to(DEV) if y_meta else b
    assert torch.equal(y, torch.matmul(a_dq, b_dq))


@pytest.mark.parametrize("x_meta", [FP8_E4M3_fn, FP4_E2M1_fn, None], ids=lambda m: m.tag if m else "None")
@pytest.mark.parametrize("w_meta", [FP8_E5M2_fn, FP6_E3M2_fn, None], ids=lambda m: m.tag if m else "None")
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_minifloat_linear_ptq(lib, x_meta, w_meta, dtype):
    torch.manual_seed(7)
    lt = layer_type_of(x_meta, w_meta, None)
    fc = torch.nn.Linear(512, 256, bias=True, device=DEV, dtype=dtype)
    q = MinifloatLinearPTQ.from_linear(fc, x_meta, w_meta, None, lt, "separate")
    x = torch.randn(64, 512, device=DEV, dtype=dtype)
    y = q(x)
    x_dq = oracle.quantize_dequantize_minifloat(x.cpu(), x_meta).to(DEV) if x_meta else x
    w_dq = oracle.quantize_dequantize_minifloat(fc.weight.detach().cpu(), w_meta).to(DEV) if w_meta else fc.weight
    assert torch.equal(y, torch.nn.functional.linear(x_dq, w_dq, fc.bias))
    if w_meta is not None:
        assert q.w_element.dtype == torch.uint16 and q.w_element.shape == (256, 512)
        r = MinifloatLinearPTQ.from_quantized(q.w_element, q.w_tensor_meta, q.bias, None, None, x_meta, lt, "fused")
        if x_meta is not None or dtype == torch.bfloat16:
            # the fused backend multiplies on the tensor cores: 8-bit codes of both operands, or (weight only
            # quantised, bf16 activation) the weight codes expanded inside the GEMM's loader
            y32 = torch.nn.functional.linear(x_dq.float(), w_dq.float(), fc.bias.float())
            tol = 2.0**-7 * y32.abs() + 2.0**-7 * y32.pow(2).mean().sqrt()
            assert bool(((r(x).float() - y32).abs() <= tol).all()) and r(x).dtype == dtype
            G.check_status(torch.device(DEV))
        else:
            with pytest.raises(NotImplementedError):        # fp32 activation, weight-only quantisation: no tensor-core kernel
                r(x)
        with pytest.raises(ChangeDtypeError):
            q._apply(lambda t: t.to(torch.float32))
    ym = MF.minifloat_matmul(x, fc.weight.t().contiguous(), x_meta, w_meta, ("Xq" if x_meta else "X") + ("Wq" if w_meta else "W"), "separate")
    assert torch.equal(ym, torch.matmul(x_dq, w_dq.t().contiguous()))


@pytest.mark.parametrize("rows,chunk", [(1000, 256), (512, 512), (37, 64), (300, 4096)])
def test_host_pipeline_matches_device_result(lib, rows, chunk):
    """The chunked pinned-host -> device -> pinned-host front end gives the bytes of one device-resident
    call, for row counts that are not a multiple of the chunk and for a single chunk."""
    from mase_triton_b200.hostpath import HostPipeline
    from mase_triton_b200.minifloat import kernels as mfk
    from mase_triton_b200.mxfp import kernels as mxk
    g = torch.Generator().manual_seed(rows)
    x = (torch.randn((rows, 2048), generator=g) * torch.exp2(torch.randint(-20, 20, (rows, 1), generator=g).float())).pin_memory()
    out = torch.empty_like(x).pin_memory()
    dev = torch.device(DEV)
    for op, direct in (
        (lambda a, b: mfk.quantize_dequantize(a, FP8_E4M3_fn, torch.float32, out=b),
         lambda t: mfk.quantize_dequantize(t, FP8_E4M3_fn, torch.float32)),
        (lambda a, b: mxk.quantize_dequantize(a.reshape(-1), MXFP8_E4M3_fn, torch.float32, out=b.reshape(-1)),
         lambda t: mxk.quantize_dequantize(t.reshape(-1), MXFP8_E4M3_fn, torch.float32).reshape(t.shape)),
    ):
        pipe = HostPipeline(op, dev, chunk_rows=chunk)
        for _ in range(2):                       # the second pass re-uses the staging buffers
            out.zero_()
            pipe.run(x, out)
            torch.cuda.synchronize()
            want = direct(x.to(dev)).cpu()
            assert torch.equal(out.view(torch.int32), want.view(torch.int32))
        assert pipe.launches == 2 * ((rows + min(chunk, rows) - 1) // min(chunk, rows))


def test_kernel_manager_autotune_picks_a_tile_width(lib):
    """With KernelManager autotune on, a fused layer times the candidate tile widths at its first call for an
    activation height, records the choice, and returns the same bytes as without tuning (the tile width does not
    change the order in which an output element is accumulated)."""
    from mase_triton_b200.manager import KernelManager

    torch.manual_seed(31)
    fc = torch.nn.Linear(256, 1000, bias=True, device=DEV, dtype=torch.bfloat16)
    x = torch.randn(300, 256, device=DEV, dtype=torch.bfloat16)
    plain = MXFPLinearPTQ.from_linear(fc, MXFP8_E4M3_fn, OCP_MXFP6_E3M2, None, "XqWqB", "fused")
    want = plain(x)
    KernelManager.enable_autotune()
    try:
        tuned = MXFPLinearPTQ.from_linear(fc, MXFP8_E4M3_fn, OCP_MXFP6_E3M2, None, "XqWqB", "fused")
        got = tuned(x)
        got_functional = MX.mxfp_linear(x, MXFP8_E4M3_fn, None, tuned.w_scales, tuned.w_elements, tuned.w_tensor_meta, tuned.bias, None, None,
                                        None, "XqWqB", "fused")
        G.check_status(DEV)
        choices = {k: v for k, v in KernelManager.tuned_choices().items() if k[0] == "mx_gemm tile_rows" and k[2:] == (1000, 256)}
        assert len(choices) == 1
        (rec,) = choices.values()
        assert rec["choice"] in G.TILE_ROW_CANDIDATES and rec["choice"] == min(rec["ms"], key=rec["ms"].get) and len(rec["ms"]) >= 2
        assert tuned.tensor_core_weight(300).tile_rows == rec["choice"]
    finally:
        KernelManager.disable_autotune()
    assert torch.equal(got, want) and torch.equal(got_functional, want)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_mxfp4_layer_runs_on_packed_nibbles(lib, dtype):
    """An MXFP4 x MXFP4 fused layer keeps weight and activation as packed 4-bit codes (the 4-bit x 4-bit tensor-core
    kind) when in_features is a multiple of 256, and the widened 8-bit form otherwise; both match the fp32 linear of
    the oracle-dequantised operands, and the functional entry gives the layer's bytes."""
    torch.manual_seed(41)
    for K, packed in ((512, True), (384, False)):
        fc = torch.nn.Linear(K, 1000, bias=True, device=DEV, dtype=dtype)
        layer = MXFPLinearPTQ.from_linear(fc, OCP_MXFP4_E2M1, OCP_MXFP4_E2M1, None, "XqWqB", backend="fused")
        x = (torch.randn(3, 100, K, device=DEV) * 2).to(dtype)
        y = layer(x)
        G.check_status(DEV)
        wq = layer.tensor_core_weight()
        assert (wq.hw_format == 5) == packed and wq.codes.numel() == (1000 * K // 2 if packed else 1000 * K)
        def oracle_dq(t):
            flat = t.detach().cpu().reshape(-1)
            return oracle.compose_mxfp_tensor(*oracle.extract_mxfp_components(flat, OCP_MXFP4_E2M1), OCP_MXFP4_E2M1, torch.float32).reshape(-1, K)

        y32 = torch.nn.functional.linear(oracle_dq(x), oracle_dq(fc.weight), fc.bias.detach().float().cpu()).reshape(3, 100, 1000)
        tol = 2.0**-7 * y32.abs() + 2.0**-7 * y32.pow(2).mean().sqrt()
        assert y.shape == (3, 100, 1000) and y.dtype == dtype and bool(((y.float().cpu() - y32).abs() <= tol).all())
        y_fn = MX.mxfp_linear(x, OCP_MXFP4_E2M1, None, layer.w_scales, layer.w_elements, layer.w_tensor_meta, layer.bias, None, None, None,
                              "XqWqB", "fused")
        shared = layer.forward_packed(layer.pack_input(x), dtype, lead_shape=(3, 100))
        G.check_status(DEV)
        assert torch.equal(y_fn, y) and torch.equal(shared, y)


def test_minifloat_fp4_layer_runs_on_packed_nibbles(lib):
    """A per-tensor FP4 x FP4 fused layer takes the 4-bit tensor-core kind (unit block scales) when in_features is a
    multiple of 256 and gives the bytes of the widened 8-bit form it takes otherwise."""
    from mase_triton_b200.minifloat.functional import linear as ML

    torch.manual_seed(43)
    fc = torch.nn.Linear(512, 600, bias=True, device=DEV, dtype=torch.bfloat16)
    with torch.no_grad():
        fc.weight.mul_(20.0)                              # spread the weights over the FP4 range
    layer = MinifloatLinearPTQ.from_linear(fc, FP4_E2M1_fn, FP4_E2M1_fn, None, "XqWqB", backend="fused")
    x = (torch.randn(200, 512, device=DEV) * 2).to(torch.bfloat16)
    y = layer(x)
    G.check_status(DEV)
    packed = ML._packed_weight(layer.w_element, layer.w_tensor_meta, True)
    assert packed.hw_format == 5 and packed.codes.numel() == 600 * 512 // 2
    x_dq = MF.quantize_dequantize(x, FP4_E2M1_fn, torch.float32).cpu()
    w_dq = MF.quantize_dequantize(fc.weight.detach(), FP4_E2M1_fn, torch.float32).cpu()
    y32 = torch.nn.functional.linear(x_dq, w_dq, fc.bias.detach().float().cpu())
    tol = 2.0**-7 * y32.abs() + 2.0**-7 * y32.pow(2).mean().sqrt()
    assert bool(((y.float().cpu() - y32).abs() <= tol).all())
    # the same layer computed with the codes widened to bytes
    codes = layer.w_element.reshape(600, 512).to(torch.uint8)
    wide_w = G.pack_codes(None, codes, 600, 512, 2, 1, G.OPERAND_B)
    from mase_triton_b200.minifloat import kernels as mfk
    a_wide = G.pack_codes(None, mfk.extract_minifloat_component(x, FP4_E2M1_fn).to(torch.uint8), 200, 512, 2, 1, G.OPERAND_A)
    assert torch.equal(G.mx_gemm(a_wide, wide_w, torch.bfloat16, bias=layer.bias), y)
