"""The block-scaled tensor-core GEMM against "dequantise, then fp32 matmul" on the same operands."""

from __future__ import annotations

import numpy as np
import pytest
import torch

import oracle
from mase_triton_b200.mxfp import functional as MX
from mase_triton_b200.mxfp import gemm as G
from mase_triton_b200.mxfp import kernels as mxk
from mase_triton_b200.mxfp.layers import MXFPLinearPTQ
from mase_triton_b200.mxfp.meta import MXFP8_E4M3_fn, MXFP8_E5M2_fn, OCP_MXFP4_E2M1, OCP_MXFP6_E2M3, OCP_MXFP6_E3M2

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ALL = [MXFP8_E4M3_fn, MXFP8_E5M2_fn, OCP_MXFP6_E2M3, OCP_MXFP6_E3M2, OCP_MXFP4_E2M1]


def dequant(x: torch.Tensor, meta) -> torch.Tensor:
    s, e = mxk.extract_mxfp_components(x.reshape(-1), meta)
    return mxk.compose_mxfp_tensor(s, e, meta, torch.float32).reshape(x.shape)


def within_tolerance(y: torch.Tensor, y32: torch.Tensor) -> bool:
    """|y - y32| <= 2^-7 |y32| + 2^-7 rms(y32): one bf16 ulp plus accumulation-order slack."""
    tol = 2.0**-7 * y32.abs() + 2.0**-7 * y32.pow(2).mean().sqrt()
    return bool(((y.float() - y32).abs() <= tol).all())


def test_pack_tables_preserve_values(lib):
    """Packing then reading the hardware bytes back as OCP FP8 gives the reference values
    (times 2 where a block was re-biased)."""
    torch.manual_seed(3)
    x = (torch.randn(256, 256, device=DEV) * 4).to(torch.bfloat16)
    for meta in ALL:
        s, e = mxk.extract_mxfp_components(x.reshape(-1), meta)
        p = G.pack_operand(s, e, 256, 256, meta, G.OPERAND_A)
        hw_dtype = torch.float8_e4m3fn if p.hw_format == 0 else torch.float8_e5m2
        vals = p.codes.view(hw_dtype).float()
        # un-chunk the scale factors: chunk (rt, kt) byte (r%32)*16 + (r/32)*4 + kb
        sf = p.sf.view(1, 2, 2, 32, 4, 4)                    # [row tile(256), k tile, chunk(128 rows), r%32, r/32, kb]
        sf = sf.permute(0, 2, 4, 3, 1, 5).reshape(256, 8)    # [row, k block]
        scale = torch.exp2(sf.float() - 127).repeat_interleave(32, dim=1)
        ref = dequant(x, meta)
        # halving a re-biased block is exact except for elements 2^-14 (E4M3) below the block maximum
        blockmax = ref.abs().reshape(256, 8, 32).amax(dim=2, keepdim=True).expand(256, 8, 32).reshape(256, 256)
        assert bool(((vals * scale - ref).abs() <= blockmax * 2.0**-16).all()), meta.tag
        assert not vals.isnan().any()
        if meta in (OCP_MXFP6_E2M3, OCP_MXFP6_E3M2, OCP_MXFP4_E2M1):
            assert torch.equal(vals * scale, ref), meta.tag


@pytest.mark.parametrize("shape", [(128, 256, 128), (128, 224, 512), (256, 512, 1024), (200, 300, 160), (1, 8, 32), (384, 1024, 4096),
                                   (2048, 4096, 512), (130, 230, 96), (1000, 2000, 1024)])
def test_gemm_e4m3_shapes(lib, shape):
    M, N, K = shape
    torch.manual_seed(M + N + K)
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    w = (0.05 * torch.randn(N, K, device=DEV)).to(torch.bfloat16)
    a = G.quantize_pack(x, MXFP8_E4M3_fn)
    b = G.quantize_pack(w, MXFP8_E4M3_fn, G.OPERAND_B)
    y32 = dequant(x, MXFP8_E4M3_fn) @ dequant(w, MXFP8_E4M3_fn).t()
    for dt in (torch.float32, torch.bfloat16, torch.float16):
        y = G.mx_gemm(a, b, dt)
        G.check_status(DEV)
        assert y.shape == (M, N) and y.dtype == dt
        assert within_tolerance(y, y32), f"{shape} {dt}: max err {(y.float() - y32).abs().max().item()}"
    bias = torch.randn(N, device=DEV).to(torch.bfloat16)
    yb = G.mx_gemm(a, b, torch.bfloat16, bias)
    G.check_status(DEV)
    assert within_tolerance(yb, y32 + bias.float())


@pytest.mark.parametrize("x_meta", ALL, ids=lambda m: m.tag)
@pytest.mark.parametrize("w_meta", ALL, ids=lambda m: m.tag)
def test_gemm_format_pairs(lib, x_meta, w_meta):
    torch.manual_seed(5)
    M, N, K = 256, 512, 512
    x = (torch.randn(M, K, device=DEV) * 3).to(torch.bfloat16)
    w = (0.02 * torch.randn(N, K, device=DEV)).to(torch.bfloat16)
    y = G.mx_gemm(G.quantize_pack(x, x_meta), G.quantize_pack(w, w_meta, G.OPERAND_B), torch.bfloat16)
    G.check_status(DEV)
    y32 = dequant(x, x_meta) @ dequant(w, w_meta).t()
    assert within_tolerance(y, y32)


def test_fused_linear_matches_separate(lib):
    """Benchmark configuration 4 at reduced M: x bf16 ~ N(0,1), W ~ N(0, 0.02), MXFP8 E4M3 both."""
    torch.manual_seed(0)
    M, N, K = 1024, 14336, 4096
    x = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    fc = torch.nn.Linear(K, N, bias=False, device=DEV, dtype=torch.bfloat16)
    with torch.no_grad():
        fc.weight.copy_((0.02 * torch.randn(N, K, device=DEV)).to(torch.bfloat16))
    sep = MXFPLinearPTQ.from_linear(fc, MXFP8_E4M3_fn, MXFP8_E4M3_fn, None, "XqWqB", "separate")
    fus = MXFPLinearPTQ.from_linear(fc, MXFP8_E4M3_fn, MXFP8_E4M3_fn, None, "XqWqB", "fused")
    y_sep, y_fus = sep(x), fus(x)
    G.check_status(DEV)
    y32 = dequant(x, MXFP8_E4M3_fn) @ dequant(fc.weight.detach(), MXFP8_E4M3_fn).t()
    assert within_tolerance(y_fus, y32)
    rel = ((y_fus.float() - y_sep.float()).abs().mean() / y_sep.float().abs().mean()).item()
    assert rel < 5e-3, rel
    # 3-D activations keep their leading dims
    y3 = fus(x.reshape(4, 256, K))
    assert y3.shape == (4, 256, N) and torch.equal(y3.reshape(M, N), y_fus)


@pytest.mark.parametrize("meta", [MXFP8_E4M3_fn, MXFP8_E5M2_fn], ids=lambda m: m.tag)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("shape", [(512, 1024), (300, 160), (1, 32), (2050, 4096)])
def test_one_pass_quantize_pack_equals_two_step(lib, meta, dtype, shape):
    torch.manual_seed(shape[0])
    x = (torch.randn(*shape, device=DEV) * torch.exp2(torch.randint(-6, 6, (shape[0], 1), device=DEV).float())).to(dtype)
    x[0, :4] = torch.tensor([0.0, -0.0, 1e-30, -1e-30], dtype=dtype)
    two = G.quantize_pack(x, meta)
    one = G.quantize_pack_fused(x, meta)
    assert one.hw_format == two.hw_format
    assert torch.equal(one.codes, two.codes)
    assert torch.equal(one.sf, two.sf)


@pytest.mark.parametrize("x_meta,w_meta", [(MXFP8_E4M3_fn, MXFP8_E4M3_fn), (MXFP8_E5M2_fn, OCP_MXFP6_E2M3), (OCP_MXFP4_E2M1, OCP_MXFP6_E3M2)],
                         ids=["e4m3-e4m3", "e5m2-e2m3", "e2m1-e3m2"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_fused_matmul_matches_separate(lib, x_meta, w_meta, dtype):
    """mxfp_matmul(backend="fused") on batched operands (reference shapes of test/test_mxfp_functional.py:183-265)."""
    torch.manual_seed(9)
    a = (torch.randn((2, 3, 128, 512), device=DEV) * 5).to(dtype)
    b = (torch.randn((2, 3, 512, 256), device=DEV) * 3).to(dtype)
    y_sep = MX.mxfp_matmul(a, b, x_meta, w_meta, "XqWq", "separate")
    y_fus = MX.mxfp_matmul(a, b, x_meta, w_meta, "XqWq", "fused")
    G.check_status(DEV)
    assert y_fus.shape == y_sep.shape == (2, 3, 128, 256) and y_fus.dtype == dtype
    a_dq = MX.quantize_dequantize(a, -1, x_meta, torch.float32)
    b_dq = MX.quantize_dequantize(b, -2, w_meta, torch.float32)
    assert within_tolerance(y_fus, torch.matmul(a_dq, b_dq))
    # a 2-D right operand is shared by every batch entry
    y2 = MX.mxfp_matmul(a, b[0, 0], x_meta, w_meta, "XqWq", "fused")
    G.check_status(DEV)
    assert within_tolerance(y2, torch.matmul(a_dq, b_dq[0, 0]))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("M,N,K,tile", [(256, 224, 128, None), (300, 448 + 64, 256, None), (100, 72, 96, None), (1024, 1792, 512, None),
                                        (2000, 1792, 256, 192), (128, 1000, 128, 160), (4096, 2048, 128, 192)])
def test_gather_epilogue_writes_every_destination(lib, dtype, M, N, K, tile):
    """The gather-fused kernel gives, in each destination and at the column offset, the bytes of the
    plain GEMM; columns outside the shard stay untouched.  Tiles narrower than the widest forward through more
    boxes (the unused end of each stage's B region), many tiles per CTA wrap the boxes' barriers several times."""
    torch.manual_seed(M + N)
    x = torch.randn((M, K), device=DEV, dtype=torch.bfloat16)
    w = (torch.randn((N, K), device=DEV) * 0.05).to(torch.bfloat16)
    bias = torch.randn((N,), device=DEV).to(dtype)
    a, b = G.quantize_pack(x, MXFP8_E4M3_fn), G.quantize_pack(w, OCP_MXFP6_E3M2, G.OPERAND_B, tile_rows=tile)
    want = G.mx_gemm(a, b, dtype, bias=bias)
    ld, off = N + 64, 40
    outs = [torch.full((M + 3, ld), 7.0, device=DEV, dtype=dtype) for _ in range(3)]
    G.mx_gemm_gather(a, b, [o.data_ptr() for o in outs], 1, ld, off, dtype, bias=bias)
    G.check_status(DEV)
    torch.cuda.synchronize()
    for o in outs:
        assert torch.equal(o[:M, off:off + N].view(torch.uint8), want.view(torch.uint8))
        assert bool((o[:M, :off] == 7).all()) and bool((o[:M, off + N:] == 7).all()) and bool((o[M:] == 7).all())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_minifloat_linear_fused_saturating_activation(lib, dtype):
    """Per-tensor minifloat codes through the block-scaled GEMM with unit scales: saturated values
    (reference E4M3 480, which the hardware format cannot hold) and signed zeros included."""
    from mase_triton_b200.minifloat import functional as MF
    from mase_triton_b200.minifloat.meta import FP6_E2M3_fn, FP8_E4M3_fn, FP8_E5M2_fn
    torch.manual_seed(21)
    for x_meta, w_meta in [(FP8_E4M3_fn, FP8_E4M3_fn), (FP8_E5M2_fn, FP6_E2M3_fn)]:
        x = (torch.randn((3, 50, 256), device=DEV) * 300).to(dtype)          # many values beyond the largest code
        x[0, 0, :8] = torch.tensor([0.0, -0.0, 1e-9, -1e-9, 480.0, -480.0, 1e6, -1e6], device=DEV).to(dtype)
        w = (torch.randn((96, 256), device=DEV) * 0.2).to(dtype)
        w_el, w_tm = MF.extract_minifloat_component(w, w_meta)
        bias = torch.randn((96,), device=DEV).to(dtype)
        y_sep = MF.minifloat_linear(x, x_meta, None, w_el, w_tm, bias, None, None, "XqWqB", "separate")
        y_fus = MF.minifloat_linear(x, x_meta, None, w_el, w_tm, bias, None, None, "XqWqB", "fused")
        G.check_status(DEV)
        assert y_fus.shape == y_sep.shape == (3, 50, 96) and y_fus.dtype == dtype
        x_dq = MF.quantize_dequantize(x, x_meta).float()
        w_dq = MF.compose_minifloat_component(w_el, w_tm).float()
        assert within_tolerance(y_fus, torch.nn.functional.linear(x_dq, w_dq, bias.float()))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_minifloat_one_pass_pack_equals_two_step(lib, dtype):
    """mxq_minifloat_quantize_pack gives the bytes of extract -> narrow -> pack with unit scales,
    saturated values, Inf/NaN inputs and ragged row counts included."""
    from helpers import adversarial_fp32
    from mase_triton_b200.minifloat import kernels as mfk
    from mase_triton_b200.minifloat.meta import FP8_E4M3_fn, FP8_E5M2_fn
    for meta in (FP8_E4M3_fn, FP8_E5M2_fn):
        for rows, K in ((300, 256), (129, 96), (5, 32)):
            x = adversarial_fp32(max(rows * K, 4096), seed=rows)[: rows * K].reshape(rows, K).clone()
            x[0, :4] = torch.tensor([480.0, -480.0, 1e9, float("inf")])
            x = x.to(dtype).to(DEV)
            one = G.minifloat_quantize_pack(x, meta.exp_bits, meta.frac_bits, meta.round_mode)
            assert one is not None
            codes = mfk.extract_minifloat_component(x, meta).to(torch.uint8)
            two = G.pack_codes(None, codes, rows, K, meta.exp_bits, meta.frac_bits, G.OPERAND_A)
            assert one.hw_format == two.hw_format
            assert torch.equal(one.codes, two.codes), f"{meta.tag} {dtype} {rows}x{K}: codes differ"
            assert torch.equal(one.sf, two.sf), f"{meta.tag} {dtype} {rows}x{K}: scale chunks differ"


def test_gemm_random_shapes(lib):
    """Ragged M and N, every K that is a multiple of 32 up to 640, all output dtypes and format pairs,
    against an fp32 matmul of the dequantised operands."""
    rng = np.random.default_rng(17)
    metas = [MXFP8_E4M3_fn, MXFP8_E5M2_fn, OCP_MXFP6_E2M3, OCP_MXFP6_E3M2, OCP_MXFP4_E2M1]
    for trial in range(24):
        M = int(rng.integers(1, 700)); N = int(rng.integers(1, 900)); K = 32 * int(rng.integers(1, 21))
        xm, wm = metas[trial % 5], metas[(trial // 5 + trial) % 5]
        dtype = (torch.bfloat16, torch.float16, torch.float32)[trial % 3]
        g = torch.Generator().manual_seed(trial)
        x = (torch.randn((M, K), generator=g) * float(rng.uniform(0.1, 30))).to(DEV)
        w = (torch.randn((N, K), generator=g) * float(rng.uniform(0.01, 3))).to(DEV)
        bias = torch.randn((N,), generator=g).to(dtype).to(DEV) if trial % 2 else None
        a, b = G.quantize_pack(x, xm), G.quantize_pack(w, wm, G.OPERAND_B)
        y = G.mx_gemm(a, b, dtype, bias=bias)
        G.check_status(DEV)
        x_dq = MX.quantize_dequantize(x, -1, xm, torch.float32)
        w_dq = MX.quantize_dequantize(w, -1, wm, torch.float32)
        y32 = x_dq @ w_dq.t() + (bias.float() if bias is not None else 0)
        assert y.shape == (M, N) and y.dtype == dtype
        assert within_tolerance(y, y32), f"trial {trial}: M={M} N={N} K={K} {xm.tag} x {wm.tag} {dtype}"


@pytest.mark.parametrize("w_meta", [OCP_MXFP6_E2M3, OCP_MXFP6_E3M2, OCP_MXFP4_E2M1], ids=lambda m: m.tag)
@pytest.mark.parametrize("x_meta", [MXFP8_E4M3_fn, MXFP8_E5M2_fn], ids=lambda m: m.tag)
@pytest.mark.parametrize("M,N,K", [(256, 448, 128), (300, 1000, 640), (128, 4096, 1024), (1, 16, 128)])
def test_native_subbyte_weight_equals_widened(lib, x_meta, w_meta, M, N, K):
    """FP6 / FP4 weights kept at their own width (dense 6- / 4-bit streams read through the packed tensor-map types)
    give the same products as the same codes widened to E4M3 bytes: the output bytes must be identical, with every
    code of the format present in the weight."""
    torch.manual_seed(M + N + K)
    x = (torch.randn(M, K, device=DEV) * 2).to(torch.bfloat16)
    bits = 1 + w_meta.element_exp_bits + w_meta.element_frac_bits
    w_elements = torch.randint(0, 1 << bits, (N * K // 32, 32), device=DEV, dtype=torch.uint8)
    w_elements.view(-1)[: 1 << bits] = torch.arange(1 << bits, device=DEV, dtype=torch.uint8)
    w_scales = torch.randint(118, 130, (N * K // 32, 1), device=DEV, dtype=torch.uint8)
    a = G.quantize_pack(x, x_meta)
    wide = G.pack_operand(w_scales, w_elements, N, K, w_meta, G.OPERAND_B, native=False)
    dense = G.pack_operand(w_scales, w_elements, N, K, w_meta, G.OPERAND_B, native=True)
    assert dense.hw_format in (3, 4, 5) and dense.codes.numel() == N * K * bits // 8 and wide.codes.numel() == N * K
    assert torch.equal(dense.sf, wide.sf)
    w32 = mxk.compose_mxfp_tensor(w_scales, w_elements, w_meta, torch.float32).reshape(N, K)
    y32 = dequant(x, x_meta) @ w32.t()
    for dt in (torch.bfloat16, torch.float32):
        y_wide = G.mx_gemm(a, wide, dt)
        y_dense = G.mx_gemm(a, dense, dt)
        G.check_status(DEV)
        assert within_tolerance(y_dense, y32), f"max err {(y_dense.float() - y32).abs().max().item()}"
        assert torch.equal(y_dense, y_wide)


@pytest.mark.parametrize("M,N,K", [(256, 448, 256), (300, 1000, 768), (128, 224, 512), (1000, 4096, 1024), (1, 16, 256)])
def test_fp4_by_fp4_on_the_4bit_tensor_core_kind(lib, M, N, K):
    """MXFP4 x MXFP4 with both operands kept as packed nibbles (tcgen05 kind::mxf4, 64 elements of K per instruction)
    against an fp32 matmul of the dequantised operands, and against the same product computed with the codes widened
    to E4M3 bytes (every product of two E2M1 values and two power-of-two scales is exact in both)."""
    torch.manual_seed(M + N + K)
    x = (torch.randn(M, K, device=DEV) * 2).to(torch.bfloat16)
    w = (0.05 * torch.randn(N, K, device=DEV)).to(torch.bfloat16)
    a4 = G.quantize_pack(x, OCP_MXFP4_E2M1, G.OPERAND_A, native=True)
    b4 = G.quantize_pack(w, OCP_MXFP4_E2M1, G.OPERAND_B, native=True)
    assert a4.hw_format == 5 and b4.hw_format == 5 and a4.codes.numel() == M * K // 2 and b4.codes.numel() == N * K // 2
    a8, b8 = G.quantize_pack(x, OCP_MXFP4_E2M1), G.quantize_pack(w, OCP_MXFP4_E2M1, G.OPERAND_B)
    y32 = dequant(x, OCP_MXFP4_E2M1) @ dequant(w, OCP_MXFP4_E2M1).t()
    bias = torch.randn(N, device=DEV).to(torch.bfloat16)
    for dt in (torch.float32, torch.bfloat16):
        y4 = G.mx_gemm(a4, b4, dt)
        y8 = G.mx_gemm(a8, b8, dt)
        G.check_status(DEV)
        assert within_tolerance(y4, y32), f"max err {(y4.float() - y32).abs().max().item()}"
        # same exact products; only the order of the fp32 additions inside an instruction may differ
        assert within_tolerance(y4, y8.float())
    yb = G.mx_gemm(a4, b4, torch.bfloat16, bias)
    G.check_status(DEV)
    assert within_tolerance(yb, y32 + bias.float())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("rows,K", [(512, 1024), (300, 256), (1, 512), (2050, 4096)])
def test_one_pass_nibble_pack_equals_two_step(lib, dtype, rows, K):
    """The one-kernel MXFP4 activation pack (packed nibbles + scale chunks) writes the bytes of extract followed by
    the native pack."""
    torch.manual_seed(rows + K)
    for scale in (1.0, 300.0):
        x = (torch.randn(rows, K, device=DEV) * scale).to(dtype)
        x[0, :32] = 0
        if rows > 2:
            x[1, 5] = float("inf")
            x[2, 40] = float("nan")
        one = G.quantize_pack_fused(x, OCP_MXFP4_E2M1)
        two = G.quantize_pack(x, OCP_MXFP4_E2M1, G.OPERAND_A, native=True)
        assert one.hw_format == 5 and two.hw_format == 5
        finite_rows = torch.isfinite(x.float()).reshape(rows, K // 32, 32).all(dim=2).repeat_interleave(16, dim=1)
        assert torch.equal(one.codes[finite_rows], two.codes[finite_rows]), "codes differ"
        assert torch.equal(one.sf, two.sf), "scale chunks differ"


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("b_meta", [MXFP8_E4M3_fn, OCP_MXFP6_E3M2, OCP_MXFP4_E2M1], ids=lambda m: m.tag)
def test_quantised_bias_is_decoded_in_the_epilogue(lib, dtype, b_meta):
    """Layer type XqWqBq called with a plain bias and bias codes (the case in which the reference uses the codes,
    src/mase_triton/mxfp/functional/linear.py:52-57): the fused backend hands the codes to the GEMM, whose epilogue decodes
    them; the result is the one obtained by dequantising the bias first, bit for bit."""
    from mase_triton_b200.mxfp.functional.cast import extract_mxfp_components, compose_mxfp_tensor

    torch.manual_seed(7)
    M, N, K = 300, 992, 256
    x = torch.randn(M, K, device=DEV).to(dtype)
    w = (0.05 * torch.randn(N, K, device=DEV)).to(dtype)
    bias = (3.0 * torch.randn(N, device=DEV)).to(dtype)
    w_scales, w_elements, w_tm = extract_mxfp_components(w, -1, OCP_MXFP6_E3M2)
    b_scales, b_elements, b_tm = extract_mxfp_components(bias, -1, b_meta)
    y = MX.mxfp_linear(x, MXFP8_E4M3_fn, None, w_scales, w_elements, w_tm, bias, b_scales, b_elements, b_tm, "XqWqBq", "fused")
    G.check_status(DEV)
    bias_dq = compose_mxfp_tensor(b_scales, b_elements, b_tm)
    want = MX.mxfp_linear(x, MXFP8_E4M3_fn, None, w_scales, w_elements, w_tm, bias_dq, None, None, None, "XqWqB", "fused")
    G.check_status(DEV)
    assert torch.equal(y, want)
    sep = MX.mxfp_linear(x, MXFP8_E4M3_fn, None, w_scales, w_elements, w_tm, bias, b_scales, b_elements, b_tm, "XqWqBq", "separate")
    assert within_tolerance(y, sep.float())
    # the GEMM entry by itself
    a = G.quantize_pack(x, MXFP8_E4M3_fn)
    wq = G.pack_operand(w_scales, w_elements, N, K, OCP_MXFP6_E3M2, G.OPERAND_B)
    assert torch.equal(G.mx_gemm(a, wq, dtype, bias_q=(b_scales, b_elements, b_meta)), G.mx_gemm(a, wq, dtype, bias=bias_dq))
