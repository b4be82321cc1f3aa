"""Host side of the block-scaled tensor-core GEMM (``csrc/mxq_gemm.cu``).

``PackedOperand`` is an MXFP tensor re-encoded for the tensor cores: one hardware E4M3/E5M2 byte
per element plus E8M0 scales in the chunked order the kernel's ``tcgen05.cp`` expects.  Weights
are packed once and cached; activations are quantised and packed per call.  The reference has no
counterpart: its ``backend="fused"`` raises ``NotImplementedError``
(``src/mase_triton/mxfp/functional/linear.py:62-63``).
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch
from torch import Tensor

from .. import _lib
from . import kernels
from .meta import MXFPMeta

_STATUS: dict[torch.device, Tensor] = {}
_STATUS_TEXT = {1: "TMA producer wait ran out", 2: "MMA issuer wait ran out", 3: "epilogue wait ran out",
                4: "copy-out (gather) wait ran out", 5: "operand dequantiser wait ran out"}


@dataclass
class PackedOperand:
    codes: Tensor        # uint8 [rows, K] hardware element codes ([rows, K * bits / 8] for the 6- / 4-bit formats)
    sf: Tensor           # uint8, hardware scale-factor chunks
    hw_format: int       # 0 = E4M3, 1 = E5M2; dense bit streams: 3 = E2M3, 4 = E3M2 (right operand), 5 = E2M1 (either side)
    rows: int
    K: int
    operand: int         # 0: packed as the left operand (A), 1: as the right operand (B)
    tile_rows: int = 0   # right operand: CTA tile width its scale factors are tiled for (0 = default 224)


def supported(meta: MXFPMeta | None) -> bool:
    """Formats the tensor-core path takes: 32-element blocks, is_finite element formats (any rounding
    mode: the mode only matters where an activation is quantised, see :func:`pack_activation`)."""
    return meta is not None and meta.block_size == 32 and meta.element_is_finite and meta.scale_exp_bits == 8


def one_pass_ok(meta: MXFPMeta) -> bool:
    """Activation formats the one-kernel quantise + pack routes cover: MXFP8 elements, round to nearest."""
    return supported(meta) and meta.element_exp_bits >= 4 and meta.round_mode == "rn"


def status_word(device: torch.device) -> Tensor:
    """The int32 word a GEMM kernel on ``device`` writes a non-zero code into when one of its bounded
    waits runs out.  It lives in pinned host memory (which the GPU addresses directly), so the host can
    look at it without synchronising: every GEMM entry of this module does so before it launches and
    raises :class:`MXQError` for a failure left by an earlier launch."""
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    if device not in _STATUS:
        _STATUS[device] = torch.zeros(1, dtype=torch.int32).pin_memory()
    return _STATUS[device]


def _raise_if_failed(device: torch.device) -> None:
    """Non-blocking look at the status word: reports (and clears) what a finished launch left there."""
    word = status_word(device)
    code = int(word[0])
    if code != 0:
        word.zero_()
        raise _lib.MXQError(f"an earlier tensor-core GEMM on {device} gave up: {_STATUS_TEXT.get(code, code)}; "
                            "its output is undefined")


def check_status(device: torch.device) -> None:
    """Wait for the device, then raise if any GEMM launched so far reported a wait that ran out."""
    torch.cuda.synchronize(device)
    _raise_if_failed(device)


OPERAND_A, OPERAND_B = 0, 1


def native_ok(exp_bits: int, frac_bits: int, K: int, operand: int) -> bool:
    """Whether the tensor cores can read the codes in their own 6- / 4-bit width: a right operand in an FP6 / FP4
    element format (whole 128-code K steps), or a left operand in E2M1 for the 4-bit x 4-bit GEMM (whole 256-code
    stages; the right operand must then be native E2M1 too)."""
    if operand == OPERAND_B:
        return K % 128 == 0 and (exp_bits, frac_bits) in ((2, 3), (3, 2), (2, 1))
    return K % 256 == 0 and (exp_bits, frac_bits) == (2, 1)


NATIVE_SUBBYTE_DEFAULT = False


def is_e2m1(meta: MXFPMeta | None) -> bool:
    return meta is not None and (meta.element_exp_bits, meta.element_frac_bits) == (2, 1)


def fp4_pair(x_meta: MXFPMeta | None, w_meta: MXFPMeta | None, K: int) -> bool:
    """MXFP4 activation and MXFP4 weight with whole 256-element stages: both operands can stay packed nibbles and
    the GEMM runs on the 4-bit x 4-bit tensor-core kind (twice the arithmetic rate of the 8-bit kinds)."""
    return is_e2m1(x_meta) and is_e2m1(w_meta) and supported(x_meta) and supported(w_meta) and K % 256 == 0


def pack_codes(scales: Tensor | None, elements: Tensor, rows: int, K: int, exp_bits: int, frac_bits: int, operand: int,
               tile_rows: int | None = None, native: bool | None = None) -> PackedOperand:
    """Element codes (one per byte, sign at bit ``exp_bits + frac_bits``) of a ``[rows, K]`` tensor and the
    E8M0 scales of its 32-element blocks along K (``None``: every scale is 2^0, i.e. per-tensor minifloat
    codes) -> ``PackedOperand`` for the left (``OPERAND_A``) or right (``OPERAND_B``) side of the GEMM.
    ``tile_rows`` (right operand only) is the CTA tile width; by default the one with the least padded
    work for ``rows`` output features.  ``native`` keeps FP6 / FP4 codes of a right operand at their own width
    (a dense bit stream, three quarters / half of the bytes) instead of widening them to E4M3 bytes."""
    _lib.require_cuda(elements, "pack_operand")
    assert elements.dtype == torch.uint8 and K % 32 == 0 and elements.numel() == rows * K
    assert scales is None or (scales.dtype == torch.uint8 and scales.numel() == rows * K // 32)
    elements = elements.contiguous()
    scales = None if scales is None else scales.contiguous()
    L = _lib.load()
    dev = elements.device
    if operand == OPERAND_A:
        tile_rows = 0
    elif tile_rows is None:
        tile_rows = L.mxq_mx_best_tile_rows(rows)
    if native is None:
        native = NATIVE_SUBBYTE_DEFAULT
    native = native and native_ok(exp_bits, frac_bits, K, operand)
    sf = torch.empty((L.mxq_mx_sf_bytes(rows, K, operand, tile_rows),), dtype=torch.uint8, device=dev)
    fmt = ctypes.c_int(0)
    if native:
        bits = 1 + exp_bits + frac_bits
        codes = torch.empty((rows, K * bits // 8), dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            rc = L.mxq_mx_pack_operand_native(None if scales is None else scales.data_ptr(), elements.data_ptr(), rows, K, exp_bits,
                                              frac_bits, operand, tile_rows, codes.data_ptr(), sf.data_ptr(), ctypes.addressof(fmt),
                                              _lib.stream_ptr(dev))
        _lib.check(rc, "mxq_mx_pack_operand_native")
        return PackedOperand(codes, sf, fmt.value, rows, K, operand, tile_rows)
    codes = torch.empty((rows, K), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        rc = L.mxq_mx_pack_operand(None if scales is None else scales.data_ptr(), elements.data_ptr(), rows, K, exp_bits, frac_bits,
                                   operand, tile_rows, codes.data_ptr(), sf.data_ptr(), ctypes.addressof(fmt), _lib.stream_ptr(dev))
    _lib.check(rc, "mxq_mx_pack_operand")
    return PackedOperand(codes, sf, fmt.value, rows, K, operand, tile_rows)


def pack_operand(scales: Tensor, elements: Tensor, rows: int, K: int, meta: MXFPMeta, operand: int,
                 tile_rows: int | None = None, native: bool | None = None) -> PackedOperand:
    """Reference ``(scales, elements)`` of a ``[rows, K]`` tensor blocked along K -> ``PackedOperand``
    laid out for the left (``OPERAND_A``) or right (``OPERAND_B``) side of the GEMM."""
    assert supported(meta)
    return pack_codes(scales, elements, rows, K, meta.element_exp_bits, meta.element_frac_bits, operand, tile_rows, native)


def quantize_pack(x: Tensor, meta: MXFPMeta, operand: int = OPERAND_A, tile_rows: int | None = None,
                  native: bool | None = None) -> PackedOperand:
    """Quantise a ``[..., K]`` tensor along its last dim and pack it."""
    K = x.shape[-1]
    rows = x.numel() // K
    scales, elements = kernels.extract_mxfp_components(x.reshape(-1), meta)
    return pack_operand(scales, elements, rows, K, meta, operand, tile_rows, native)


def quantize_pack_fused(x: Tensor, meta: MXFPMeta) -> PackedOperand:
    """One-kernel version of :func:`quantize_pack` for a left operand with MXFP8 elements (round to nearest), or with
    MXFP4 elements as packed nibbles (the left operand of the 4-bit x 4-bit GEMM)."""
    _lib.require_cuda(x, "quantize_pack_fused")
    nibbles = is_e2m1(meta) and supported(meta) and meta.round_mode == "rn"
    assert one_pass_ok(meta) or nibbles, "one-pass quantise + pack covers MXFP8 and MXFP4 elements with round_mode 'rn' only"
    K = x.shape[-1]
    rows = x.numel() // K
    x2 = x.reshape(rows, K).contiguous()
    L = _lib.load()
    codes = torch.empty((rows, K // 2 if nibbles else K), dtype=torch.uint8, device=x.device)
    sf = torch.empty((L.mxq_mx_sf_bytes(rows, K, OPERAND_A, 0),), dtype=torch.uint8, device=x.device)
    fmt = ctypes.c_int(0)
    with torch.cuda.device(x.device):
        rc = L.mxq_mx_quantize_pack(x2.data_ptr(), _lib.DTYPE_ID[x2.dtype], rows, K, meta.element_exp_bits, meta.element_frac_bits,
                                    codes.data_ptr(), sf.data_ptr(), ctypes.addressof(fmt), _lib.stream_ptr(x.device))
    _lib.check(rc, "mxq_mx_quantize_pack")
    return PackedOperand(codes, sf, fmt.value, rows, K, OPERAND_A)


def pack_activation(x: Tensor, meta: MXFPMeta, nibbles: bool = False) -> PackedOperand:
    """Quantise a ``[..., K]`` activation along its last dim, as ``meta`` says (element format and rounding
    mode), into the left operand of the GEMM: one kernel for MXFP8 / round to nearest, extract + pack
    otherwise.  ``nibbles``: keep an MXFP4 activation as packed 4-bit codes for a weight packed the same way.
    The result can be fed to several layers that share the activation (q / k / v, gate / up)
    through ``MXFPLinearPTQ.forward_packed`` so that it is quantised once."""
    if nibbles:
        return quantize_pack_fused(x, meta) if meta.round_mode == "rn" and x.dtype in _lib.DTYPE_ID else quantize_pack(x, meta, OPERAND_A, native=True)
    return quantize_pack_fused(x, meta) if one_pass_ok(meta) else quantize_pack(x, meta)


def minifloat_quantize_pack(x: Tensor, exp_bits: int, frac_bits: int, round_mode: str) -> PackedOperand | None:
    """Per-tensor minifloat FP8 quantisation of a ``[..., K]`` activation in one kernel, as a left operand
    with unit scales.  ``None`` when the library does not cover the format (the caller then extracts,
    narrows and packs)."""
    _lib.require_cuda(x, "minifloat_quantize_pack")
    K = x.shape[-1]
    rows = x.numel() // K
    x2 = x.reshape(rows, K).contiguous()
    L = _lib.load()
    codes = torch.empty((rows, K), dtype=torch.uint8, device=x.device)
    sf = torch.empty((L.mxq_mx_sf_bytes(rows, K, OPERAND_A, 0),), dtype=torch.uint8, device=x.device)
    fmt = ctypes.c_int(0)
    with torch.cuda.device(x.device):
        rc = L.mxq_minifloat_quantize_pack(x2.data_ptr(), _lib.DTYPE_ID[x2.dtype], rows, K, exp_bits, frac_bits, _lib.ROUND_ID[round_mode],
                                           codes.data_ptr(), sf.data_ptr(), ctypes.addressof(fmt), _lib.stream_ptr(x.device))
    if rc == -3:
        return None
    _lib.check(rc, "mxq_minifloat_quantize_pack")
    return PackedOperand(codes, sf, fmt.value, rows, K, OPERAND_A)


_TUNED_TILE_ROWS: dict[tuple, int] = {}
TILE_ROW_CANDIDATES = (224, 208, 192, 176, 160)


def choose_tile_rows(w_scales: Tensor, w_elements: Tensor, shape: tuple[int, int], meta: MXFPMeta, rows: int | None) -> int:
    """CTA tile width for a weight of ``shape`` multiplied with an activation of ``rows`` rows.

    By default the width with the least padded work (``mxq_mx_best_tile_rows``).  With
    ``KernelManager.enable_autotune()`` (the switch that turns Triton's autotuner on in the reference,
    ``src/mase_triton/manager.py:7-32``) and a known ``rows``, the candidates whose padded work is within 8 % of the
    least are each packed and timed on the GPU once per (device, rows rounded up to 256, shape) and the fastest is
    kept; nothing is measured while a CUDA graph is being captured."""
    from ..manager import KernelManager

    n, k = shape
    best = _lib.load().mxq_mx_best_tile_rows(n)
    dev = w_elements.device
    if not KernelManager.autotune_is_enabled() or not rows or torch.cuda.is_current_stream_capturing():
        return best
    m = min(-(-rows // 256) * 256, 16384)
    key = (dev, m, n, k, meta)
    if key in _TUNED_TILE_ROWS:
        return _TUNED_TILE_ROWS[key]
    padded = {t: -(-n // t) * t for t in TILE_ROW_CANDIDATES}
    least = min(padded.values())
    candidates = [t for t in TILE_ROW_CANDIDATES if padded[t] <= 1.08 * least]
    if best not in candidates:
        candidates.append(best)
    a_codes = torch.randint(0, 0x78, (m, k), dtype=torch.uint8, device=dev)             # finite E4M3 codes, unit scales
    a = pack_codes(None, a_codes, m, k, 4, 3, OPERAND_A)
    out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    timings = {}
    for t in candidates:
        b = pack_operand(w_scales, w_elements, n, k, meta, OPERAND_B, tile_rows=t)
        for _ in range(2):
            mx_gemm(a, b, torch.bfloat16, out=out)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            mx_gemm(a, b, torch.bfloat16, out=out)
        e1.record()
        torch.cuda.synchronize(dev)
        timings[t] = e0.elapsed_time(e1) / 5
    choice = min(timings, key=timings.get)
    _TUNED_TILE_ROWS[key] = choice
    KernelManager.record_choice(("mx_gemm tile_rows", m, n, k), choice, timings)
    return choice


def packed_weight(w_scales: Tensor, w_elements: Tensor, shape: tuple[int, int], meta: MXFPMeta, rows: int | None = None,
                  nibbles: bool = False) -> PackedOperand:
    """Packed form of a quantised weight.  The result is kept on the ``w_elements`` tensor object itself
    (so it dies with it and can never be confused with another tensor that re-uses the same address)
    and is rebuilt when either code tensor was modified in place or replaced, or when the tile width chosen
    for ``rows`` activation rows (:func:`choose_tile_rows`) differs from the one it was packed for."""
    tile = choose_tile_rows(w_scales, w_elements, tuple(shape), meta, rows)
    tag = (w_elements._version, w_scales.data_ptr(), w_scales._version, tuple(shape), meta, tile, nibbles)
    cached = getattr(w_elements, "_mxq_packed", None)
    if cached is None or cached[0] != tag:
        cached = (tag, pack_operand(w_scales, w_elements, shape[0], shape[1], meta, OPERAND_B, tile_rows=tile, native=nibbles))
        w_elements._mxq_packed = cached
    return cached[1]


def bias_codes_ok(b_scales: Tensor | None, b_elements: Tensor | None, b_meta: MXFPMeta | None, n: int, bias_dtype, out_dtype) -> bool:
    """Whether the GEMM's epilogue can decode this quantised bias itself: 32-element blocks, an is_finite element
    format, ``n`` a multiple of 32, and a bias that dequantises to the output dtype (so the rounding is the compose
    kernel's)."""
    return (b_scales is not None and b_elements is not None and supported(b_meta) and n % 32 == 0 and b_elements.numel() == n
            and bias_dtype == out_dtype)


def mx_gemm(a: PackedOperand, b: PackedOperand, out_dtype: torch.dtype, bias: Tensor | None = None,
            out: Tensor | None = None, bias_q: tuple[Tensor, Tensor, MXFPMeta] | None = None) -> Tensor:
    """``a [M,K] @ b[N,K]^T (+ bias)`` on the tensor cores; returns ``[M, N]`` of ``out_dtype``.
    ``bias_q = (scales, elements, meta)``: an MXFP-quantised bias decoded by the epilogue (instead of ``bias``)."""
    assert a.K == b.K and out_dtype in _lib.DTYPE_ID and a.operand == OPERAND_A and b.operand == OPERAND_B
    assert a.hw_format <= 1 or (a.hw_format == 5 and b.hw_format == 5), "a packed 4-bit left operand needs a packed 4-bit right one"
    dev = a.codes.device
    _raise_if_failed(dev)
    if out is None:
        out = torch.empty((a.rows, b.rows), dtype=out_dtype, device=dev)
    if bias_q is not None:
        assert bias is None, "pass the bias either dense or as codes"
        q_scales, q_elements, q_meta = bias_q
        q_scales, q_elements = q_scales.contiguous(), q_elements.contiguous()
        assert q_elements.numel() == b.rows and q_scales.numel() == b.rows // 32 and supported(q_meta)
        with torch.cuda.device(dev):
            rc = _lib.load().mxq_mx_gemm_qbias(a.codes.data_ptr(), a.sf.data_ptr(), a.hw_format, b.codes.data_ptr(), b.sf.data_ptr(),
                                               b.hw_format, b.tile_rows, out.data_ptr(), _lib.DTYPE_ID[out_dtype],
                                               q_scales.data_ptr(), q_elements.data_ptr(), q_meta.element_exp_bits, q_meta.element_frac_bits,
                                               a.rows, b.rows, a.K, status_word(dev).data_ptr(), _lib.stream_ptr(dev))
        _lib.check(rc, "mxq_mx_gemm_qbias")
        return out
    if bias is not None:
        bias = bias.to(out_dtype).contiguous()
        assert bias.numel() == b.rows
    with torch.cuda.device(dev):
        rc = _lib.load().mxq_mx_gemm(a.codes.data_ptr(), a.sf.data_ptr(), a.hw_format, b.codes.data_ptr(), b.sf.data_ptr(),
                                     b.hw_format, b.tile_rows, out.data_ptr(), _lib.DTYPE_ID[out_dtype],
                                     None if bias is None else bias.data_ptr(), a.rows, b.rows, a.K,
                                     status_word(dev).data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc, "mxq_mx_gemm")
    return out


def mx_gemm_gather(a: PackedOperand, b: PackedOperand, out_ptrs: list[int], self_index: int, ld: int, col_offset: int,
                   out_dtype: torch.dtype, bias: Tensor | None = None) -> None:
    """``a [M,K] @ b[N,K]^T (+ bias)`` written by the GEMM kernel itself into EVERY buffer of
    ``out_ptrs`` (device addresses of row-major ``[>=M, ld]`` matrices of ``out_dtype``:
    ``out_ptrs[self_index]`` is this GPU's output, the others are the peers' outputs mapped into this
    process) at columns ``[col_offset, col_offset + N)``.  This is the all-gather of a column-parallel
    linear done by the producing kernel with plain stores over NVLink; the caller orders it against the
    consumers on the other ranks."""
    assert a.K == b.K and out_dtype in _lib.DTYPE_ID and a.operand == OPERAND_A and b.operand == OPERAND_B
    dev = a.codes.device
    _raise_if_failed(dev)
    if bias is not None:
        bias = bias.to(out_dtype).contiguous()
        assert bias.numel() == b.rows
    ptrs = (ctypes.c_void_p * len(out_ptrs))(*out_ptrs)
    with torch.cuda.device(dev):
        rc = _lib.load().mxq_mx_gemm_gather(a.codes.data_ptr(), a.sf.data_ptr(), a.hw_format, b.codes.data_ptr(), b.sf.data_ptr(),
                                            b.hw_format, b.tile_rows, ctypes.addressof(ptrs), len(out_ptrs), self_index, ld, col_offset,
                                            _lib.DTYPE_ID[out_dtype], None if bias is None else bias.data_ptr(),
                                            a.rows, b.rows, a.K, status_word(dev).data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc, "mxq_mx_gemm_gather")


_SCRATCH: dict[tuple[torch.device, int], Tensor] = {}


def _scratch(device: torch.device, nbytes: int) -> Tensor:
    """Scratch buffer for the quantised activation, one per (device, stream) so that layers running on
    different streams never share it; grown on demand and re-used.  A replaced buffer goes back to
    PyTorch's caching allocator, which keeps it tied to the stream it was allocated on."""
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    buf = _SCRATCH.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty((nbytes,), dtype=torch.uint8, device=device)
        _SCRATCH[key] = buf
    return buf


def mx_linear(x: Tensor, x_meta: MXFPMeta, w: PackedOperand, bias: Tensor | None = None, out: Tensor | None = None,
              bias_q: tuple[Tensor, Tensor, MXFPMeta] | None = None) -> Tensor:
    """``quantise(x) @ w^T (+ bias)``.  Round-to-nearest activations go through the single C entry point
    ``mxq_mx_linear`` (quantisation, packing and the tensor-core GEMM enqueued back to back on the
    current stream); the other rounding modes are quantised by the extract kernel, which implements
    them, packed, and multiplied by the same GEMM.  An MXFP4 activation against a weight packed as 4-bit codes is
    packed as 4-bit codes too and multiplied on the 4-bit x 4-bit tensor-core kind."""
    _lib.require_cuda(x, "mx_linear")
    assert supported(x_meta) and w.operand == OPERAND_B and x.shape[-1] == w.K
    if x.dtype not in _lib.DTYPE_ID:
        x = x.float()
    x2 = x.reshape(-1, w.K).contiguous()
    M, dev = x2.shape[0], x2.device
    if bias_q is not None:
        # a quantised bias: the activation is packed by its own kernel, the GEMM's epilogue decodes the bias codes
        nib = w.hw_format == 5 and is_e2m1(x_meta) and w.K % 256 == 0
        y = mx_gemm(pack_activation(x2, x_meta, nibbles=nib), w, x2.dtype, out=out, bias_q=bias_q)
        return y.reshape(*x.shape[:-1], w.rows)
    if w.hw_format == 5 and is_e2m1(x_meta) and w.K % 256 == 0 and x_meta.round_mode != "rn":
        # MXFP4 x MXFP4 with the weight kept as packed nibbles: the activation is packed the same way (kind::mxf4);
        # round to nearest goes through the single C entry point below, which does the same
        y = mx_gemm(pack_activation(x2, x_meta, nibbles=True), w, x2.dtype, bias=bias, out=out)
        return y.reshape(*x.shape[:-1], w.rows)
    if x_meta.round_mode != "rn":
        y = mx_gemm(quantize_pack(x2, x_meta), w, x2.dtype, bias=bias, out=out)
        return y.reshape(*x.shape[:-1], w.rows)
    _raise_if_failed(dev)
    L = _lib.load()
    if out is None:
        out = torch.empty((M, w.rows), dtype=x2.dtype, device=dev)
    if bias is not None:
        bias = bias.to(out.dtype).contiguous()
    nbytes = L.mxq_mx_linear_scratch_bytes(M, w.K)
    scratch = _scratch(dev, nbytes)
    with torch.cuda.device(dev):
        rc = L.mxq_mx_linear(x2.data_ptr(), _lib.DTYPE_ID[x2.dtype], M, w.K, x_meta.element_exp_bits, x_meta.element_frac_bits,
                             w.codes.data_ptr(), w.sf.data_ptr(), w.hw_format, w.tile_rows, w.rows, out.data_ptr(), _lib.DTYPE_ID[out.dtype],
                             None if bias is None else bias.data_ptr(), scratch.data_ptr(), scratch.numel(),
                             status_word(dev).data_ptr(), _lib.stream_ptr(dev))
    _lib.check(rc, "mxq_mx_linear")
    return out.reshape(*x.shape[:-1], w.rows)
