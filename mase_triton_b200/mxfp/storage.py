"""Compact, serialisable form of a quantised ``MXFPLinearPTQ``.

The reference stores one element code per byte and keeps the tensor metas (shape, block dim, format)
outside ``state_dict``, so a layer can only be restored through ``MXFPLinearPTQ.from_quantized`` with
metas carried along by hand (``src/mase_triton/mxfp/layers.py:175-211``).  ``export_packed`` writes
everything needed into one plain dict of tensors and Python scalars (``torch.save``-able): the element
codes bit-packed to their true width (4 bits for MXFP4, 6 for MXFP6, 8 for MXFP8), the E8M0 scales, the
bias and the metas.  ``import_packed`` rebuilds the layer on any CUDA device; the codes and scales it
yields are byte-identical to the exported layer's.  Packing and unpacking run on the GPU
(``csrc/mxq_bitpack.cu``).
"""

from __future__ import annotations

import torch
from torch import Tensor

from .. import _lib
from .meta import MXFPMeta, MXFPTensorMeta

FORMAT_VERSION = 1


def element_bits(meta: MXFPMeta) -> int:
    """Significant bits of one element code: sign + exponent + fraction."""
    return 1 + meta.element_exp_bits + meta.element_frac_bits


def pack_codes(elements: Tensor, bits: int) -> Tensor:
    """uint8 codes (one per byte, CUDA) -> dense little-endian bit stream of ``bits`` bits per code."""
    _lib.require_cuda(elements, "pack_codes")
    assert elements.dtype == torch.uint8 and bits in (4, 6, 8)
    flat = elements.contiguous().reshape(-1)
    n = flat.numel()
    assert n % 16 == 0, "the number of codes must be a multiple of 16"
    L = _lib.load()
    out = torch.empty((L.mxq_packed_bytes(n, bits),), dtype=torch.uint8, device=flat.device)
    with torch.cuda.device(flat.device):
        rc = L.mxq_pack_codes(flat.data_ptr(), out.data_ptr(), n, bits, _lib.stream_ptr(flat.device))
    _lib.check(rc, "mxq_pack_codes")
    return out


def unpack_codes(packed: Tensor, n: int, bits: int) -> Tensor:
    """Inverse of :func:`pack_codes`: ``n`` uint8 codes."""
    _lib.require_cuda(packed, "unpack_codes")
    assert packed.dtype == torch.uint8 and bits in (4, 6, 8) and n % 16 == 0
    packed = packed.contiguous()
    L = _lib.load()
    assert packed.numel() == L.mxq_packed_bytes(n, bits), "packed tensor has the wrong size"
    out = torch.empty((n,), dtype=torch.uint8, device=packed.device)
    with torch.cuda.device(packed.device):
        rc = L.mxq_unpack_codes(packed.data_ptr(), out.data_ptr(), n, bits, _lib.stream_ptr(packed.device))
    _lib.check(rc, "mxq_unpack_codes")
    return out


def _meta_dict(m: MXFPMeta) -> dict:
    return {"block_size": m.block_size, "scale_exp_bits": m.scale_exp_bits, "element_exp_bits": m.element_exp_bits,
            "element_frac_bits": m.element_frac_bits, "element_is_finite": m.element_is_finite, "round_mode": m.round_mode, "tag": m.tag}


def _tensor_record(scales: Tensor, elements: Tensor, tm: MXFPTensorMeta) -> dict:
    bits = element_bits(tm.meta)
    return {"packed": pack_codes(elements, bits).cpu(), "scales": scales.detach().reshape(-1).cpu(), "bits": bits, "numel": elements.numel(),
            "shape": tuple(tm.shape), "dtype": tm.dtype, "block_dim": tm.block_dim, "meta": _meta_dict(tm.meta)}


def _restore_tensor(rec: dict, device) -> tuple[Tensor, Tensor, MXFPTensorMeta]:
    meta = MXFPMeta(**rec["meta"])
    elements = unpack_codes(rec["packed"].to(device), rec["numel"], rec["bits"]).reshape(-1, meta.block_size)
    scales = rec["scales"].to(device).reshape(-1, 1)
    tm = MXFPTensorMeta(device=device, dtype=rec["dtype"], shape=rec["shape"], block_dim=rec["block_dim"], meta=meta)
    return scales, elements, tm


def export_packed(layer) -> dict:
    """Everything needed to rebuild ``layer`` (an ``MXFPLinearPTQ`` with a quantised weight on a CUDA device)."""
    assert layer.w_scales is not None, "export_packed needs a layer with a quantised weight"
    rec = {"format_version": FORMAT_VERSION, "layer_type": layer.layer_type, "backend": layer.backend,
           "x_meta": None if layer.x_mxfp_meta is None else _meta_dict(layer.x_mxfp_meta),
           "weight": _tensor_record(layer.w_scales.data, layer.w_elements.data, layer.w_tensor_meta),
           "bias": None if layer.bias is None else layer.bias.detach().cpu(), "bias_q": None}
    if layer.b_scales is not None:
        b = layer.b_elements.data
        pad = (-b.numel()) % 16                      # a bias may hold any multiple of the block size
        rec["bias_q"] = _tensor_record(layer.b_scales.data, torch.nn.functional.pad(b.reshape(-1), (0, pad)), layer.b_tensor_meta)
        rec["bias_q"]["numel_unpadded"] = b.numel()
    return rec


def import_packed(rec: dict, device="cuda", backend: str | None = None):
    """Rebuild the layer exported by :func:`export_packed` on ``device``."""
    from .layers import MXFPLinearPTQ

    assert rec.get("format_version") == FORMAT_VERSION, "unknown packed-layer format"
    device = torch.device(device)
    w_scales, w_elements, w_tm = _restore_tensor(rec["weight"], device)
    b_scales = b_elements = b_tm = None
    if rec["bias_q"] is not None:
        b_scales, b_elements, b_tm = _restore_tensor(rec["bias_q"], device)
        n = rec["bias_q"]["numel_unpadded"]
        b_elements = b_elements.reshape(-1)[:n].reshape(-1, b_tm.meta.block_size).contiguous()
    bias = None if rec["bias"] is None else rec["bias"].to(device)
    x_meta = None if rec["x_meta"] is None else MXFPMeta(**rec["x_meta"])
    return MXFPLinearPTQ.from_quantized(w_scales, w_elements, w_tm, bias, b_scales, b_elements, b_tm, x_meta, rec["layer_type"],
                                        backend or rec["backend"])
