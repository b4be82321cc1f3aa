"""``MXFPLinearPTQ`` (reference: ``src/mase_triton/mxfp/layers.py:11-211``).

A post-training-quantised linear layer.  With ``Wq`` the weight lives as uint8 Parameters
``w_scales`` ``[out*in/B, 1]`` and ``w_elements`` ``[out*in/B, B]`` (blocks along ``in_features``) plus
the plain attribute ``w_tensor_meta``; with ``Bq`` the bias likewise (blocks along dim 0).
Parameter names, constructor arguments and class methods match the reference.
"""

from __future__ import annotations

from typing import Literal

import torch
from torch import Tensor, nn

from .._ptq_base import PTQLinearBase
from . import functional as MXFP_F
from .meta import MXFPMeta, MXFPTensorMeta

LayerType = Literal["XWB", "XWBq", "XWqB", "XWqBq", "XqWB", "XqWBq", "XqWqB", "XqWqBq"]


def _all_given(*items) -> bool:
    return all(i is not None for i in items)


class MXFPLinearPTQ(PTQLinearBase):
    _code_tensors = ("w_scales", "w_elements", "b_scales", "b_elements")
    _meta_follows = {"w_tensor_meta": "w_scales", "b_tensor_meta": "b_scales"}

    def __init__(
        self,
        weight: Tensor,
        bias: Tensor | None,
        x_mxfp_meta: MXFPMeta | None,
        w_mxfp_meta: MXFPMeta | None,
        b_mxfp_meta: MXFPMeta | None,
        layer_type: LayerType,
        backend: Literal["separate", "fused"] = "fused",
        dtype: torch.dtype | None = None,
        device: torch.device | None = None,
        w_scales: Tensor | None = None,
        w_elements: Tensor | None = None,
        w_tensor_meta: MXFPTensorMeta | None = None,
        b_scales: Tensor | None = None,
        b_elements: Tensor | None = None,
        b_tensor_meta: MXFPTensorMeta | None = None,
    ):
        super().__init__()
        assert weight is None or weight.ndim == 2
        assert bias is None or bias.ndim == 1
        assert (weight is not None) ^ _all_given(w_scales, w_elements, w_tensor_meta)
        if bias is not None and _all_given(b_scales, b_elements, b_tensor_meta):
            raise ValueError("Either bias or b_scales, b_elements, b_tensor_meta must be None, not both.")
        out_features, in_features = w_tensor_meta.shape if weight is None else weight.shape
        assert bias is None or bias.shape[0] == out_features

        self.in_features, self.out_features = in_features, out_features
        self.x_mxfp_meta, self.w_mxfp_meta, self.b_mxfp_meta = x_mxfp_meta, w_mxfp_meta, b_mxfp_meta
        self.layer_type = layer_type
        self.backend = backend
        self.dtype, self.device = dtype, device

        self.weight = self.w_scales = self.w_elements = self.w_tensor_meta = None
        self.bias = self.b_scales = self.b_elements = self.b_tensor_meta = None
        # tensor-core form of the quantised weight (hardware codes + tiled scale factors), built on first use.
        # Non-persistent buffers: they follow .to() / .cuda() with the module and stay out of state_dict().
        self.register_buffer("_tc_codes", None, persistent=False)
        self.register_buffer("_tc_sf", None, persistent=False)
        self._tc_info = None          # (versions of the code tensors it was built from, hw_format, tile_rows)

        if "Wq" in layer_type:
            if w_scales is None:
                w_scales, w_elements, w_tensor_meta = MXFP_F.extract_mxfp_components(weight, block_dim=1, mxfp_meta=w_mxfp_meta)
            self.w_scales, self.w_elements = self._frozen(w_scales), self._frozen(w_elements)
            self.w_tensor_meta = w_tensor_meta
        else:
            assert weight is not None
            self.weight = self._frozen(weight.to(dtype=dtype, device=device))

        if "Bq" in layer_type:
            if bias is not None and b_scales is None:
                b_scales, b_elements, b_tensor_meta = MXFP_F.extract_mxfp_components(bias, block_dim=0, mxfp_meta=b_mxfp_meta)
            if b_scales is not None:
                self.b_scales, self.b_elements = self._frozen(b_scales), self._frozen(b_elements)
                self.b_tensor_meta = b_tensor_meta
        elif bias is not None:
            self.bias = self._frozen(bias.to(dtype=dtype, device=device))

    def tensor_core_weight(self, rows: int | None = None):
        """The quantised weight re-encoded for the block-scaled GEMM, kept on the module: rebuilt only when the
        code tensors were written (``load_state_dict``, in-place edits), moved - not rebuilt - by ``.to()``.
        ``rows`` (the height of the activation it will be multiplied with) only matters while
        ``KernelManager`` autotune is enabled: the tile width is then the one measured fastest for that height."""
        from . import gemm as _gemm

        versions = (self.w_elements._version, self.w_scales._version)
        tile = _gemm.choose_tile_rows(self.w_scales.data, self.w_elements.data, tuple(self.w_tensor_meta.shape), self.w_tensor_meta.meta, rows)
        stale = (self._tc_codes is None or self._tc_info is None or self._tc_info[0] != versions
                 or self._tc_codes.device != self.w_elements.device or self._tc_info[2] != tile)
        if stale:
            n, k = self.w_tensor_meta.shape
            # an MXFP4 layer (activation and weight) keeps its weight as packed 4-bit codes for the 4-bit x 4-bit GEMM
            nibbles = _gemm.fp4_pair(self.x_mxfp_meta, self.w_tensor_meta.meta, k)
            p = _gemm.pack_operand(self.w_scales.data, self.w_elements.data, n, k, self.w_tensor_meta.meta, _gemm.OPERAND_B, tile_rows=tile,
                                   native=nibbles)
            self._tc_codes, self._tc_sf = p.codes, p.sf
            self._tc_info = (versions, p.hw_format, p.tile_rows)
        n, k = self.w_tensor_meta.shape
        return _gemm.PackedOperand(self._tc_codes, self._tc_sf, self._tc_info[1], n, k, _gemm.OPERAND_B, self._tc_info[2])

    def export_packed(self) -> dict:
        """A ``torch.save``-able dict holding this layer with its element codes bit-packed to their true width
        (4 / 6 / 8 bits) and its tensor metas; see ``mase_triton_b200.mxfp.storage``."""
        from .storage import export_packed

        return export_packed(self)

    @classmethod
    def from_packed(cls, record: dict, device="cuda", backend: str | None = None):
        """Rebuild a layer from :meth:`export_packed` output on ``device``."""
        from .storage import import_packed

        return import_packed(record, device, backend)

    @torch.no_grad()
    def forward(self, input: Tensor) -> Tensor:
        if (self.backend == "fused" and "Xq" in self.layer_type and "Wq" in self.layer_type
                and MXFP_F.linear.block_scaled_ok(input, self.x_mxfp_meta, self.w_tensor_meta)):
            # both operands stay quantised: the module's own tensor-core form of the weight, no per-call packing.
            # A layer with a quantised bias holds no plain one and then adds none (the reference's rule).
            from . import gemm as _gemm

            return _gemm.mx_linear(input, self.x_mxfp_meta, self.tensor_core_weight(input.numel() // self.in_features), self.bias)
        return MXFP_F.mxfp_linear(
            x=input, x_meta=self.x_mxfp_meta,
            w=self.weight, w_scales=self.w_scales, w_elements=self.w_elements, w_tensor_meta=self.w_tensor_meta,
            b=self.bias, b_scales=self.b_scales, b_elements=self.b_elements, b_tensor_meta=self.b_tensor_meta,
            layer_type=self.layer_type, backend=self.backend,
        )

    def pack_input(self, input: Tensor):
        """Quantise ``input`` as this layer's ``forward`` would (``x_mxfp_meta``) into the tensor-core operand
        form.  Layers that read the same activation (q / k / v, gate / up) can share the result through
        :meth:`forward_packed`, so the activation is quantised once instead of once per layer."""
        from . import gemm as _gemm

        assert "Xq" in self.layer_type and "Wq" in self.layer_type and _gemm.supported(self.x_mxfp_meta), \
            "pack_input needs a layer with quantised activation and weight (32-element blocks)"
        return _gemm.pack_activation(input.reshape(-1, self.in_features), self.x_mxfp_meta,
                                     nibbles=_gemm.fp4_pair(self.x_mxfp_meta, self.w_tensor_meta.meta, self.in_features))

    @torch.no_grad()
    def forward_packed(self, packed, out_dtype: torch.dtype = torch.bfloat16, lead_shape: tuple[int, ...] | None = None) -> Tensor:
        """``forward`` on an activation already quantised by :meth:`pack_input` (of this or of another layer
        with the same ``x_mxfp_meta`` and ``in_features``); returns ``[rows, out_features]`` of ``out_dtype``,
        reshaped to ``lead_shape + (out_features,)`` when given."""
        from . import gemm as _gemm

        assert packed.K == self.in_features and self.w_scales is not None
        wq = self.tensor_core_weight(packed.rows)
        # a layer with a quantised bias holds no plain one, and forward() then adds none (the reference's rule)
        y = _gemm.mx_gemm(packed, wq, out_dtype, bias=self.bias)
        return y if lead_shape is None else y.reshape(*lead_shape, self.out_features)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, "
                f"layer_type={self.layer_type}, w_mxfp_meta={self.w_mxfp_meta}, x_mxfp_meta={self.x_mxfp_meta}, "
                f"b_mxfp_meta={self.b_mxfp_meta}")

    @classmethod
    def from_linear(cls, layer: nn.Linear, x_mxfp_meta: MXFPMeta | None, w_mxfp_meta: MXFPMeta | None,
                    b_mxfp_meta: MXFPMeta | None, layer_type: LayerType, backend: Literal["separate", "fused"]):
        """Quantise an existing ``nn.Linear`` (its tensors are cloned, the layer is left untouched)."""
        assert isinstance(layer, nn.Linear), "layer must be an instance of nn.Linear"
        with torch.no_grad():
            return cls(weight=layer.weight.clone(), bias=None if layer.bias is None else layer.bias.clone(),
                       x_mxfp_meta=x_mxfp_meta, w_mxfp_meta=w_mxfp_meta, b_mxfp_meta=b_mxfp_meta,
                       layer_type=layer_type, backend=backend)

    @classmethod
    def from_quantized(cls, w_scales: Tensor | None, w_elements: Tensor | None, w_tensor_meta: MXFPTensorMeta | None,
                       bias: Tensor | None, b_scales: Tensor | None, b_elements: Tensor | None,
                       b_tensor_meta: MXFPTensorMeta | None, x_mxfp_meta: MXFPMeta | None,
                       layer_type: Literal["XWqB", "XWqBq", "XqWqB", "XqWqBq"], backend: Literal["separate", "fused"]):
        """Rebuild a layer from stored codes (tensor metas are not part of ``state_dict``)."""
        assert _all_given(w_scales, w_elements, w_tensor_meta)
        return cls(weight=None, bias=bias, x_mxfp_meta=x_mxfp_meta, w_mxfp_meta=None, b_mxfp_meta=None,
                   layer_type=layer_type, backend=backend,
                   dtype=getattr(torch, w_tensor_meta.dtype), device=torch.device(w_tensor_meta.device),
                   w_scales=w_scales, w_elements=w_elements, w_tensor_meta=w_tensor_meta,
                   b_scales=b_scales, b_elements=b_elements, b_tensor_meta=b_tensor_meta)
