"""``MinifloatLinearPTQ`` (reference: ``src/mase_triton/minifloat/layers.py:11-188``).

A post-training-quantised linear layer: the weight is either a plain ``weight`` Parameter or
uint16 codes ``w_element`` + ``w_tensor_meta``; the bias likewise (``bias`` or ``b_element`` +
``b_tensor_meta``).  Parameter names, constructor arguments and class methods match the
reference so state dicts and call sites interchange.
"""

from __future__ import annotations

from typing import Literal

import torch
from torch import Tensor, nn

from .._ptq_base import PTQLinearBase
from . import functional as MinifloatF
from .meta import MinifloatMeta, MinifloatTensorMeta

LayerType = Literal["XWB", "XWBq", "XWqB", "XWqBq", "XqWB", "XqWBq", "XqWqB", "XqWqBq"]


class MinifloatLinearPTQ(PTQLinearBase):
    _code_tensors = ("w_element", "b_element")
    _meta_follows = {"w_tensor_meta": "w_element", "b_tensor_meta": "b_element"}

    def __init__(
        self,
        weight: Tensor,
        bias: Tensor | None,
        x_minifloat_meta: MinifloatMeta | None,
        w_minifloat_meta: MinifloatMeta | None,
        b_minifloat_meta: MinifloatMeta | None,
        layer_type: LayerType,
        backend: Literal["separate", "fused"] = "fused",
        dtype: torch.dtype | None = None,
        device: torch.device | None = None,
        w_element: Tensor | None = None,
        w_tensor_meta: MinifloatTensorMeta | None = None,
        b_element: Tensor | None = None,
        b_tensor_meta: MinifloatTensorMeta | None = None,
    ):
        super().__init__()
        assert weight is None or weight.ndim == 2
        assert bias is None or bias.ndim == 1
        have_w_codes = w_element is not None and w_tensor_meta is not None
        have_b_codes = b_element is not None and b_tensor_meta is not None
        assert (weight is not None) ^ have_w_codes
        if bias is not None and have_b_codes:
            raise ValueError("Either bias or b_element, b_tensor_meta must be None, not both.")
        out_features, in_features = w_tensor_meta.shape if weight is None else weight.shape
        assert bias is None or bias.shape[0] == out_features

        self.in_features, self.out_features = in_features, out_features
        self.x_minifloat_meta = x_minifloat_meta
        self.w_minifloat_meta = w_minifloat_meta
        self.b_minifloat_meta = b_minifloat_meta
        self.layer_type = layer_type
        self.backend = backend
        self.dtype, self.device = dtype, device

        self.weight = self.w_element = self.w_tensor_meta = None
        self.bias = self.b_element = self.b_tensor_meta = None

        if "Wq" in layer_type:
            if w_element is None:
                w_element, w_tensor_meta = MinifloatF.extract_minifloat_component(weight, w_minifloat_meta)
            self.w_element, self.w_tensor_meta = self._frozen(w_element), w_tensor_meta
        else:
            assert weight is not None
            self.weight = self._frozen(weight.to(dtype=dtype, device=device))

        if "Bq" in layer_type:
            if bias is not None and b_element is None:
                b_element, b_tensor_meta = MinifloatF.extract_minifloat_component(bias, b_minifloat_meta)
            if b_element is not None:
                self.b_element, self.b_tensor_meta = self._frozen(b_element), b_tensor_meta
        elif bias is not None:
            self.bias = self._frozen(bias.to(dtype=dtype, device=device))

    @torch.no_grad()
    def forward(self, input: Tensor) -> Tensor:
        return MinifloatF.minifloat_linear(
            x=input, x_meta=self.x_minifloat_meta,
            w=self.weight, w_element=self.w_element, w_tensor_meta=self.w_tensor_meta,
            b=self.bias, b_element=self.b_element, b_tensor_meta=self.b_tensor_meta,
            layer_type=self.layer_type, backend=self.backend,
        )

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, "
                f"layer_type={self.layer_type}, w_minifloat_meta={self.w_minifloat_meta}, "
                f"x_minifloat_meta={self.x_minifloat_meta}, b_minifloat_meta={self.b_minifloat_meta}")

    @classmethod
    def from_linear(cls, layer: nn.Linear, x_minifloat_meta: MinifloatMeta | None, w_minifloat_meta: MinifloatMeta | None,
                    b_minifloat_meta: MinifloatMeta | None, layer_type: LayerType, backend: Literal["separate", "fused"]):
        """Quantise an existing ``nn.Linear`` (its tensors are cloned, the layer is left untouched)."""
        assert isinstance(layer, nn.Linear), "layer must be an instance of nn.Linear"
        with torch.no_grad():
            return cls(weight=layer.weight.clone(), bias=None if layer.bias is None else layer.bias.clone(),
                       x_minifloat_meta=x_minifloat_meta, w_minifloat_meta=w_minifloat_meta,
                       b_minifloat_meta=b_minifloat_meta, layer_type=layer_type, backend=backend)

    @classmethod
    def from_quantized(cls, w_element: Tensor | None, w_tensor_meta: MinifloatTensorMeta | None, bias: Tensor | None,
                       b_element: Tensor | None, b_tensor_meta: MinifloatTensorMeta | None,
                       x_minifloat_meta: MinifloatMeta | None, layer_type: Literal["XWqB", "XWqBq", "XqWqB", "XqWqBq"],
                       backend: Literal["separate", "fused"]):
        """Rebuild a layer from stored codes (tensor metas are not part of ``state_dict``)."""
        assert w_element is not None and w_tensor_meta is not None
        return cls(weight=None, bias=bias, x_minifloat_meta=x_minifloat_meta, w_minifloat_meta=None,
                   b_minifloat_meta=None, layer_type=layer_type, backend=backend,
                   dtype=getattr(torch, w_tensor_meta.dtype), device=torch.device(w_tensor_meta.device),
                   w_element=w_element, w_tensor_meta=w_tensor_meta, b_element=b_element, b_tensor_meta=b_tensor_meta)
