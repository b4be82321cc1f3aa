"""Behaviour shared by ``MXFPLinearPTQ`` and ``MinifloatLinearPTQ``.

Both layers keep integer code tensors as ``nn.Parameter``s (so they travel with
``state_dict``) next to plain-Python tensor metas (which do not).  Moving the module
must never re-type a code tensor, and must refresh the device recorded in the metas
because ``compose_*`` dispatches on the meta's device string
(reference: ``src/mase_triton/mxfp/layers.py:100-121``, ``src/mase_triton/minifloat/layers.py:89-108``).
"""

from __future__ import annotations

from torch import nn

from .utils.qlayer import ChangeDtypeError


class PTQLinearBase(nn.Module):
    # names of the integer code tensors, and for each tensor meta the code tensor whose device it follows
    _code_tensors: tuple[str, ...] = ()
    _meta_follows: dict[str, str] = {}

    in_features: int
    out_features: int

    def _apply(self, fn, recurse=True):
        before = {name: getattr(self, name).dtype for name in self._code_tensors if getattr(self, name) is not None}
        result = super()._apply(fn, recurse)
        for name, dtype in before.items():
            now = getattr(self, name).dtype
            if now != dtype:
                raise ChangeDtypeError(f"Changing dtype of {name} from {dtype} to {now} is not allowed.")
        for meta_name, tensor_name in self._meta_follows.items():
            meta, tensor = getattr(self, meta_name), getattr(self, tensor_name)
            if meta is not None and tensor is not None:
                setattr(self, meta_name, meta.create(device=tensor.device))
        return result

    @staticmethod
    def _frozen(t):
        return nn.Parameter(t, requires_grad=False)
