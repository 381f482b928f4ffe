"""RMSNorm: x * (1 / sqrt(mean(x^2) + eps)) * w, statistics in 32 bits
(reference: crates/ferrox-core/src/matmul.rs:62-69,121-123)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Norm, register_part


class RmsNorm(Norm):
    """``one_plus``: the stored weight lies around zero and the norm multiplies by 1 + w (added once, in 32 bits,
    when the weights are loaded)."""

    graph_safe = True

    def _name(self):
        return getattr(self.spec, "name", None) or self.spec.prefix + "weight"

    def tensor_decls(self):
        one_plus = getattr(self.spec, "one_plus", False)
        return [TensorDecl(self._name(), (self.spec.size,), init="normal" if one_plus else "ones")]

    def load(self, src, rt):
        super().load(src, rt)
        self.weight = src.get(self._name())
        if getattr(self.spec, "one_plus", False):
            self.weight = (1.0 + self.weight.to(torch.float32)).contiguous()

    def forward(self, h, rows=None):
        n = h.shape[0] if rows is None else rows.numel()
        out = self.rt.empty(n, self.spec.size)
        return ops.rmsnorm(h, self.weight, self.spec.eps, out, rows=rows)


    def as_rms(self):
        return self.weight, self.spec.eps


class LayerNorm(Norm):
    """(x - mean) / sqrt(variance + eps) * w, the variance being the mean of the squared deviations; a weight and
    no bias; statistics in 32 bits."""

    graph_safe = True

    def tensor_decls(self):
        return [TensorDecl(self.spec.name, (self.spec.size,), init="ones")]

    def load(self, src, rt):
        super().load(src, rt)
        self.weight = src.get(self.spec.name)

    def forward(self, h, rows=None):
        n = h.shape[0] if rows is None else rows.numel()
        out = self.rt.empty(n, self.spec.size)
        return ops.layernorm(h, self.weight, self.spec.eps, out, rows=rows)

    def forward_in_place(self, h):
        """The 32-bit stream normed where it lies."""
        return ops.layernorm(h, self.weight, self.spec.eps, h)

    def as_layer_norm(self):
        return self.weight, self.spec.eps


register_part("rms_norm", RmsNorm, replace=True)
register_part("layer_norm", LayerNorm, replace=True)
