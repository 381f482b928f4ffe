"""Several mixers side by side: all read the same input and the result is the weighted sum of their outputs,

    y = sum_i scales[i] * mixers[i](x)

Each keeps its own cache needs: at most one of them may ask for pages (the layer has one block table), and the
states of all are named tensors of the layer's one state block, under ``<index>.<name>``.  The sum itself is not
made here when the block norms the mixer's output before adding it: the block's norm kernel takes the outputs
and their scales (:meth:`MixerSum.forward_parts`); ``forward_add`` serves blocks that add directly.
"""
from __future__ import annotations

from dataclasses import replace

import torch

from ..cache.specs import CacheSpec, StateSpec
from ..kernels import ops
from .base import Mixer, build_part, register_part


class MixerSum(Mixer):
    def __init__(self, spec):
        super().__init__(spec)
        if len(spec.mixers) != len(spec.scales) or not spec.mixers:
            raise ValueError("mixer_sum: one scale per mixer, at least one mixer")
        self.mixers = [build_part(m) for m in spec.mixers]
        self.scales = [float(x) for x in spec.scales]

    @property
    def graph_safe(self):
        return all(m.graph_safe for m in self.mixers)

    def tensor_decls(self):
        return [d for m in self.mixers for d in m.tensor_decls()]

    def load(self, src, rt):
        super().load(src, rt)
        for m in self.mixers:
            m.load(src, rt)

    def reset_after_fault(self):
        for m in self.mixers:
            m.reset_after_fault()

    def cache_spec(self):
        paged, parts, dtype = None, [], torch.float32
        for i, m in enumerate(self.mixers):
            cs = m.cache_spec()
            if cs is None:
                continue
            if cs.paged is not None:
                if paged is not None:
                    raise ValueError("mixer_sum: only one of the mixers may keep pages")
                paged = cs.paged
            if cs.state is not None:
                own = cs.state.parts or (("state", cs.state.shape),)
                parts += [(f"{i}.{name}", shape) for name, shape in own]
                dtype = cs.state.dtype
        if paged is None and not parts:
            return None
        return CacheSpec(paged=paged, state=StateSpec(parts=tuple(parts), dtype=dtype) if parts else None)

    def _view(self, i, cache):
        """The layer's cache as mixer i sees it: its own state tensors under their own names."""
        pre = f"{i}."
        own = {n[len(pre):]: t for n, t in (cache.states or {}).items() if n.startswith(pre)}
        return replace(cache, states=own or None, state=own.get("state"))

    def forward_parts(self, x, batch, cache):
        """[(32-bit output of mixer i, scale i)]: for a caller that sums them itself."""
        outs = []
        for i, m in enumerate(self.mixers):
            y = self.rt.empty(x.shape[0], self.spec_hidden(m), dtype=torch.float32)
            m.forward_into(x, y, batch, self._view(i, cache), accumulate=False)
            outs.append((y, self.scales[i]))
        return outs

    @staticmethod
    def spec_hidden(m):
        return m.spec.hidden

    def forward_add(self, x, h, batch, cache):
        for i, m in enumerate(self.mixers):
            if self.scales[i] == 1.0:
                m.forward_add(x, h, batch, self._view(i, cache))
            else:
                y = self.rt.empty(x.shape[0], h.shape[1], dtype=torch.float32)
                m.forward_into(x, y, batch, self._view(i, cache), accumulate=False)
                ops.scale_(y, self.scales[i], stream=batch.stream)
                ops.residual_add(h, y, stream=batch.stream)


register_part("mixer_sum", MixerSum, replace=True)
