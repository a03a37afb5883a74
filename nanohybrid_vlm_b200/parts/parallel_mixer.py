"""Two mixers side by side on the same input: out = left_scale * left(x) + right_scale * right(x).

Parameters: ``left`` and ``right`` (PartSpecs of registered mixers), ``left_scale``, ``right_scale``,
``prefixes`` (where each side's tensors sit under this part's own prefix; default ("left.", "right.")).
Each side keeps its own cache or state: the need is the composite of both, and each side gets its child view.
A block that adds weighted terms in 32-bit (``forward_terms``) receives the two outputs with their scales and no
sum is rounded on the way; ``forward`` gives the one summed tensor.
"""
from __future__ import annotations

from dataclasses import replace

from ..kernels import ops
from .base import MIXERS, CompositeNeed, Mixer


class ParallelMixers(Mixer):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.sides = [MIXERS.get(spec[name].kind)(spec[name], env) for name in ("left", "right")]
        self.scales = (float(spec.get("left_scale", 1.0)), float(spec.get("right_scale", 1.0)))
        self.prefixes = tuple(spec.get("prefixes", ("left.", "right.")))

    def params(self):
        decls = []
        for side, prefix in zip(self.sides, self.prefixes):
            for d in side.params():
                srcs = tuple(replace(s, name=prefix + s.name) for s in d.resolved_sources())
                decls.append(replace(d, name=prefix + d.name, sources=srcs))
        return decls

    def bind(self, tensors):
        for side, prefix in zip(self.sides, self.prefixes):
            side.bind({name[len(prefix):]: t for name, t in tensors.items() if name.startswith(prefix)})

    def cache_need(self):
        return CompositeNeed(tuple(side.cache_need() for side in self.sides))

    def streamed_weights(self):
        return [w for side in self.sides for w in side.streamed_weights()]

    def forward_terms(self, x, batch, cache):
        return tuple((side.forward(x, batch, view), scale)
                     for side, view, scale in zip(self.sides, cache.children, self.scales))

    def forward(self, x, batch, cache):
        (a, ca), (b, cb) = self.forward_terms(x, batch, cache)
        out = self.new(*a.shape)
        ops.scaled_sum(out, a, b, ca, cb)
        return out


MIXERS.register("parallel_mixers", ParallelMixers)
