"""RMSNorm with the residual add fused in (nanovllm/layers/layernorm.py:5-50).

Parameters: ``width``, ``eps``, ``weight_offset`` (0 for ``x * w``; 1 for the ``x * (1 + w)``
convention some models store), ``source`` (the checkpoint's name of the weight, default "weight").

Over a residual stream kept in float32 (``forward_add`` / ``forward_add_rows`` given a :class:`Pending`) the terms
are added in 32-bit, the statistics and the product with the weight are 32-bit, and the result is rounded once.
"""
from __future__ import annotations

from ..kernels import ops
from .base import NORMS, Norm, Pending
from .spec import ParamDecl, Source


class RMSNorm(Norm):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.width = spec["width"]
        self.eps = float(spec["eps"])
        self.weight_offset = float(spec.get("weight_offset", 0.0))
        self.source = spec.get("source", "weight")

    def params(self):
        return [ParamDecl("weight", (self.width,), init="norm" if self.weight_offset == 0.0 else "zeros_noise",
                          sources=(Source(self.source, 0, self.width),))]

    def forward(self, x):
        out = self.new(*x.shape)
        ops.rmsnorm(out, x, self.w_weight, self.eps, weight_offset=self.weight_offset)
        return out

    def forward_add(self, x, residual):
        if isinstance(x, Pending):
            out = self.new(*residual.shape)
            ops.rmsnorm_stream(out, residual, self.w_weight, self.eps, addends=x.terms, weight_offset=self.weight_offset)
            return out
        out = self.new(*x.shape)
        ops.rmsnorm(out, x, self.w_weight, self.eps, residual=residual, weight_offset=self.weight_offset)
        return out

    def forward_add_rows(self, x, residual, rows):
        if isinstance(x, Pending):
            out = self.new(rows.numel(), residual.shape[-1])
            ops.rmsnorm_stream(out, residual, self.w_weight, self.eps, addends=x.terms, rows=rows, write_stream=False,
                               weight_offset=self.weight_offset)
            return out
        out = self.new(rows.numel(), x.shape[-1])
        ops.rmsnorm(out, x, self.w_weight, self.eps, residual=residual, rows=rows, write_residual=False,
                    weight_offset=self.weight_offset)
        return out


NORMS.register("rmsnorm", RMSNorm)
