"""Pre-norm block with the residual carried apart (nanovllm/models/qwen3.py:146-159).

Every sub-block's output is added to the residual stream inside the next norm, so the
block hands on (output of its feed-forward, residual) and the model's final norm does the
last add.
"""
from __future__ import annotations

import torch

from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Block, Pending


class PreNormResidualBlock(Block):
    def forward(self, hidden, residual, batch, cache):
        if residual is None:
            residual = hidden
            x = self.mixer_norm.forward(hidden)
        else:
            x = self.mixer_norm.forward_add(hidden, residual)
        a = self.mixer.forward(x, batch, cache)
        x = self.ffn_norm.forward_add(a, residual)
        m = self.ffn.forward(x, batch)
        return m, residual


class ParallelResidualBlock(Block):
    """One norm whose output both the mixer and the feed-forward read: x <- x + mult * (mixer(h) + ffn(h)) with
    h = norm(x).  The residual stream x is kept in float32: the block hands on its sub-blocks' outputs as a
    :class:`Pending` (each with its factor) and the next norm (the next layer's, or the model's last) adds them in
    32-bit.  Parameter: ``residual_mult``.  A layer may have no feed-forward."""
    SLOTS = {"mixer": MIXERS, "norm": NORMS, "ffn": FEED_FORWARDS}
    OPTIONAL = ("ffn",)

    def __init__(self, spec, parts):
        super().__init__(spec, parts)
        self.mult = float(spec.get("residual_mult", 1.0))

    def forward(self, hidden, residual, batch, cache):
        if residual is None:
            residual = hidden if hidden.dtype == torch.float32 else hidden.float()
            hidden = Pending()
        x = self.norm.forward_add(hidden, residual)
        terms = [(t, self.mult * c) for t, c in self.mixer.forward_terms(x, batch, cache)]
        ffn = self.parts.get("ffn")
        if ffn is not None:
            terms.append((ffn.forward(x, batch), self.mult))
        return Pending(tuple(terms)), residual


BLOCKS.register("prenorm_residual", PreNormResidualBlock)
BLOCKS.register("parallel_residual", ParallelResidualBlock)
