"""The Mamba-2 mixer (state-space duality with a scalar decay per head).

Parameters: ``num_heads``, ``head_dim`` (P, the width of a head's x), ``state_size`` (N), ``groups`` (G: heads
h of one group share B and C; head h uses group h // (heads / G)), ``conv`` (taps of the short convolution),
``norm_groups`` (the gated norm works on this many equal parts of a row), ``eps``.

With inner = heads * P the input projection gives [z: inner | x: inner | B: G N | C: G N | dt: heads].  x, B and C
pass one causal convolution per channel (with bias) and SiLU.  dt = softplus(dt + dt_bias), no clamp.  Per head:
S <- exp(-exp(A_log) dt) S + dt B x^T (S is N x P), y = S^T C + D x.  Then y * silu(z), scaled to unit root mean
square in ``norm_groups`` parts, times the weight ``norm``, and the output projection.

Tensors: ``in`` [2 inner + 2 G N + heads, width], ``conv`` [inner + 2 G N, taps], ``conv.b``, ``dt_bias`` / ``A_log``
/ ``D`` [heads] (float32), ``norm`` [inner], ``o`` [width, inner].  Per request the mixer keeps the last taps - 1
inputs of the convolution and S, both in float32.  The convolution writes float32, so x, B and C enter the
recurrence unrounded; dt, the decay, the recurrence and the gated norm are 32-bit.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import MIXERS, CompositeNeed, FixedStateNeed, Mixer
from .spec import ParamDecl


class Mamba2(Mixer):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.heads = int(spec["num_heads"])
        self.P = int(spec["head_dim"])
        self.N = int(spec["state_size"])
        self.G = int(spec.get("groups", 1))
        self.taps = int(spec["conv"])
        self.norm_groups = int(spec.get("norm_groups", 1))
        self.eps = float(spec["eps"])
        if self.heads % self.G:
            raise ValueError(f"{self.heads} heads do not divide into {self.G} groups")
        self.inner = self.heads * self.P
        if self.inner % self.norm_groups:
            raise ValueError(f"{self.inner} channels do not divide into {self.norm_groups} norm groups")
        self.conv_channels = self.inner + 2 * self.G * self.N

    def params(self):
        W = self.env.hidden_size
        C = self.conv_channels
        return [
            ParamDecl("in", (self.inner + C + self.heads, W)),
            ParamDecl("conv", (C, self.taps)),
            ParamDecl("conv.b", (C,), init="zeros_noise"),
            ParamDecl("dt_bias", (self.heads,), init="zeros_noise", storage="float32"),
            ParamDecl("A_log", (self.heads,), init="zeros_noise", storage="float32"),
            ParamDecl("D", (self.heads,), init="norm", storage="float32"),
            ParamDecl("norm", (self.inner,), init="norm"),
            ParamDecl("o", (W, self.inner)),
        ]

    def bind(self, tensors):
        super().bind(tensors)
        split = self.inner + self.conv_channels
        self.w_in_main, self.w_in_dt = self.w_in[:split], self.w_in[split:]     # row ranges: contiguous matrices

    def cache_need(self):
        return CompositeNeed((FixedStateNeed(((self.taps - 1) * self.conv_channels,)),
                              FixedStateNeed((self.heads * self.P * self.N,))))

    def streamed_weights(self):
        return [(self.w_in_main, 0), (self.w_o, 0)]

    def forward(self, x, batch, cache):
        T = x.shape[0]
        conv_state, ssm_state = cache.children[0].state, cache.children[1].state
        zxbc = self.new(T, self.inner + self.conv_channels)
        ops.linear(zxbc, x, self.w_in_main)
        dt = self.new(T, self.heads, dtype=torch.float32)
        ops.linear_f32(dt, x, self.w_in_dt)
        xbc = self.new(T, self.conv_channels, dtype=torch.float32)      # what enters the recurrence stays 32-bit
        ops.short_conv_silu(xbc, zxbc[:, self.inner:], self.w_conv, self.w_conv_b, conv_state, batch)
        y = self.new(T, self.inner, dtype=torch.float32)
        ops.ssd_scan(y, xbc, dt, self.w_dt_bias, self.w_A_log, self.w_D, ssm_state, batch, self.heads, self.P, self.N,
                     self.G)
        gated = self.new(T, self.inner)
        ops.gated_rmsnorm(gated, y, zxbc[:, :self.inner], self.w_norm, self.norm_groups, self.eps, gate_first=True)
        out = self.new(T, self.env.hidden_size)
        ops.linear(out, gated, self.w_o)
        return out


MIXERS.register("mamba2", Mamba2)
