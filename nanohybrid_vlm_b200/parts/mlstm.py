"""The matrix-memory mixer of xLSTM (mLSTM) with capped gates.

Parameters: ``num_heads`` (H), ``head_dim`` (d of q and k), ``v_head_dim`` (dv), ``gate_cap`` (cap), ``eps`` (of the
output norm).

q = W_q x * d^-1/2, k = W_k x, v = W_v x.  Per head a log input gate i = cap tanh((W_i x + b_i) / cap) and a log forget
gate f = logsigmoid(cap tanh((W_f x + b_f) / cap)).  With the memory S [d, dv], the normaliser n [d] and a running
maximum m (S, n start at zero, m at 0): m' = max(f + m, i); S <- exp(f + m - m') S + exp(i - m') k v^T, n likewise with
k alone; o = S^T q / (max(|n . q|, exp(-m')) + 1e-6).  Each head's o is divided by its root mean square over dv,
multiplied by the weight ``norm`` [H dv] and by sigmoid(W_g x); then the output projection.

Tensors: ``qkvg`` [2 H d + 2 H dv, width] packed from the checkpoint's ``q``, ``k``, ``v``, ``g``; ``if`` [2 H, width]
from ``i``, ``f``; ``if_bias`` [2 H] (float32) from ``i.b``, ``f.b``; ``norm`` [H dv]; ``o`` [width, H dv].  Per request
the mixer keeps S, n and m in float32.  The gates' projections keep their 32-bit sums; cap, tanh, logsigmoid, the
exponentials, the recurrence and the output norm are 32-bit.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import MIXERS, FixedStateNeed, Mixer
from .spec import ParamDecl, Source


class MLSTM(Mixer):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.H = int(spec["num_heads"])
        self.d = int(spec["head_dim"])
        self.dv = int(spec.get("v_head_dim") or self.d)
        self.cap = float(spec["gate_cap"])
        self.eps = float(spec["eps"])
        if min(self.H, self.d, self.dv) <= 0 or self.cap <= 0:
            raise ValueError("an mLSTM needs positive sizes and a positive gate cap")
        self.qk_size, self.v_size = self.H * self.d, self.H * self.dv

    def params(self):
        W, qk, v, H = self.env.hidden_size, self.qk_size, self.v_size, self.H
        return [
            ParamDecl("qkvg", (2 * qk + 2 * v, W), sources=(Source("q", 0, qk), Source("k", qk, qk), Source("v", 2 * qk, v),
                                                            Source("g", 2 * qk + v, v))),
            ParamDecl("if", (2 * H, W), sources=(Source("i", 0, H), Source("f", H, H))),
            ParamDecl("if_bias", (2 * H,), init="gate_bias", storage="float32",
                      sources=(Source("i.b", 0, H), Source("f.b", H, H))),
            ParamDecl("norm", (v,), init="norm"),
            ParamDecl("o", (W, v)),
        ]

    def cache_need(self):
        return FixedStateNeed((ops.mlstm_state_floats(self.H, self.d, self.dv),))

    def streamed_weights(self):
        return [(self.w_qkvg, 0), (self.w_o, 0)]

    def forward(self, x, batch, cache):
        T = x.shape[0]
        qk, v = self.qk_size, self.v_size
        proj = self.new(T, 2 * qk + 2 * v)
        ops.linear(proj, x, self.w_qkvg)
        gates = self.new(T, 2 * self.H, dtype=torch.float32)
        ops.linear_f32(gates, x, self.w_if)
        o = self.new(T, v, dtype=torch.float32)
        ops.mlstm_scan(o, proj, gates, self.w_if_bias, self.cap, cache.state, batch, self.H, self.d, self.dv)
        gated = self.new(T, v)
        ops.gated_rmsnorm(gated, o, proj[:, 2 * qk + v:], self.w_norm, self.H, self.eps, gate_first=False, gate="sigmoid")
        out = self.new(T, self.env.hidden_size)
        ops.linear(out, gated, self.w_o)
        return out


MIXERS.register("mlstm", MLSTM)
