"""Grouped-query attention with a learned sink per head, rotation before a weightless q/k norm, and value heads
whose size may differ from the key heads'.

Parameters: ``num_heads``, ``num_kv_heads``, ``head_dim`` (queries and keys), ``v_head_dim`` (values; default
``head_dim``), ``scale`` (on q . k; None: head_dim ** -0.5), ``position`` (a PartSpec of a position encoding with a
rotary table, or None), ``unit_norm_eps`` (after the rotation each q and k head is divided by its root mean square
with this eps inside the root; None: no norm), ``sink`` (True: the softmax denominator of head h also holds
exp(sink_h), a learned number with no key and no value, unscaled, counted once), ``window`` (None: all keys).

Tensors: ``qkv`` [(nq + nkv) d + nkv dv, width], rows q then k then v, packed from the checkpoint's ``q``, ``k``,
``v``; ``sink`` [nq] (float32); ``o`` [width, nq dv].  Scores, softmax, rotation and norm are computed in 32-bit.
"""
from __future__ import annotations

from ..kernels import ops
from .base import MIXERS, Mixer, PagedKVNeed
from .spec import ParamDecl, Source


class SinkAttention(Mixer):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.nq = int(spec["num_heads"])
        self.nkv = int(spec["num_kv_heads"])
        self.d = int(spec["head_dim"])
        self.dv = int(spec.get("v_head_dim") or self.d)
        if self.nq % self.nkv:
            raise ValueError(f"{self.nq} query heads do not divide into {self.nkv} KV heads")
        scale = spec.get("scale")
        self.scale = float(scale) if scale is not None else self.d ** -0.5
        eps = spec.get("unit_norm_eps")
        self.eps = None if eps is None else float(eps)
        self.has_sink = bool(spec.get("sink", True))
        self.window = spec.get("window")
        self.position = env.position(spec.get("position"))
        self.q_size, self.k_size, self.v_size = self.nq * self.d, self.nkv * self.d, self.nkv * self.dv

    def params(self):
        H = self.env.hidden_size
        decls = [
            ParamDecl("qkv", (self.q_size + self.k_size + self.v_size, H), sources=(
                Source("q", 0, self.q_size), Source("k", self.q_size, self.k_size),
                Source("v", self.q_size + self.k_size, self.v_size))),
            ParamDecl("o", (H, self.nq * self.dv)),
        ]
        if self.has_sink:
            decls.append(ParamDecl("sink", (self.nq,), storage="float32"))
        return decls

    def cache_need(self):
        return PagedKVNeed(self.nkv, self.d, self.window, v_head_dim=self.dv)

    def streamed_weights(self):
        return [(self.w_qkv, 0), (self.w_o, 0)]

    def forward(self, x, batch, cache):
        T = x.shape[0]
        qkv = self.new(T, self.q_size + self.k_size + self.v_size)
        ops.linear(qkv, x, self.w_qkv)
        rot = self.position.rotary() if self.position is not None else None
        table, rotary_dim = rot if rot is not None else (None, 0)
        q = self.new(T, self.q_size)
        ops.rope_norm_store(qkv, q, cache.pages if cache.writes else None, cache.tables.slot_mapping, batch.positions,
                            table, rotary_dim, self.nq, self.nkv, self.d, self.dv, self.eps)
        o = self.new(T, self.nq * self.dv)
        ops.attention_sink(o, q, cache.pages, cache.tables, batch, self.nq, self.nkv, self.d, self.dv, self.scale,
                           self.w_sink if self.has_sink else None, self.window or 0)
        y = self.new(T, self.env.hidden_size)
        ops.linear(y, o, self.w_o)
        return y


MIXERS.register("sink_attention", SinkAttention)
