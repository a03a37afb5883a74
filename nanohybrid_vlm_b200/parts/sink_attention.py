"""Grouped-query attention with options that several designs combine differently: a learned sink per head, rotation
before a weightless q/k norm, value heads whose size may differ from the key heads', values that are the keys
themselves, a window or chunks, projection biases, and a sigmoid gate on the output.

Parameters: ``num_heads``, ``num_kv_heads``, ``head_dim`` (queries and keys), ``v_head_dim`` (values; default
``head_dim``), ``scale`` (on q . k; None: head_dim ** -0.5), ``position`` (a PartSpec of a position encoding with a
rotary table, or None), ``unit_norm_eps`` (after the rotation each q and k head is divided by its root mean square
with this eps inside the root; None: no norm), ``sink`` (True: the softmax denominator of head h also holds
exp(sink_h), a learned number with no key and no value, unscaled, counted once), ``window`` (None: all keys; n: the
last n), ``chunk`` (None, or n: a query sees only the keys of its own chunk of n positions, chunks counted from
position 0 of the request), ``values`` ("projected": a projection of their own; "keys": the values are the key heads as
projected, bias included, before the rotation, and there is no value projection), ``bias`` (True: q, k and the output
projection have biases ``q.b``, ``k.b``, ``o.b``), ``output_gate`` (None, or "sigmoid": the concatenated heads are
multiplied by sigmoid(g(x)) before the output projection, g a projection of the mixer's input).

Tensors: ``qkv`` [(nq + nkv) d (+ nkv dv) (+ nq dv), width], rows q then k then v then g, packed from the
checkpoint's ``q``, ``k``, ``v``, ``g`` (those that exist); ``qk_bias`` [(nq + nkv) d] from ``q.b``, ``k.b``; ``sink``
[nq] (float32); ``o`` [width, nq dv]; ``o.b`` [width].  Scores, softmax, rotation, bias and norm are computed in 32-bit.
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
        self.chunk = spec.get("chunk")
        self.values = spec.get("values", "projected")
        if self.values not in ("projected", "keys"):
            raise ValueError(f"values are 'projected' or 'keys', not {self.values!r}")
        if self.values == "keys" and self.dv != self.d:
            raise ValueError(f"values that are the keys have the keys' size {self.d}, not {self.dv}")
        self.bias = bool(spec.get("bias", False))
        self.gate = spec.get("output_gate")
        if self.gate not in (None, "sigmoid"):
            raise ValueError(f"an output gate is None or 'sigmoid', not {self.gate!r}")
        self.position = env.position(spec.get("position"))
        self.q_size, self.k_size = self.nq * self.d, self.nkv * self.d
        self.v_size = self.nkv * self.dv if self.values == "projected" else 0
        self.g_size = self.nq * self.dv if self.gate else 0

    def params(self):
        H = self.env.hidden_size
        sources = [Source("q", 0, self.q_size), Source("k", self.q_size, self.k_size)]
        if self.v_size:
            sources.append(Source("v", self.q_size + self.k_size, self.v_size))
        if self.g_size:
            sources.append(Source("g", self.q_size + self.k_size + self.v_size, self.g_size))
        decls = [
            ParamDecl("qkv", (self.q_size + self.k_size + self.v_size + self.g_size, H), sources=tuple(sources)),
            ParamDecl("o", (H, self.nq * self.dv)),
        ]
        if self.has_sink:
            decls.append(ParamDecl("sink", (self.nq,), storage="float32"))
        if self.bias:
            decls += [ParamDecl("qk_bias", (self.q_size + self.k_size,), init="zeros_noise",
                                sources=(Source("q.b", 0, self.q_size), Source("k.b", self.q_size, self.k_size))),
                      ParamDecl("o.b", (H,), init="zeros_noise")]
        return decls

    def cache_need(self):
        return PagedKVNeed(self.nkv, self.d, self.window, v_head_dim=self.dv, chunk=self.chunk)

    def streamed_weights(self):
        return [(self.w_qkv, 0), (self.w_o, 0)]

    def forward(self, x, batch, cache):
        T = x.shape[0]
        qkv = self.new(T, self.q_size + self.k_size + self.v_size + self.g_size)
        ops.linear(qkv, x, self.w_qkv)
        rot = self.position.rotary() if self.position is not None else None
        table, rotary_dim = rot if rot is not None else (None, 0)
        q = self.new(T, self.q_size)
        ops.rope_norm_store(qkv, q, cache.pages if cache.writes else None, cache.tables.slot_mapping, batch.positions,
                            table, rotary_dim, self.nq, self.nkv, self.d, self.dv, self.eps,
                            bias=self.w_qk_bias if self.bias else None, values_from_keys=self.values == "keys")
        o = self.new(T, self.nq * self.dv)
        ops.attention_sink(o, q, cache.pages, cache.tables, batch, self.nq, self.nkv, self.d, self.dv, self.scale,
                           self.w_sink if self.has_sink else None, self.window or 0, self.chunk or 0)
        if self.gate:
            ops.sigmoid_mul(o, o, qkv[:, self.q_size + self.k_size + self.v_size:])
        y = self.new(T, self.env.hidden_size)
        ops.linear(y, o, self.w_o)
        if self.bias:
            ops.add_row_bias(y, self.w_o_b)
        return y


MIXERS.register("sink_attention", SinkAttention)
