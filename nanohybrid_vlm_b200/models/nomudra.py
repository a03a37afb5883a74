"""Nomudra: a decoder-only model whose layers are listed one by one in config.json; attention in chunks whose values
are its keys, or an mLSTM, each followed by a mixture of experts, between Dynamic Tanh norms.

config.json: ``architecture`` "Nomudra"; ``vocab``, ``width``; ``norm.eps``; ``layers``: a list of {``type``, ``mixer``,
``mlp``}.  Every layer norms a sub-block's input and its output: x <- x + norm1b(mixer(norm1(x))), then, if the layer
has a feed-forward, x <- x + norm2b(mlp(norm2(x))); the stream x is float32 and every norm a Dynamic Tanh
(tanh(alpha x) w + b; tensors ``<name>``, ``<name>.b``, ``<name>.alpha``).  Layer types:

* ``attention`` (``mixer``: heads, kv_heads, dim, vdim, scale, rot {base, dims}, mask {size}): q and k with biases,
  the values are the keys as projected (vdim = dim), rotary positions on the first rot.dims dimensions in the
  rotate-half layout, a query sees the keys of its own chunk of mask.size positions (no mask: all earlier keys),
  ordinary softmax, a sigmoid output gate ``g`` on the concatenated heads, output projection with bias;
* ``mlstm`` (``mixer``: heads, dim, vdim, gate_cap): the matrix memory of xLSTM with capped log gates.

``mlp`` is null or {``kind``: "moe", ``router`` {experts, identity, top, groups {count, keep}}, ``expert`` {ff, limit},
``shared`` {ff, limit} or null}: clamped gated experts chosen by a softmax router with a correction for the choice and
groups, identity experts, and a shared expert with a sigmoid gate per token.

The model begins with the embedding through the norm ``embed.norm`` and ends with ``final.norm`` and the untied table
``head``.  Tensors per layer i: ``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.norm2``, ``l<i>.norm2b`` (each with ``.b`` and
``.alpha``), ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""
from __future__ import annotations

import json
from dataclasses import dataclass

from ..config.model_config import ConfigError, ModelConfig, parse_dtype, take
from ..config.registry import register_architecture
from ..parts.spec import LayerRun, LayerSpec, ModelSpec, PartUse, part

ARCHITECTURE = "Nomudra"
NO_POSITION_LIMIT = 1 << 20     # the design names no longest sequence; the engine's max_model_len is the limit in use
EXPERT_ALPHA = 1.702            # the experts' sigmoid takes 1.702 g: fixed by the design


def _sub(raw: dict, key: str, where: str) -> dict:
    v = raw.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: key {key!r} must be an object")
    return v


def _check_attention(m: dict, where: str) -> None:
    heads, kv = take(m, "heads", int, where=where), take(m, "kv_heads", int, where=where)
    dim, vdim = take(m, "dim", int, where=where), take(m, "vdim", int, where=where)
    take(m, "scale", float, where=where)
    if min(heads, kv, dim) <= 0 or heads % kv:
        raise ConfigError(f"{where}: heads {heads} must be a positive multiple of kv_heads {kv}, sizes positive")
    if vdim != dim:
        raise ConfigError(f"{where}: the values are the keys, so vdim {vdim} must equal dim {dim}")
    rot = _sub(m, "rot", where)
    dims = take(rot, "dims", int, where=where + ".rot")
    take(rot, "base", float, where=where + ".rot")
    if dims <= 0 or dims % 2 or dims > dim:
        raise ConfigError(f"{where}.rot: dims {dims} must be even and at most dim {dim}")
    if m.get("mask") is not None and take(_sub(m, "mask", where), "size", int, where=where + ".mask") <= 0:
        raise ConfigError(f"{where}.mask: size must be positive")


def _check_mlstm(m: dict, where: str) -> None:
    sizes = [take(m, k, int, where=where) for k in ("heads", "dim", "vdim")]
    if min(sizes) <= 0 or take(m, "gate_cap", float, where=where) <= 0:
        raise ConfigError(f"{where}: heads, dim, vdim and gate_cap must be positive")


def _check_moe(mlp: dict, where: str) -> None:
    if take(mlp, "kind", str, where=where) != "moe":
        raise ConfigError(f"{where}: only kind 'moe' (or null) is known")
    r = _sub(mlp, "router", where)
    experts, top = take(r, "experts", int, where=where + ".router"), take(r, "top", int, where=where + ".router")
    identity = take(r, "identity", int, 0, where=where + ".router")
    n = experts + identity
    if experts <= 0 or identity < 0 or not 0 < top <= n:
        raise ConfigError(f"{where}.router: {experts} experts, {identity} identity experts, top {top}")
    g = r.get("groups") or {}
    count = take(g, "count", int, 1, where=where + ".router.groups")
    keep = take(g, "keep", int, count, where=where + ".router.groups")
    if count <= 0 or n % count or not 0 < keep <= count or keep * (n // count) < top:
        raise ConfigError(f"{where}.router.groups: {n} outputs in {count} groups of which {keep} are kept, top {top}")
    for key in ("expert",) + (("shared",) if mlp.get("shared") is not None else ()):
        e = _sub(mlp, key, where)
        if take(e, "ff", int, where=f"{where}.{key}") <= 0 or take(e, "limit", float, where=f"{where}.{key}") <= 0:
            raise ConfigError(f"{where}.{key}: ff and limit must be positive")


@dataclass(frozen=True)
class NomudraConfig(ModelConfig):
    layers_json: str = "[]"         # the ``layers`` list as canonical JSON (the dataclass stays hashable)
    norm_eps: float = 1e-6

    @property
    def layers(self) -> list:
        return json.loads(self.layers_json)

    @classmethod
    def from_json_dict(cls, raw: dict) -> "NomudraConfig":
        vocab, width = take(raw, "vocab", int), take(raw, "width", int)
        if vocab <= 0 or width <= 0:
            raise ConfigError("config.json: vocab and width must be positive")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        for i, layer in enumerate(layers):
            where = f"config.json: layers[{i}]"
            if not isinstance(layer, dict):
                raise ConfigError(f"{where} must be an object")
            kind = take(layer, "type", str, where=where)
            mixer = _sub(layer, "mixer", where)
            if kind == "attention":
                _check_attention(mixer, where + ".mixer")
            elif kind == "mlstm":
                _check_mlstm(mixer, where + ".mixer")
            else:
                raise ConfigError(f"{where}: unknown layer type {kind!r} (known: 'attention', 'mlstm')")
            if layer.get("mlp") is not None:
                if not isinstance(layer["mlp"], dict):
                    raise ConfigError(f"{where}.mlp must be an object or null")
                _check_moe(layer["mlp"], where + ".mlp")
        eos = raw.get("eos_token_id")
        return cls(
            architecture=ARCHITECTURE, model_type=take(raw, "model_type", str, "nomudra"), vocab_size=vocab,
            hidden_size=width, max_position_embeddings=take(raw, "max_position_embeddings", int, NO_POSITION_LIMIT),
            dtype=parse_dtype(raw.get("dtype", raw.get("torch_dtype", "bfloat16"))),
            eos_token_id=eos if isinstance(eos, int) and not isinstance(eos, bool) else None,
            layers_json=json.dumps(layers, sort_keys=True),
            norm_eps=take(_sub(raw, "norm", "config.json"), "eps", float))

    def to_json_dict(self) -> dict:
        return {"architecture": ARCHITECTURE, "vocab": self.vocab_size, "width": self.hidden_size,
                "norm": {"eps": self.norm_eps}, "layers": self.layers, "dtype": str(self.dtype).replace("torch.", ""),
                **({"eos_token_id": self.eos_token_id} if self.eos_token_id is not None else {})}


def _mixer(kind: str, m: dict, eps: float):
    if kind == "mlstm":
        return part("mlstm", num_heads=m["heads"], head_dim=m["dim"], v_head_dim=m["vdim"], gate_cap=float(m["gate_cap"]),
                    eps=eps)
    rot = m["rot"]
    rope = part("rope_banded", theta=float(rot["base"]), rotary_dim=int(rot["dims"]))
    mask = m.get("mask")
    return part("sink_attention", num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                v_head_dim=m["vdim"], scale=float(m["scale"]), position=rope, unit_norm_eps=None, sink=False,
                chunk=int(mask["size"]) if mask is not None else None, values="keys", bias=True, output_gate="sigmoid")


def _moe(mlp: dict):
    r, e, s = mlp["router"], mlp["expert"], mlp.get("shared")
    g = r.get("groups") or {}
    count = int(g.get("count", 1))
    shared = None
    if s is not None:
        shared = part("clamped_glu", intermediate_size=int(s["ff"]), limit=float(s["limit"]), alpha=EXPERT_ALPHA)
    return part("routed_moe", experts=int(r["experts"]), identity=int(r.get("identity", 0)), top=int(r["top"]),
                groups=count, keep=int(g.get("keep", count)), correction=True, intermediate_size=int(e["ff"]),
                limit=float(e["limit"]), alpha=EXPERT_ALPHA, shared=shared, shared_gate=shared is not None)


def build_spec(cfg: NomudraConfig) -> ModelSpec:
    """Nomudra as data: per layer a block that norms each sub-block's input and output, over a float32 stream."""
    def norm(name: str):
        return part("dyntanh", width=cfg.hidden_size, source=name)

    block = part("sandwich_residual")
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        uses = dict(mixer=PartUse(_mixer(layer["type"], layer["mixer"], cfg.norm_eps), p + "mix."),
                    mixer_norm=PartUse(norm("norm1"), p), mixer_post_norm=PartUse(norm("norm1b"), p))
        if layer.get("mlp") is not None:
            uses.update(ffn=PartUse(_moe(layer["mlp"]), p + "mlp."), ffn_norm=PartUse(norm("norm2"), p),
                        ffn_post_norm=PartUse(norm("norm2b"), p))
        layers.append(LayerSpec(block, **uses))
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
        max_position=cfg.max_position_embeddings,
        embedding=PartUse(part("token_embedding", vocab_size=cfg.vocab_size, stream="float32", source="embed",
                               norm=norm("embed.norm")), ""),
        layers=tuple(layers), order=tuple(LayerRun(i) for i in range(len(layers))),
        final_norm=PartUse(norm("final.norm"), ""),
        head=PartUse(part("lm_head", vocab_size=cfg.vocab_size, tied=False, exact=True, source="head"), ""))


register_architecture(ARCHITECTURE, model_types=("nomudra",), parse_config=NomudraConfig.from_json_dict,
                      build_spec=build_spec)
