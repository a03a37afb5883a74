"""Muvonex: a decoder-only model whose layers are listed one by one in config.json.

config.json: ``architecture`` "Muvonex"; ``vocab``, ``width``; ``embedding.scale``; ``norm.eps``; ``residual_mult``;
``layers``: a list of {``type``, ``mixer``, ``mlp``}.  Every layer is a parallel block: with h = norm1(x),
x <- x + residual_mult * (mixer(h) + mlp(h)), the stream x in float32, the norm an RMS norm whose weight is stored
as an offset from one.  Layer types:

* ``delta``: the gated delta rule (``mixer``: heads, kv_heads, dim, vdim, conv);
* ``parallel``: attention with a sink (``mixer.left``: heads, kv_heads, dim, vdim, scale, rot {base, dims, scaling
  {factor, low, high, original}}) beside a Mamba-2 mixer (``mixer.right``: heads, vdim, state, groups, conv,
  norm_groups), summed with ``left_scale`` and ``right_scale``.

``mlp`` is null or {``kind``: "dense", ``ff``}: down(gelu_tanh(gate h) * (up h)).  The logits are the last norm
(``final.norm``) times the embedding table itself, without its scale.  Tensors: ``embed``, ``final.norm``, and per
layer i ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.{gate,up,down}``.
"""
from __future__ import annotations

import json
from dataclasses import dataclass

from ..config.model_config import ConfigError, ModelConfig, parse_dtype, take
from ..config.registry import register_architecture
from ..parts.spec import LayerRun, LayerSpec, ModelSpec, PartUse, part

ARCHITECTURE = "Muvonex"
NO_POSITION_LIMIT = 1 << 20     # the design names no longest sequence; the engine's max_model_len is the limit in use


def _sub(raw: dict, key: str, where: str) -> dict:
    v = raw.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: key {key!r} must be an object")
    return v


def _check_delta(m: dict, where: str) -> None:
    heads, kv = take(m, "heads", int, where=where), take(m, "kv_heads", int, where=where)
    dim, vdim, conv = take(m, "dim", int, where=where), take(m, "vdim", int, where=where), take(m, "conv", int, where=where)
    if min(heads, kv, dim, vdim) <= 0 or heads % kv:
        raise ConfigError(f"{where}: heads {heads} must be a positive multiple of kv_heads {kv}, sizes positive")
    if not 1 <= conv <= 8:
        raise ConfigError(f"{where}: conv must be 1 to 8 taps, got {conv}")


def _check_parallel(m: dict, where: str) -> None:
    a, s = _sub(m, "left", where), _sub(m, "right", where)
    heads, kv = take(a, "heads", int, where=where + ".left"), take(a, "kv_heads", int, where=where + ".left")
    dim, vdim = take(a, "dim", int, where=where + ".left"), take(a, "vdim", int, where=where + ".left")
    take(a, "scale", float, where=where + ".left")
    if min(heads, kv, dim, vdim) <= 0 or heads % kv:
        raise ConfigError(f"{where}.left: heads {heads} must be a positive multiple of kv_heads {kv}, sizes positive")
    rot = _sub(a, "rot", where + ".left")
    dims = take(rot, "dims", int, where=where + ".left.rot")
    take(rot, "base", float, where=where + ".left.rot")
    if dims <= 0 or dims % 2 or dims > dim:
        raise ConfigError(f"{where}.left.rot: dims {dims} must be even and at most dim {dim}")
    if rot.get("scaling") is not None:
        for k in ("factor", "low", "high", "original"):
            take(rot["scaling"], k, float, where=where + ".left.rot.scaling")
    sh, sg = take(s, "heads", int, where=where + ".right"), take(s, "groups", int, 1, where=where + ".right")
    sp, sn = take(s, "vdim", int, where=where + ".right"), take(s, "state", int, where=where + ".right")
    ng, conv = take(s, "norm_groups", int, 1, where=where + ".right"), take(s, "conv", int, where=where + ".right")
    if min(sh, sg, sp, sn, ng) <= 0 or sh % sg or (sh * sp) % ng:
        raise ConfigError(f"{where}.right: heads {sh} must divide into groups {sg}, heads * vdim into norm_groups {ng}")
    if not 1 <= conv <= 8:
        raise ConfigError(f"{where}.right: conv must be 1 to 8 taps, got {conv}")
    take(m, "left_scale", float, 1.0, where=where)
    take(m, "right_scale", float, 1.0, where=where)


@dataclass(frozen=True)
class MuvonexConfig(ModelConfig):
    layers_json: str = "[]"         # the ``layers`` list as canonical JSON (the dataclass stays hashable)
    norm_eps: float = 1e-6
    residual_mult: float = 1.0
    embedding_scale: float = 1.0

    @property
    def layers(self) -> list:
        return json.loads(self.layers_json)

    @classmethod
    def from_json_dict(cls, raw: dict) -> "MuvonexConfig":
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
            if kind == "delta":
                _check_delta(mixer, where + ".mixer")
            elif kind == "parallel":
                _check_parallel(mixer, where + ".mixer")
            else:
                raise ConfigError(f"{where}: unknown layer type {kind!r} (known: 'delta', 'parallel')")
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or take(mlp, "kind", str, where=where + ".mlp") != "dense":
                    raise ConfigError(f"{where}.mlp: only kind 'dense' (or null) is known")
                if take(mlp, "ff", int, where=where + ".mlp") <= 0:
                    raise ConfigError(f"{where}.mlp: ff must be positive")
        eos = raw.get("eos_token_id")
        return cls(
            architecture=ARCHITECTURE, model_type=take(raw, "model_type", str, "muvonex"), vocab_size=vocab,
            hidden_size=width, max_position_embeddings=take(raw, "max_position_embeddings", int, NO_POSITION_LIMIT),
            dtype=parse_dtype(raw.get("dtype", raw.get("torch_dtype", "bfloat16"))),
            eos_token_id=eos if isinstance(eos, int) and not isinstance(eos, bool) else None,
            layers_json=json.dumps(layers, sort_keys=True),
            norm_eps=take(_sub(raw, "norm", "config.json"), "eps", float),
            residual_mult=take(raw, "residual_mult", float, 1.0),
            embedding_scale=take(raw.get("embedding") or {}, "scale", float, 1.0))

    def to_json_dict(self) -> dict:
        return {"architecture": ARCHITECTURE, "vocab": self.vocab_size, "width": self.hidden_size,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
                "residual_mult": self.residual_mult, "layers": self.layers,
                "dtype": str(self.dtype).replace("torch.", ""),
                **({"eos_token_id": self.eos_token_id} if self.eos_token_id is not None else {})}


def _mixer(kind: str, m: dict, eps: float):
    if kind == "delta":
        return part("gated_delta_rule", num_heads=m["heads"], num_qk_heads=m["kv_heads"], head_dim=m["dim"],
                    v_head_dim=m["vdim"], conv=m["conv"], eps=eps)
    a, s = m["left"], m["right"]
    rot = a["rot"]
    bands = {k: float(v) for k, v in (rot.get("scaling") or {}).items() if k in ("factor", "low", "high", "original")}
    rope = part("rope_banded", theta=float(rot["base"]), rotary_dim=int(rot["dims"]), **bands)
    left = part("sink_attention", num_heads=a["heads"], num_kv_heads=a["kv_heads"], head_dim=a["dim"],
                v_head_dim=a["vdim"], scale=float(a["scale"]), position=rope, unit_norm_eps=eps, sink=True)
    right = part("mamba2", num_heads=s["heads"], head_dim=s["vdim"], state_size=s["state"], groups=s.get("groups", 1),
                 conv=s["conv"], norm_groups=s.get("norm_groups", 1), eps=eps)
    return part("parallel_mixers", left=left, right=right, left_scale=float(m.get("left_scale", 1.0)),
                right_scale=float(m.get("right_scale", 1.0)))


def build_spec(cfg: MuvonexConfig) -> ModelSpec:
    """Muvonex as data: per layer a parallel block (one norm, mixer and feed-forward side by side, float32 stream)."""
    block = part("parallel_residual", residual_mult=cfg.residual_mult)
    layers = []
    for i, layer in enumerate(cfg.layers):
        uses = dict(mixer=PartUse(_mixer(layer["type"], layer["mixer"], cfg.norm_eps), f"l{i}.mix."),
                    norm=PartUse(part("rmsnorm", width=cfg.hidden_size, eps=cfg.norm_eps, weight_offset=1.0,
                                      source="norm1"), f"l{i}."))
        if layer.get("mlp") is not None:
            uses["ffn"] = PartUse(part("gated_mlp", intermediate_size=layer["mlp"]["ff"], activation="gelu_tanh"),
                                  f"l{i}.mlp.")
        layers.append(LayerSpec(block, **uses))
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
        max_position=cfg.max_position_embeddings,
        embedding=PartUse(part("token_embedding", vocab_size=cfg.vocab_size, scale=cfg.embedding_scale,
                               stream="float32", source="embed"), ""),
        layers=tuple(layers), order=tuple(LayerRun(i) for i in range(len(layers))),
        final_norm=PartUse(part("rmsnorm", width=cfg.hidden_size, eps=cfg.norm_eps, weight_offset=1.0, source="norm"),
                           "final."),
        head=PartUse(part("lm_head", vocab_size=cfg.vocab_size, tied=True, exact=True), "head."))


register_architecture(ARCHITECTURE, model_types=("muvonex",), parse_config=MuvonexConfig.from_json_dict,
                      build_spec=build_spec)
