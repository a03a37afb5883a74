"""Muvonex without a GPU: config.json parsing and its errors, the model as data (parts per layer), the tensors it
asks a checkpoint for, and what its layers ask of the cache manager."""
import copy

import pytest
import torch

import plain_muvonex as pm
import nanohybrid_vlm_b200.models  # noqa: F401  (registers the architectures)
from nanohybrid_vlm_b200.cache import CacheLayout
from nanohybrid_vlm_b200.config.model_config import ConfigError
from nanohybrid_vlm_b200.config.registry import ARCHITECTURES
from nanohybrid_vlm_b200.engine.model import CausalLM
from nanohybrid_vlm_b200.parts import CompositeNeed, FixedStateNeed, PagedKVNeed

CFG = dict(
    architecture="Muvonex", vocab=90, width=48, embedding=dict(scale=2.0), norm=dict(eps=1e-5), residual_mult=0.25,
    layers=[
        dict(type="delta", mlp=None, mixer=dict(heads=4, kv_heads=2, dim=8, vdim=12, conv=3)),
        dict(type="parallel", mlp=dict(kind="dense", ff=56), mixer=dict(
            left=dict(heads=3, kv_heads=1, dim=16, vdim=20, scale=0.3, rot=dict(base=100.0, dims=8, scaling=None)),
            right=dict(heads=2, groups=2, state=6, vdim=10, conv=2, norm_groups=2), left_scale=0.5, right_scale=2.0)),
    ])


def build(raw):
    entry = ARCHITECTURES.resolve(raw)
    return entry, entry.parse_config(raw)


def test_registry_and_spec():
    entry, cfg = build(CFG)
    assert cfg.vocab_size == 90 and cfg.hidden_size == 48 and cfg.residual_mult == 0.25 and cfg.embedding_scale == 2.0
    spec = entry.build_spec(cfg)
    assert [l.block.kind for l in spec.layers] == ["parallel_residual"] * 2
    assert spec.layers[0].mixer.spec.kind == "gated_delta_rule" and "ffn" not in dict(spec.layers[0].parts)
    assert dict(spec.layers[1].parts)["ffn"].spec["activation"] == "gelu_tanh"
    mixer = spec.layers[1].mixer.spec
    assert mixer.kind == "parallel_mixers" and mixer["left"].kind == "sink_attention" and mixer["right"].kind == "mamba2"
    assert mixer["left_scale"] == 0.5 and mixer["right_scale"] == 2.0
    assert entry.parse_config(cfg.to_json_dict()) == cfg


def test_checkpoint_names_and_shapes():
    entry, cfg = build(CFG)
    model = CausalLM(entry.build_spec(cfg), torch.bfloat16, "cpu")
    asked = {}
    for bp in model.param_table():
        for src in bp.decl.sources:
            asked[src.name] = tuple(src.checkpoint_shape(bp.decl.shape))
    assert asked == pm.tensor_shapes(CFG)


def test_cache_needs():
    entry, cfg = build(CFG)
    model = CausalLM(entry.build_spec(cfg), torch.bfloat16, "cpu")
    layout = CacheLayout.from_needs(model.cache_needs())
    d, p = layout.needs
    assert d == CompositeNeed((FixedStateNeed((2 * (2 * 2 * 8 + 4 * 12),)), FixedStateNeed((4 * 12 * 8,))))
    assert p == CompositeNeed((PagedKVNeed(1, 16, None, v_head_dim=20),
                               CompositeNeed((FixedStateNeed((1 * (2 * 10 + 2 * 2 * 6),)), FixedStateNeed((2 * 10 * 6,))))))
    assert layout.needs_state_slots and len(layout.groups) == 1 and layout.run_group == [None, 0]
    assert layout.page_bytes(16, torch.bfloat16) == [2 * 1 * 16 * 20 * 2]
    assert layout.state_bytes_per_slot(torch.bfloat16) == 4 * (160 + 384 + 44 + 120)


@pytest.mark.parametrize("change,words", [
    (lambda c: c["layers"][0].update(type="gru"), "unknown layer type"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"].update(conv=9), "conv must be 1 to 8"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=18), "dims"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(groups=3), "groups"),
    (lambda c: c["layers"][1]["mlp"].update(kind="experts"), "dense"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.update(layers=[]), "layers"),
    (lambda c: c["layers"][1]["mixer"]["left"].pop("scale"), "scale"),
])
def test_config_errors(change, words):
    raw = copy.deepcopy(CFG)
    change(raw)
    with pytest.raises(ConfigError, match=words):
        build(raw)


def test_plain_model_carries_its_states():
    """The plain recurrences started from a handed-on state give what one pass over all tokens gives."""
    g = torch.Generator().manual_seed(0)
    T, G, H, d, dv = 12, 2, 4, 6, 5
    q, k = torch.randn(T, G, d, generator=g, dtype=torch.float64), torch.randn(T, G, d, generator=g, dtype=torch.float64)
    v, beta = torch.randn(T, H, dv, generator=g, dtype=torch.float64), torch.rand(T, H, generator=g, dtype=torch.float64)
    decay = torch.rand(T, H, generator=g, dtype=torch.float64)
    whole = pm.delta_recurrence(q, k, v, beta, decay)
    a, S = pm.delta_recurrence(q[:5], k[:5], v[:5], beta[:5], decay[:5], torch.zeros(H, d, dv, dtype=torch.float64))
    b, _ = pm.delta_recurrence(q[5:], k[5:], v[5:], beta[5:], decay[5:], S)
    torch.testing.assert_close(torch.cat([a, b]), whole)


def test_random_weights_folder(tmp_path):
    """The random-weights mode writes every tensor the design names, under its checkpoint name and shape, and the
    plain model runs on the folder."""
    from safetensors.torch import load_file
    from nanohybrid_vlm_b200.weights import write_random_model
    write_random_model(str(tmp_path), dict(CFG, dtype="bfloat16"), seed=3)
    tensors = load_file(str(tmp_path / "model.safetensors"))
    assert {k: tuple(v.shape) for k, v in tensors.items()} == pm.tensor_shapes(CFG)
    logits = pm.forward(CFG, {k: v.to(torch.float64) for k, v in tensors.items()}, [1, 2, 3, 4])
    assert logits.shape == (4, CFG["vocab"]) and torch.isfinite(logits).all()
