"""Nomudra on the CPU: its config.json keys and their checks, the tensor table against the design's tensor names, and
the cache manager's handling of chunked attention (pages behind the current chunk go back to the pool)."""
import copy

import pytest
import torch

import plain_nomudra as pn
from nanohybrid_vlm_b200.cache.manager import CacheManager, GroupSpec
from nanohybrid_vlm_b200.config.model_config import ConfigError
from nanohybrid_vlm_b200.config.registry import ARCHITECTURES
from nanohybrid_vlm_b200.engine.model import CausalLM
from nanohybrid_vlm_b200.parts.base import FixedStateNeed, PagedKVNeed

CFG = dict(architecture="Nomudra", vocab=120, width=64, norm=dict(eps=1e-5), layers=[
    dict(type="mlstm", mixer=dict(heads=2, dim=12, vdim=20, gate_cap=12.0), mlp=None),
    dict(type="attention", mixer=dict(heads=4, kv_heads=2, dim=16, vdim=16, scale=0.25, rot=dict(base=10000.0, dims=8),
                                      mask=dict(size=40)),
         mlp=dict(kind="moe", router=dict(experts=5, identity=1, top=2, groups=dict(count=3, keep=2)),
                  expert=dict(ff=24, limit=1.5), shared=dict(ff=32, limit=2.0))),
])


def build(cfg):
    import nanohybrid_vlm_b200.models  # noqa: F401
    entry = ARCHITECTURES.resolve(cfg)
    parsed = entry.parse_config(cfg)
    return parsed, entry.build_spec(parsed)


def test_tensor_table_names_and_shapes_are_the_designs():
    parsed, spec = build(CFG)
    model = CausalLM(spec, torch.bfloat16, "cpu")
    got = {}
    for bp in model.param_table():
        for src in bp.decl.sources:
            got[src.name] = tuple(src.checkpoint_shape(bp.decl.shape))
    assert got == {k: tuple(v) for k, v in pn.tensor_shapes(CFG).items()}
    assert parsed.to_json_dict()["layers"] == CFG["layers"]


def test_cache_needs_follow_the_layers():
    _, spec = build(CFG)
    needs = CausalLM(spec, torch.float32, "cpu").cache_needs()
    assert isinstance(needs[0], FixedStateNeed) and needs[0].dtype == "float32"
    assert needs[1] == PagedKVNeed(2, 16, None, v_head_dim=16, chunk=40)


@pytest.mark.parametrize("path,value,words", [
    (("layers", 1, "mixer", "vdim"), 8, "vdim"),
    (("layers", 1, "mixer", "rot", "dims"), 7, "dims"),
    (("layers", 1, "mixer", "kv_heads"), 3, "kv_heads"),
    (("layers", 1, "mixer", "mask", "size"), 0, "size"),
    (("layers", 1, "mlp", "router", "top"), 7, "top"),
    (("layers", 1, "mlp", "router", "groups", "count"), 4, "groups"),
    (("layers", 1, "mlp", "router", "groups", "keep"), 1, "groups"),       # with top raised to 3 below: one kept group of two
    (("layers", 1, "mlp", "kind"), "dense", "moe"),
    (("layers", 0, "mixer", "gate_cap"), 0.0, "gate_cap"),
    (("layers", 0, "type"), "conv", "unknown layer type"),
    (("width",), 0, "positive"),
])
def test_bad_values_are_refused(path, value, words):
    cfg = copy.deepcopy(CFG)
    at = cfg
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    if path[-1] == "keep":
        cfg["layers"][1]["mlp"]["router"]["top"] = 3        # three outputs from one kept group of two
    with pytest.raises(ConfigError, match=words):
        build(cfg)


def test_optional_keys():
    cfg = copy.deepcopy(CFG)
    cfg["layers"][1]["mixer"]["mask"] = None                  # no chunks: plain causal attention, nothing given back
    del cfg["layers"][1]["mlp"]["router"]["groups"]
    cfg["layers"][1]["mlp"]["router"]["identity"] = 0
    cfg["layers"][1]["mlp"]["shared"] = None
    _, spec = build(cfg)
    model = CausalLM(spec, torch.float32, "cpu")
    assert model.cache_needs()[1].chunk is None
    names = {s.name for bp in model.param_table() for s in bp.decl.sources}
    assert "l1.mlp.shared.sg" not in names and "l1.mlp.router" in names


def test_pages_behind_the_current_chunk_go_back():
    """Chunks of 40 positions, pages of 16: once position 40 is the next to be computed, no query reads pages 0 and 1
    again (page 2 holds positions 32 to 47); after position 80, pages 0 to 4."""
    cm = CacheManager([GroupSpec(None, chunk=40)], page_size=16, num_pages=8)
    assert cm.has_windows and not CacheManager.prefix_cache_possible(cm.groups, 0)
    cm.allocate("a", 39)
    assert cm.release_behind_window("a", 39) == 0
    cm.allocate("a", 41)
    assert cm.release_behind_window("a", 40) == 2
    assert cm.block_table("a")[:2] == [-1, -1] and cm.block_table("a")[2] >= 0
    cm.allocate("a", 90)
    assert cm.release_behind_window("a", 85) == 3              # pages 2, 3 and 4: the chunk of position 85 starts at 80
    cm.allocate("b", 32)                                       # the pool of 8 has room again
    cm.check()
    cm.free("a")
    cm.free("b")
    cm.check()
    # a window and a chunk together: the later of the two bounds decides
    both = CacheManager([GroupSpec(20, chunk=64)], page_size=8, num_pages=16)
    both.allocate("c", 70)
    assert both.release_behind_window("c", 70) == 8            # chunk start 64 is later than 70 - 20 + 1
    both.check()
