"""Mozepel without a GPU: its configuration, its model description, and the cache groups it needs (pages that a
window gives back beside pages of pooled entries, one per block of positions)."""
import copy

import pytest
import torch

from aegean_tge_b200 import ConfigError, architecture_of
from aegean_tge_b200.cache import CacheManager, PoolExhausted
from aegean_tge_b200.config.model_spec import expected_tensors
from aegean_tge_b200.parts.base import PagedCacheSpec, StateSpec

RETENTION = {"type": "retention", "mlp": {"kind": "dense", "ff": 40},
             "mixer": {"heads": 2, "dim": 8, "vdim": 12, "decay": [0.9, 0.99], "rot": {"base": 100.0, "dims": 4}}}
PARALLEL = {"type": "parallel", "mlp": None,
            "mixer": {"left_scale": 0.8, "right_scale": 1.2,
                      "left": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "scale": 0.3, "conv": 3, "mask": {"size": 10, "pool": 4},
                               "rot": {"base": 50.0, "dims": 8, "scaling": {"factor": 2.0, "low": 1.0, "high": 2.0, "original": 16}}},
                      "right": {"heads": 3, "dim": 4, "vdim": 8, "decay": [0.5, 0.7, 1.0]}}}
CONFIG = {"architecture": "Mozepel", "vocab": 50, "width": 24, "norm": {"eps": 1e-5}, "postln_alpha": 2.5,
          "layers": [RETENTION, PARALLEL, dict(RETENTION, weights_of=0), dict(PARALLEL, weights_of=1)]}


def _parse(raw):
    arch = architecture_of(raw)
    return arch, arch.parse_config(raw)


def test_config_round_trip_and_description():
    arch, config = _parse(CONFIG)
    assert config.to_dict() == CONFIG
    spec = arch.build_spec(config)
    spec.validate()
    assert [layer.weights_from for layer in spec.layers] == [None, None, 0, 1]
    assert [layer.block for layer in spec.layers] == ["post_norm"] * 4
    assert spec.layers[1].feed_forward is None and spec.layers[1].ffn_norm.params["optional"]
    names = set(expected_tensors(spec))
    assert "l1.mix.left.q.conv" in names and "l1.mix.right.norm" in names and "l0.mix.g" in names and "l0.norm2" in names
    assert not any(name.startswith(("l2.", "l3.")) for name in names)
    planned = {name: shape for name, shape, _role, _draw in arch.random_plan(config)}
    assert set(planned) == names - {"l1.norm2"}         # a layer without feed-forward may, but need not, bring a second norm
    assert planned["l1.mix.left.v.conv"] == (12, 3) and planned["l1.mix.left.o"] == (24, 24) and planned["l0.mix.v"] == (24, 24)


@pytest.mark.parametrize("path,value", [
    (("layers", 0, "type"), "attention"), (("layers", 0, "mixer", "decay"), [0.9]), (("layers", 0, "mixer", "decay"), [0.9, 1.5]),
    (("layers", 0, "mixer", "rot", "dims"), 5), (("layers", 0, "mixer", "rot", "dims"), 10), (("layers", 1, "mixer", "left", "kv_heads"), 3),
    (("layers", 1, "mixer", "left", "mask"), None), (("layers", 1, "mixer", "left", "conv"), 17), (("layers", 2, "weights_of"), 2),
    (("layers", 3, "weights_of"), 2), (("layers", 2, "mlp"), None), (("layers", 1, "mlp"), {"kind": "routed", "ff": 8}),
    (("postln_alpha",), None), (("norm",), {}), (("layers", 1, "mixer", "left", "rot", "scaling", "high"), 0.5)])
def test_config_errors_name_the_key(path, value):
    raw = copy.deepcopy(CONFIG)
    at = raw
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError) as error:
        _parse(raw)
    assert str(path[-1]) in str(error.value) or "layer" in str(error.value)


def test_what_a_model_may_leave_out():
    raw = copy.deepcopy(CONFIG)
    raw["layers"] = [copy.deepcopy(PARALLEL), copy.deepcopy(RETENTION)]
    left = raw["layers"][0]["mixer"]["left"]
    del left["conv"], left["mask"]["pool"], left["rot"]["scaling"]
    del raw["layers"][1]["mixer"]["rot"]
    arch, config = _parse(raw)
    assert config.layers[0].mixer.left.conv == 0 and config.layers[0].mixer.left.pool == 0 and config.layers[1].mixer.rot is None
    assert config.to_dict() == raw
    names = set(expected_tensors(arch.build_spec(config)))
    assert "l0.mix.left.q.conv" not in names and "l0.mix.left.q.norm" in names


TOKENS = PagedCacheSpec((("k", (2, 8)), ("v", (2, 6))), 10)
POOLED = PagedCacheSpec((("k", (2, 8)), ("v", (2, 6))), None, stride=4)


def _manager(pages=(6, 3), slots=3):
    m = CacheManager(4, slots)
    m.add_layer(0, TOKENS, StateSpec((("conv", (2, 5)),)), extra={"pooled": POOLED})
    m.add_layer(1, None, StateSpec((("state", (2, 3, 3)),)))
    m.add_layer(2, TOKENS, None, extra={"pooled": POOLED})
    m.set_pool_sizes(list(pages))
    return m


def test_pooled_entries_take_a_page_per_block_of_blocks():
    m = _manager()
    assert len(m.groups) == 2 and m.groups[1].spec.stride == 4 and m.groups[0].layers == [0, 2]
    m.allocate_storage(torch.float32, torch.device("cpu"))
    view = m.layer_cache(2)
    assert view.paged["k"].shape == (7, 2, 4, 8) and view.more["pooled"].paged["v"].shape == (4, 2, 4, 6)
    assert view.more["pooled"].group == 1 and view.group == 0
    assert view.more["pooled"].paged["k"].data_ptr() != m.layer_cache(0).more["pooled"].paged["k"].data_ptr()
    m.admit("a")
    assert m.pages_missing("a", 3) == [1, 0]                 # no whole block yet
    assert m.pages_missing("a", 4) == [1, 1]
    assert m.pages_missing("a", 19) == [5, 1]                # four blocks: one page of entries
    assert m.pages_missing("a", 20) == [5, 2]                # the fifth block starts the second page
    m.grow("a", 20)
    assert len(m.groups[1].tables["a"]) == 2 and len(m.groups[0].tables["a"]) == 5
    m.set_computed("a", 20)
    # the window (10 tokens) gives back the tokens' pages before position 11; the pooled entries stay
    assert m.groups[0].tables["a"][:2] == [-1, -1] and -1 not in m.groups[0].tables["a"][2:]
    assert -1 not in m.groups[1].tables["a"]
    m.admit("b")
    assert m.can_grow("b", 12) and not m.can_grow("b", 13)   # three token pages are free, a fourth is not
    m.free("a")
    assert m.can_grow("b", 24) and not m.can_grow("b", 25)
    assert m.fits_empty_pool(24) and not m.fits_empty_pool(25)
    m.check()


def test_pages_and_slots_come_back_and_are_used_again():
    m = _manager(pages=(6, 3), slots=2)
    m.allocate_storage(torch.float32, torch.device("cpu"))
    seen_pages, seen_slots = set(), set()
    for round_ in range(5):
        a, b = f"a{round_}", f"b{round_}"
        slot = m.admit(a)
        m.state_storage[0]["conv"][slot] += 1.0
        seen_slots.add(slot)
        seen_slots.add(m.admit(b))
        with pytest.raises(PoolExhausted):
            m.admit("c")
        m.grow(a, 9)
        m.grow(b, 12)
        seen_pages.update(m.groups[0].tables[a] + m.groups[0].tables[b])
        assert m.groups[0].pool.free_count == 0 and not m.can_grow(a, 13)
        m.free(a)
        m.free(b)
        m.check()
    assert seen_slots == {0, 1} and len(seen_pages) == 6
    assert float(m.state_storage[0]["conv"].abs().max()) == 1.0      # a slot is zeroed for each request that takes it


def test_pool_sizes_for_a_token_count():
    m = _manager()
    assert m.plan_pool_sizes(tokens=64) == [16, 4 + 3]          # 64 tokens in pages of 4; 16 blocks in pages of 4, a partly filled page per request
