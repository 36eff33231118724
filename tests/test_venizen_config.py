"""Venizen without a GPU: its configuration checks, its plan (layers, the order
in which they run, tensor names and shapes), the random-weights writer, and the
cache manager's rule for a window that keeps the first tokens."""
import copy
import json
import os

import pytest
import torch

from kipp_b200.cache import CacheManager
from kipp_b200.config import config_from_dict
from kipp_b200.config.base import ConfigError
from kipp_b200.config.registry import get_architecture
from kipp_b200.parts.base import PagedKVSpec
from venizen_util import CONFIGS, INIT, write_folder

import plain_venizen as P


def spec_of(cfg):
    c = config_from_dict(cfg)
    return get_architecture(c.architecture).build(c)


def test_the_model_class_is_chosen_by_the_architecture_key():
    c = config_from_dict(CONFIGS["P"])
    assert c.architecture == "Venizen" and c.to_dict()["layers"][0]["type"] == "general_delta"
    assert config_from_dict(c.to_dict()).to_dict() == c.to_dict()


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_runs_follow_the_loop_with_a_cache_each(name):
    cfg = CONFIGS[name]
    plan = spec_of(cfg).plan
    runs = [(o["layer"], bool(o["adds_embedding"])) for o in plan["order"]]
    assert runs == P.layer_runs(cfg)
    assert [o["cache"] for o in plan["order"]] == list(range(len(runs)))       # every run its own cache and state


def test_tensor_names_and_shapes():
    specs = {s.name: tuple(s.shape) for s in spec_of(CONFIGS["P"]).tensor_specs()}
    assert specs["embed"] == (300, 64) and specs["head"] == (300, 64) and specs["final.norm"] == (64,)
    assert specs["l0.mix.w1"] == (8, 64) and specs["l0.mix.w2"] == (32, 8) and specs["l0.mix.a.b"] == (32,)
    assert specs["l1.mix.left.q"] == (64, 64) and specs["l1.mix.left.v"] == (96, 64)      # value heads of 24
    assert specs["l1.mix.left.o"] == (64, 96) and specs["l1.mix.left.talk"] == (4, 4)
    assert specs["l1.mix.left.q.norm"] == (16,) and specs["l1.mix.right.g"] == (24, 64)
    assert specs["l2.mix.left.k"] == (32, 64) and specs["l2.mlp.act"] == (4,) and specs["l2.mlp.up"] == (72, 64)
    assert "l1.norm2" not in specs and "l1.mlp.up" not in specs                            # a layer without a feed-forward
    assert "l0.norm2" in specs


def test_the_width_of_the_decay_bottleneck_may_be_left_to_the_tensor():
    cfg = copy.deepcopy(CONFIGS["P"])
    del cfg["layers"][0]["mixer"]["decay_rank"]
    specs = {s.name: tuple(s.shape) for s in spec_of(cfg).tensor_specs()}
    assert specs["l0.mix.w1"] == (-1, 64) and specs["l0.mix.w2"] == (32, -1)


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(decay=[0.5]), "one decay per head"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c["layers"][2]["mlp"].update(kind="routed"), "not supported"),
])
def test_bad_configurations_are_refused_by_name(change, message):
    cfg = copy.deepcopy(CONFIGS["P"])
    change(cfg)
    with pytest.raises((ConfigError, ValueError, RuntimeError), match=message):
        config_from_dict(cfg)


def test_random_weights_folder_holds_what_the_plan_declares(tmp_path):
    folder = write_folder(str(tmp_path / "m"), CONFIGS["Q"], INIT["Q"])
    from tiny import read_weights
    w = read_weights(folder)
    specs = {s.name: tuple(s.shape) for s in spec_of(CONFIGS["Q"]).tensor_specs()}
    assert {k: tuple(v.shape) for k, v in w.items()} == specs
    assert json.load(open(os.path.join(folder, "config.json")))["architecture"] == "Venizen"
    talk = w["l0.mix.left.talk"]
    assert torch.allclose(talk.diagonal(), torch.ones(2), atol=0.5) and talk.abs().sum() > 0


def test_plain_model_is_causal_and_its_window_keeps_the_first_tokens():
    assert P.visible(6, 2, 1).int().tolist() == [[1, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0],
                                                 [1, 0, 1, 1, 0, 0], [1, 0, 0, 1, 1, 0], [1, 0, 0, 0, 1, 1]]
    assert P.visible(4, 0, 0).int().tolist() == [[1, 0, 0, 0], [1, 1, 0, 0], [1, 1, 1, 0], [1, 1, 1, 1]]


def test_a_window_group_keeps_the_pages_of_the_first_tokens():
    spec = PagedKVSpec(2, 16, window=8, keep_first=5)            # pages of 4: positions 0..4 live in pages 0 and 1
    plain = PagedKVSpec(2, 16, window=8)
    cm = CacheManager({0: spec, 1: plain}, page_size=4, pages_per_group=16, max_requests=2)
    cm.admit("a")
    at = 0
    for n in (3, 6, 1, 1, 9, 2, 30):
        cm.reserve([("a", at + n)])
        at += n
        cm.advance("a", at)
        cm.check()
    kept, gone = cm.table("a", 0), cm.table("a", 1)
    first_needed = (at - 8 + 1) // 4
    assert all(p >= 0 for p in kept[:2]) and all(p < 0 for p in kept[2:first_needed])
    assert all(p < 0 for p in gone[:first_needed]) and all(p >= 0 for p in gone[first_needed:])
    assert cm.pages_held("a")[0] == cm.pages_held("a")[1] + 2
    cm.release("a")
    cm.check()
    assert cm.groups[0].pool.free_pages == 16 and cm.groups[1].pool.free_pages == 16
