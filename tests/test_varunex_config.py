"""Varunex without a GPU: its configuration checks, its plan (the parts of every
layer and their parameters, tensor names and shapes), the random-weights writer,
and properties of the plain model that the GPU tests lean on."""
import copy
import json
import math
import os

import pytest
import torch

from kipp_b200.config import config_from_dict
from kipp_b200.config.base import ConfigError
from kipp_b200.config.registry import get_architecture
from varunex_util import CONFIGS, INIT, write_folder

import plain_varunex as P


def spec_of(cfg):
    c = config_from_dict(cfg)
    return get_architecture(c.architecture).build(c)


def test_the_model_class_is_chosen_by_the_architecture_key():
    c = config_from_dict(CONFIGS["A"])
    assert c.architecture == "Varunex" and c.to_dict()["layers"][0]["type"] == "latent_attention"
    assert config_from_dict(c.to_dict()).to_dict() == c.to_dict()
    assert c.vocab_size == 300 and c.hidden_size == 64


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_every_layer_is_a_block_with_one_norm_and_its_own_cache(name):
    cfg = CONFIGS[name]
    plan = spec_of(cfg).plan
    kinds = {"mlstm": "gated_memory", "latent_attention": "latent_attention", "attention": "attention"}
    assert [o["layer"] for o in plan["order"]] == list(range(len(cfg["layers"])))
    assert [o["cache"] for o in plan["order"]] == list(range(len(cfg["layers"])))
    for layer, block in zip(cfg["layers"], plan["layers"]):
        part = block["part"]
        assert part["kind"] == "parallel_block" and part["norm"]["kind"] == "layernorm"
        assert part["mixer"]["kind"] == kinds[layer["type"]]
        assert (part["ffn"] is None) == (layer["mlp"] is None)
        if layer["mlp"]:
            assert part["ffn"]["activation"] == "relu_squared" and part["ffn"]["intermediate_size"] == layer["mlp"]["ff"]
    assert plan["final_norm"]["part"]["kind"] == "layernorm"


def test_the_mixers_take_their_constants_from_the_configuration():
    plan = spec_of(CONFIGS["A"]).plan
    latent, diff, memory, plain_diff = (plan["layers"][i]["part"]["mixer"] for i in (0, 1, 2, 3))
    assert latent["kv_rank"] == 32 and latent["q_rank"] == 40 and latent["rot_dim"] == 8 and latent["value_dim"] == 24
    assert latent["sink"] is True and latent["gate"] == "sigmoid" and latent["position"]["rotary_dim"] == 8
    assert diff["score_maps"] == 2 and diff["combine_maps"] is True and diff["bias"] is True and diff["window"] == 20
    assert diff["lambda_init"] == 0.3 and diff["num_kv_heads"] == 2 and diff["position"]["kind"] == "stretched_rotary"
    assert diff["position"]["factor"] == 8.0 and diff["position"]["original"] == 64
    assert plain_diff["window"] == 0 and plain_diff["position"]["kind"] == "rotary"
    assert memory["gate_cap"] == 10.0 and memory["value_dim"] == 40 and memory["head_dim"] == 16


def test_tensor_names_and_shapes():
    specs = {s.name: tuple(s.shape) for s in spec_of(CONFIGS["A"]).tensor_specs()}
    assert specs["embed"] == (300, 64) and specs["head"] == (300, 64)
    assert specs["final.norm"] == (64,) and specs["final.norm.b"] == (64,) and specs["l3.norm1.b"] == (64,)
    assert specs["l0.mix.dq"] == (40, 64) and specs["l0.mix.dq.norm"] == (40,) and specs["l0.mix.uq"] == (4 * 24, 40)
    assert specs["l0.mix.dkv"] == (40, 64) and specs["l0.mix.dkv.norm"] == (32,) and specs["l0.mix.uk"] == (64, 32)
    assert specs["l0.mix.uv"] == (96, 32) and specs["l0.mix.sink"] == (4,) and specs["l0.mix.g"] == (4, 64)
    assert specs["l0.mix.o"] == (64, 96)
    assert specs["l1.mix.q"] == (4 * 2 * 16, 64) and specs["l1.mix.k"] == (2 * 2 * 16, 64) and specs["l1.mix.v"] == (48, 64)
    assert specs["l1.mix.q.b"] == (128,) and specs["l1.mix.lq1"] == (16,) and specs["l1.mix.o"] == (64, 96)
    assert specs["l2.mix.q"] == (32, 64) and specs["l2.mix.v"] == (80, 64) and specs["l2.mix.i"] == (2, 64)
    assert specs["l2.mix.f.b"] == (2,) and specs["l2.mix.norm"] == (80,) and specs["l2.mix.g"] == (80, 64)
    assert "l1.mlp.up" not in specs and specs["l2.mlp.up"] == (72, 64) and specs["l2.mlp.down"] == (64, 72)
    assert not any(k.endswith("norm2") for k in specs)


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=4), "rot_dim"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].pop("low"), "low"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18), "at most"),
    (lambda c: c["layers"][2]["mixer"].update(gate_cap=0), "gate_cap"),
    (lambda c: c["layers"][1]["mixer"].pop("diff"), "diff"),
    (lambda c: c["layers"][2]["mlp"].update(kind="routed"), "not supported"),
])
def test_bad_configurations_are_refused_by_name(change, message):
    cfg = copy.deepcopy(CONFIGS["A"])
    change(cfg)
    with pytest.raises((ConfigError, ValueError, RuntimeError), match=message):
        config_from_dict(cfg)


def test_random_weights_folder_holds_what_the_plan_declares(tmp_path):
    folder = write_folder(str(tmp_path / "m"), CONFIGS["B"], INIT["B"])
    from tiny import read_weights
    w = read_weights(folder)
    specs = {s.name: tuple(s.shape) for s in spec_of(CONFIGS["B"]).tensor_specs()}
    assert {k: tuple(v.shape) for k, v in w.items()} == specs
    assert json.load(open(os.path.join(folder, "config.json")))["architecture"] == "Varunex"
    assert torch.allclose(w["l0.norm1"], torch.ones(100), atol=0.11) and w["l0.norm1.b"].abs().sum() > 0


def test_stretched_wavelengths_have_three_zones():
    rot = {"base": 10000.0, "dims": 16, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}
    plain = P.frequencies({"base": 10000.0, "dims": 16})
    got = P.frequencies(rot)
    wave = 2 * math.pi / plain
    assert torch.equal(got[wave < 16], plain[wave < 16]) and (wave < 16).any()
    assert torch.allclose(got[wave > 64], plain[wave > 64] / 8.0) and (wave > 64).any()
    mid = (wave >= 16) & (wave <= 64)
    assert mid.any() and ((got[mid] < plain[mid]) & (got[mid] > plain[mid] / 8.0)).all()


def test_the_plain_memory_starts_its_running_maximum_at_zero():
    """With gates far below zero the state takes e^(i - 0): a maximum that started
    at minus infinity would take 1 instead."""
    torch.manual_seed(0)
    W, H, D = 8, 1, 4
    m = {"heads": H, "dim": D, "vdim": D, "gate_cap": 15.0}
    w = {"q": torch.randn(D, W), "k": torch.randn(D, W), "v": torch.randn(D, W), "g": torch.zeros(D, W), "o": torch.eye(W, D),
         "norm": torch.ones(D), "i": torch.zeros(H, W), "i.b": torch.full((H,), -6.0), "f": torch.zeros(H, W),
         "f.b": torch.full((H,), 8.0)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(1, W, dtype=torch.float64)
    q, k, v = (w["q"] @ h[0]) * D ** -0.5, w["k"] @ h[0], w["v"] @ h[0]
    take = math.exp(15.0 * math.tanh(-6.0 / 15.0))
    o = take * v * (k @ q) / (max(abs(take * (k @ q)), 1.0) + 1e-6)
    want = (o / torch.sqrt((o * o).mean() + 1e-5)) * 0.5
    assert torch.allclose(P.mlstm(w, "", m, h, 1e-5)[0, :D], want, atol=1e-12)


def test_the_plain_attentions_are_causal():
    cfg = CONFIGS["D"]
    from tiny import read_weights
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        w = read_weights(write_folder(os.path.join(tmp, "m"), cfg, INIT["D"]))
    toks = list(range(20))
    full = P.forward(cfg, w, toks)
    assert torch.allclose(P.forward(cfg, w, toks[:9]), full[:9], atol=1e-12)
    assert P.causal(4, 2).int().tolist() == [[1, 0, 0, 0], [1, 1, 0, 0], [0, 1, 1, 0], [0, 0, 1, 1]]


def test_the_parts_can_be_described_from_python_for_another_design():
    """A model put together in Python from the descriptions of the same parts gives
    the plan the library's own builder makes (apart from the configuration kept in it)."""
    from kipp_b200.models.spec import LayerRun, ModelSpec
    from kipp_b200.parts import (AttentionMixer, DenseFeedForward, GatedMemoryMixer, LatentAttentionMixer, LayerNorm,
                                 OutputHead, ParallelBlock, RotaryEncoding, StretchedRotaryEncoding, TokenEmbedding)
    cfg = CONFIGS["A"]
    eps, width = cfg["norm"]["eps"], cfg["width"]
    layers = []
    for i, layer in enumerate(cfg["layers"]):
        m = layer["mixer"]
        if layer["type"] == "mlstm":
            mixer = GatedMemoryMixer(width, m["heads"], m["dim"], m["gate_cap"], eps, value_dim=m["vdim"])
        elif layer["type"] == "latent_attention":
            mixer = LatentAttentionMixer(width, m["heads"], m["dim"], m["rot_dim"], m["kv_rank"], m["q_rank"],
                                         RotaryEncoding(m["rot_dim"], m["rot"]["base"]), eps, value_dim=m["vdim"],
                                         scale=m["scale"], sink=True, gate="sigmoid")
        else:
            sc = m["rot"].get("scaling")
            pos = (StretchedRotaryEncoding(m["dim"], m["rot"]["base"], sc["factor"], sc["low"], sc["high"], sc["original"],
                                           m["rot"]["dims"]) if sc else RotaryEncoding(m["dim"], m["rot"]["base"], m["rot"]["dims"]))
            names = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b",
                     "lq1": "lq1", "lk1": "lk1", "lq2": "lq2", "lk2": "lk2"}
            mixer = AttentionMixer(width, m["heads"], m["kv_heads"], m["dim"], pos, None, (m.get("mask") or {}).get("size", 0),
                                   m["scale"], value_dim=m["vdim"], bias=True, score_maps=2, combine_maps=True,
                                   lambda_init=m["diff"], combine_eps=eps, names=names)
        ffn = DenseFeedForward(width, layer["mlp"]["ff"]) if layer["mlp"] else None
        layers.append((f"l{i}.", ParallelBlock(LayerNorm(width, eps, "norm1", "norm1.b"), mixer, ffn, ("", "mix.", "mlp."))))
    spec = ModelSpec(config=None, hidden_size=width, vocab_size=cfg["vocab"],
                     embedding=TokenEmbedding(cfg["vocab"], width, weight_name="embed"), layers=layers,
                     order=[LayerRun(i, i) for i in range(len(layers))],
                     final_norm=("", LayerNorm(width, eps, "final.norm", "final.norm.b")),
                     head=("", OutputHead(cfg["vocab"], width, tied_to=None, weight_name="head")))
    mine = {s.name: tuple(s.shape) for s in spec.tensor_specs()}
    theirs = {s.name: tuple(s.shape) for s in spec_of(cfg).tensor_specs()}
    assert mine == theirs
