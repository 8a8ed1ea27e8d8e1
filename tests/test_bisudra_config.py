"""The Bisudra configuration as data: keys read and written back, records that may be absent, the cache every run keeps,
checkpoint names and shapes, what is refused, random weights, and the plain implementation on a model so small that its
mechanisms can be checked by hand."""
import copy
import math

import pytest
import torch

import plain_bisudra as P
from bisudra_helpers import CONFIGS, make_bisudra_dir, plain_inputs
from gpullama3.java_b200.cache import EntryNeeds, KVCacheNeed, StateNeed
from gpullama3.java_b200.config import BisudraConfig, ConfigError, config_from_dict
from gpullama3.java_b200.engine.model import CausalLM, parameter_specs_by_checkpoint_name

F = torch.float64


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_round_trip(name):
    d = CONFIGS[name]
    cfg = config_from_dict(d)
    assert isinstance(cfg, BisudraConfig) and config_from_dict(cfg.to_dict()) == cfg
    assert [e.layer for e in cfg.schedule()] == list(range(len(d["layers"])))
    assert cfg.canon_taps == (d.get("canon") or {}).get("taps", 0) and cfg.side_dim == (d.get("token_side") or {}).get("dim", 0)
    assert cfg.tie_word_embeddings and cfg.embedding_scale() == 1.0


def test_names_shapes_and_needs():
    d = CONFIGS["A"]
    cfg = config_from_dict(d)
    specs = parameter_specs_by_checkpoint_name(cfg)
    for n in ("embed", "side.embed", "final.norm", "final.norm.b", "l0.norm1", "l0.norm1.b", "l0.norm2", "l0.norm2.b", "l0.rg1",
              "l0.rg1.b", "l0.rg2", "l0.rg2.b", "l0.canon1", "l0.dwa", "l0.side.gate", "l0.side.proj", "l0.side.norm", "l0.mix.q",
              "l0.mix.k", "l0.mix.v", "l0.mix.g", "l0.mix.o", "l0.mix.q.norm", "l0.mix.k.norm", "l0.mix.lq1", "l0.mix.lk1",
              "l0.mix.lq2", "l0.mix.lk2", "l0.mlp.router", "l0.mlp.router.b", "l0.mlp.e5.gate", "l0.mlp.e0.down", "l2.mlp.up",
              "l2.mlp.up.b", "l2.mlp.down", "l2.mlp.down.b"):
        assert n in specs, n
    assert not any(n in specs for n in ("head", "l1.norm2", "l1.rg2", "l1.mlp.up", "l0.canon2", "l0.mlp.e6.up"))
    assert {"l1.norm2", "l1.norm2.b", "l1.rg2", "l1.rg2.b"} <= cfg.optional_tensor_names()
    assert specs["l0.mix.q"].shape == (4 * 2 * 16, 64) and specs["l0.mix.k"].shape == (2 * 2 * 16, 64)
    assert specs["l0.mix.v"].shape == (2 * 32, 64) and specs["l0.mix.g"].shape == (4 * 32, 64) and specs["l0.mix.o"].shape == (64, 4 * 32)
    assert specs["l0.mix.q.norm"].shape == (16,) and specs["l1.mix.lk2"].shape == (24,)
    assert specs["side.embed"].shape == (160, 3 * 12) and specs["l1.side.gate"].shape == (12, 64) and specs["l1.side.proj"].shape == (64, 12)
    assert [specs[f"l{i}.dwa"].shape for i in range(3)] == [(2,), (3,), (4,)]
    assert specs["l0.canon1"].shape == (64, 4) and specs["l0.rg1"].shape == (64, 64) and specs["l2.mlp.up.b"].shape == (96,)
    model = CausalLM(cfg, torch.float32, "cpu")
    needs = model.cache_needs()
    assert len(needs) == 3
    # two maps of 16 side by side fill a row of 32; two of 24 are widened to 64; two of 8 lie in the 32 the values need
    assert [needs[i].named()["mixer"] for i in range(3)] == [KVCacheNeed(2, 32, 40), KVCacheNeed(2, 64, 130), KVCacheNeed(2, 32, None)]
    assert all(isinstance(n, EntryNeeds) and n.named()["inputs"] == StateNeed((3 * 64,), torch.float32) for n in needs.values())
    assert model.graph_safe and not model.pad_safe
    # a single tap keeps no inputs, and neither does a model without the convolution
    for name in ("C", "D"):
        m = CausalLM(config_from_dict(CONFIGS[name]), torch.float32, "cpu")
        assert all(isinstance(n, KVCacheNeed) for n in m.cache_needs().values())
    assert CausalLM(config_from_dict(CONFIGS["C"]), torch.float32, "cpu").cache_needs()[0] == KVCacheNeed(1, 96, 7)


def test_absent_records_build_the_model_without_the_mechanism():
    d = copy.deepcopy(CONFIGS["A"])
    del d["canon"], d["token_side"]
    for L in d["layers"]:
        L["mixer"].pop("mask", None)
        L["mixer"].pop("rot", None)
    specs = parameter_specs_by_checkpoint_name(config_from_dict(d))
    assert not any(n.endswith("canon1") or "side" in n for n in specs)
    model = CausalLM(config_from_dict(d), torch.float32, "cpu")
    assert model.cache_needs()[0] == KVCacheNeed(2, 32, None)
    assert model.blocks[0].mixer.position.rotary_dim == 0 and model.blocks[0].mixer.window is None


@pytest.mark.parametrize("change, message", [
    (lambda d: d["layers"][0].update(type="delta"), "unknown mixer type"),
    (lambda d: d["layers"][0]["mixer"].update(heads=3), "not a multiple"),
    (lambda d: d["layers"][0]["mixer"].pop("diff"), "diff"),
    (lambda d: d["layers"][0]["mixer"].update(scale=0.0), "positive"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=3), "rot.dims"),
    (lambda d: d["layers"][0]["mixer"].update(mask={}), "size"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=7), "7 of 6"),
    (lambda d: d["layers"][2]["mlp"].pop("ff"), "ff"),
    (lambda d: d["layers"][2]["mlp"].update(kind="gated"), "kind"),
    (lambda d: d.update(norm={}), "eps"),
    (lambda d: d.update(canon=3), "taps"),
    (lambda d: d.pop("width"), "width"),
    (lambda d: d["layers"][0]["mixer"].update(dim=300), "attention kernels"),
])
def test_refusals(change, message):
    d = copy.deepcopy(CONFIGS["A"])
    change(d)
    with pytest.raises((ConfigError, ValueError)) as e:
        CausalLM(config_from_dict(d), torch.float32, "cpu")
    assert message in str(e.value)


def test_random_weights_fill_every_tensor(tmp_path):
    d = make_bisudra_dir(tmp_path, CONFIGS["C"], seed=3)
    cfg, weights = plain_inputs(d)
    specs = parameter_specs_by_checkpoint_name(config_from_dict(cfg))
    assert set(weights) == set(specs) and all(tuple(weights[n].shape) == tuple(specs[n].shape) for n in specs)
    assert all(float(w.abs().max()) > 0 for w in weights.values())
    logits = P.forward(cfg, weights, [3, 1, 4, 1, 5, 9, 2, 6])
    assert logits.shape == (8, cfg["vocab"]) and torch.isfinite(logits).all()


def test_plain_mechanisms_by_hand():
    # a window of 2 over values that are one-hot: each query's result is the mean of the last two values when all scores are equal
    q = torch.zeros(4, 2, dtype=F)
    v = torch.eye(4, dtype=F)
    out = P.windowed_softmax_attention(q, q, v, 1.0, 2)
    assert torch.allclose(out, torch.tensor([[1, 0, 0, 0], [.5, .5, 0, 0], [0, .5, .5, 0], [0, 0, .5, .5]], dtype=F))
    assert torch.allclose(P.windowed_softmax_attention(q, q, v, 1.0, None)[3], torch.full((4,), 0.25, dtype=F))
    # rotation: position 0 stays; a pair turns by position * base^(-2i/dims); what lies beyond dims stays
    x = torch.tensor([[[1.0, 0.0, 1.0, 0.0, 7.0, 8.0]], [[1.0, 0.0, 1.0, 0.0, 7.0, 8.0]]], dtype=F)
    r = P.rotate_interleaved(x, torch.tensor([0, 3]), 100.0, 4)
    assert torch.equal(r[0], x[0]) and torch.equal(r[1, 0, 4:], x[1, 0, 4:])
    assert torch.allclose(r[1, 0, :4], torch.tensor([math.cos(3.0), math.sin(3.0), math.cos(0.3), math.sin(0.3)], dtype=F))
    # convolution: the last tap is the token itself
    h = torch.arange(1.0, 5.0, dtype=F)[:, None]
    assert torch.allclose(P.causal_conv(h, torch.tensor([[100.0, 10.0, 1.0]], dtype=F))[:, 0], torch.tensor([1.0, 12.0, 123.0, 234.0], dtype=F))
    # the router: the largest logits, weighted by the softmax over them alone
    W = {"x.mlp.router": torch.eye(3, dtype=F), "x.mlp.router.b": torch.tensor([0.0, 0.0, 5.0], dtype=F)}
    chosen, weights = P.router_choice(torch.tensor([[4.0, 1.0, 0.0]], dtype=F), W, "x.", 2)
    assert chosen.tolist() == [[2, 0]] and torch.allclose(weights, torch.softmax(torch.tensor([[5.0, 4.0]], dtype=F), -1))
    # the mix over the levels, and lambda
    assert torch.equal(P.depth_average([torch.ones(2), 2 * torch.ones(2), 4 * torch.ones(2)], torch.tensor([1.0, 0.5, -0.25])), torch.ones(2))
    one = torch.ones(2, dtype=F)
    lam = P.differential_weight({"x.mix.lq1": one, "x.mix.lk1": one, "x.mix.lq2": one, "x.mix.lk2": 2 * one}, "x.", 0.3)
    assert abs(lam - (math.exp(2.0) - math.exp(4.0) + 0.3)) < 1e-12
    assert torch.allclose(P.squared_relu(torch.tensor([-2.0, 3.0])), torch.tensor([0.0, 9.0]))
