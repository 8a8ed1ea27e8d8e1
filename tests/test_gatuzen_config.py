"""The Gatuzen configuration as data: keys read and written back, the order of runs with its loop, the cache every run
keeps, checkpoint names, what is refused, random weights, and the plain implementation's order of runs."""
import copy
import json

import pytest
import torch

import plain_gatuzen
from gatuzen_helpers import CONFIGS, make_gatuzen_dir, plain_inputs
from gpullama3.java_b200.cache import EntryNeeds, KVCacheNeed, SequenceCache, StateNeed
from gpullama3.java_b200.config import ConfigError, GatuzenConfig, config_from_dict
from gpullama3.java_b200.engine.model import CausalLM, parameter_specs_by_checkpoint_name


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_round_trip_and_schedule(name):
    d = CONFIGS[name]
    cfg = config_from_dict(d)
    assert isinstance(cfg, GatuzenConfig) and config_from_dict(cfg.to_dict()) == cfg
    runs = [(e.layer, e.enters) for e in cfg.schedule()]
    assert runs == plain_gatuzen.layer_runs(d)
    assert [e.cache for e in cfg.schedule()] == list(range(len(runs)))          # every run has a cache entry of its own
    assert cfg.pass_offsets() == (d["loop"]["times"] if "loop" in d else 0)
    assert cfg.embedding_scale() == d["embedding"]["scale"] and cfg.output_scale() == d["logit_scale"]


def test_loop_runs():
    cfg = config_from_dict(CONFIGS["A"])
    assert [(e.layer, e.enters) for e in cfg.schedule()] == [(0, 0), (1, None), (0, 1), (1, None), (0, 2), (1, None), (2, None)]
    cfg = config_from_dict(CONFIGS["C"])
    assert [(e.layer, e.enters) for e in cfg.schedule()] == [(0, None), (1, 0), (2, None)]


def test_names_and_needs():
    d = CONFIGS["A"]
    cfg = config_from_dict(d)
    specs = parameter_specs_by_checkpoint_name(cfg)
    for n in ("embed", "head", "final.norm", "loop.step", "l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b", "l0.canon1",
              "l0.canon2", "l0.mix.q", "l0.mix.dkv", "l0.mix.dkv.norm", "l0.mix.uk", "l0.mix.uv", "l0.mix.g", "l0.mix.o",
              "l0.mlp.table", "l0.mlp.e5.down", "l1.mix.a1", "l1.mix.a2", "l1.mix.a2.b", "l1.mix.norm", "l2.mix.in",
              "l2.mix.conv", "l2.mix.conv.b", "l2.mix.dt_bias", "l2.mix.A_log", "l2.mix.D", "l2.mix.norm"):
        assert n in specs, n
    assert "l1.norm2" not in specs and "l1.canon2" not in specs and "l1.mlp.table" not in specs
    assert {"l1.norm2", "l1.norm2b", "l1.canon2"} <= cfg.optional_tensor_names()
    assert specs["loop.step"].shape == (3, 64) and specs["l0.mlp.table"].shape == (160, 2)
    assert specs["l0.mix.q"].shape == (4 * (16 + 8), 64) and specs["l0.mix.dkv"].shape == (40 + 8, 64)
    assert specs["l2.mix.in"].shape == (2 * 64 + 2 * 2 * 24 + 4, 64) and specs["l2.mix.conv"].shape == (64 + 96, 3)
    assert specs["l0.canon1"].shape == (64, 3)
    model = CausalLM(cfg, torch.float32, "cpu")
    needs = model.cache_needs()
    assert len(needs) == 7
    first = needs[0]
    assert isinstance(first, EntryNeeds) and first.named()["mixer"] == KVCacheNeed(1, 64, None)   # 40 + 8 widened to 64
    assert first.named()["inputs"] == StateNeed((2 * 2 * 64,), torch.float32)
    assert needs[1].named()["inputs"] == StateNeed((2 * 64,), torch.float32)                     # no feed-forward: one convolution
    assert needs[1].named()["mixer"] == StateNeed((3 * 24 * 16,), torch.float32)
    assert needs[6].named()["mixer"] == StateNeed((4 * 24 * 16 + 2 * (64 + 96),), torch.float32)
    assert model.graph_safe and not model.pad_safe
    # a single tap keeps no inputs
    b = CausalLM(config_from_dict(CONFIGS["B"]), torch.float32, "cpu")
    assert b.cache_needs()[1] == KVCacheNeed(1, 128, None) and b.pass_offsets is None


def test_entries_with_several_needs_share_groups():
    needs = {0: EntryNeeds((("mixer", KVCacheNeed(1, 32)), ("inputs", StateNeed((6,))))),
             1: EntryNeeds((("mixer", StateNeed((10,))), ("inputs", StateNeed((6,))))),
             2: KVCacheNeed(1, 32), 3: StateNeed((10,))}
    cache = SequenceCache(needs, max_tokens=256, max_slots=3, dtype=torch.float32, device="cpu")
    assert len(cache.paged_groups) == 1 and len(cache.slot_groups) == 2
    v0, v1 = cache.view(0), cache.view(1)
    assert set(v0) == {"mixer", "inputs"} and v0["mixer"].k.shape[1:] == (1, 64, 32)
    assert v0["inputs"].data.shape == (3, 6) and v1["mixer"].data.shape == (3, 10)
    assert v0["inputs"].data.data_ptr() != v1["inputs"].data.data_ptr()
    assert cache.view(2).k.data_ptr() != v0["mixer"].k.data_ptr() and cache.view(3).data.shape == (3, 10)
    s = cache.acquire()
    v1["inputs"].data[s] = 1.0
    cache.release(s)
    assert cache.acquire() == s and float(v1["inputs"].data[s].abs().sum()) == 0.0     # a slot used again starts from zero
    cache.check_invariants()


@pytest.mark.parametrize("change, message", [
    (lambda d: d["layers"][0].update(type="conv"), "unknown mixer type"),
    (lambda d: d["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda d: d["layers"][0]["mixer"]["rot"].update(dims=4), "rotated"),
    (lambda d: d["layers"][0]["mixer"]["rot"]["scaling"].pop("original"), "original"),
    (lambda d: d["layers"][2]["mixer"].update(groups=3), "groups"),
    (lambda d: d["layers"][0]["mlp"]["router"].update(top=9), "experts"),
    (lambda d: d["layers"][0].update(mlp={"kind": "dense", "ff": 8}), "kind 'moe'"),
    (lambda d: d["loop"].update(stop=5), "loop"),
    (lambda d: d["norm"].update(groups=5), "equal parts"),
    (lambda d: d["layers"][1]["mixer"].update(tau=0.0), "tau"),
])
def test_refused(change, message):
    d = copy.deepcopy(CONFIGS["A"])
    change(d)
    with pytest.raises(ConfigError, match=message):
        CausalLM(config_from_dict(d), torch.float32, "cpu")


def test_random_weights_and_tables(tmp_path):
    d = make_gatuzen_dir(tmp_path, CONFIGS["A"], seed=3)
    cfg, weights = plain_inputs(d)
    assert json.loads((d / "config.json").read_text()) == cfg
    table = weights["l0.mlp.table"]
    assert table.dtype == torch.int32 and int(table.min()) >= 0 and int(table.max()) < 6
    assert bool((table[:, 0] != table[:, 1]).all()) and len(set(table[:, 0].tolist())) > 2
    logits = plain_gatuzen.forward(cfg, weights, [1, 2, 3, 4, 5])
    assert logits.shape == (5, 160) and bool(torch.isfinite(logits).all())
    # the plain implementation's own pieces: causality, and the state of its recurrences carried by whole-sequence calls
    longer = plain_gatuzen.forward(cfg, weights, [1, 2, 3, 4, 5, 6, 7])
    assert float((longer[:5] - logits).abs().max()) < 1e-9
