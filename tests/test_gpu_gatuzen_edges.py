"""Keys far back and at page borders in Gatuzen's latent attention, memory far back in its two recurrences, the first
tokens of a sequence, the reach of the input convolutions, the rotation's position, and long decoding.  Each test first
shows on the plain implementation that the thing it probes moves the logits by far more than the tolerance (the far keys
hidden, the early tokens dropped, the positions shifted, a tap removed), so that an engine that got it wrong could not
pass.  The far-key model's score scale is large, so that single keys carry the result."""
import copy

import pytest
import torch

import plain_gatuzen
from conftest import random_prompts
from gatuzen_helpers import assert_logits, make_gatuzen_dir, plain_inputs

pytestmark = pytest.mark.gpu
DTYPES = pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])


def _moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


FAR = {
    "architecture": "Gatuzen", "vocab": 64, "width": 32, "embedding": {"scale": 4.0}, "norm": {"eps": 1e-6, "groups": 2},
    "canon": {"taps": 2}, "logit_scale": 1.0, "residual_mult": 0.8, "initializer_range": 0.1,
    "layers": [
        {"type": "latent_attention", "mlp": _moe(24, 3, 1),
         "mixer": {"heads": 2, "dim": 16, "rot_dim": 16, "vdim": 16, "kv_rank": 48, "scale": 1.2,
                   "rot": {"base": 2000.0, "dims": 16, "scaling": {"factor": 4.0, "original": 128, "fast": 8.0, "slow": 1.0}}}},
    ],
}
MEMORY = {
    "architecture": "Gatuzen", "vocab": 64, "width": 32, "embedding": {"scale": 4.0}, "norm": {"eps": 1e-6, "groups": 1},
    "canon": {"taps": 4}, "logit_scale": 1.0, "residual_mult": 0.8, "initializer_range": 0.1,
    "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [
        {"type": "gla", "mixer": {"heads": 2, "dim": 16, "vdim": 16, "tau": 64.0, "decay_rank": 4}, "mlp": None},
        {"type": "mamba2", "mlp": _moe(24, 2, 2),
         "mixer": {"heads": 2, "vdim": 16, "state": 16, "groups": 1, "conv": 4, "norm_groups": 2}},
    ],
}


def _run(model_dir, dtype, tokens, prompt_len, chunk=None):
    """Logits at every position: the first ``prompt_len`` tokens as a prompt (in portions of ``chunk``), the rest one
    token a step."""
    from gpullama3.java_b200.engine.step import SequenceInput, StepFunction
    from gpullama3.java_b200.engine.trace import load_model

    model = load_model(model_dir, dtype)
    cache = model.new_cache(64 * (len(tokens) // 64 + 2))
    step = StepFunction(model, cache)
    slot = cache.acquire()
    out, at = [], 0
    while at < len(tokens):
        n = 1 if at >= prompt_len else min(chunk or prompt_len, prompt_len - at)
        out.append(step([SequenceInput(slot, tokens[at:at + n], list(range(n)))]).cpu().clone())
        at += n
    cache.release(slot)
    cache.check_invariants()
    return torch.cat(out)


def _moved(a, b, scale):
    """Per position: how far two sets of logits are apart, in units of the float32 tolerance."""
    return (a - b).abs().amax(dim=1) / (5e-5 * scale)


@DTYPES
@pytest.mark.parametrize("prompt_len, chunk", [(700, None), (520, 130), (64, None), (3, None)])
def test_far_keys_positions_and_page_borders(session_tmp, dtype, prompt_len, chunk):
    """700 tokens: eleven pages of latent rows with peaked scores; what a query finds depends on keys hundreds of
    positions back and on both positions of every rotated pair."""
    d = make_gatuzen_dir(session_tmp, FAR, seed=4)
    cfg, weights = plain_inputs(d)
    tokens = random_prompts(cfg["vocab"], [700], seed=5)[0]
    ref = plain_gatuzen.forward(cfg, weights, tokens)
    scale = float(ref.abs().max())
    # without the first 300 tokens the late logits differ: far keys count
    late = plain_gatuzen.forward(cfg, weights, tokens[300:])
    assert float((_moved(late[250:], ref[550:], scale) > 20).float().mean()) > 0.9
    # other frequencies, another magnitude, no stretching: the rotation counts, and so does its constant factor
    for change in (dict(base=1000.0), dict(scaling=None), dict(scaling={"factor": 2.0, "original": 128, "fast": 8.0, "slow": 1.0})):
        c2 = copy.deepcopy(cfg)
        c2["layers"][0]["mixer"]["rot"].update(change)
        if change.get("scaling", 0) is None:
            del c2["layers"][0]["mixer"]["rot"]["scaling"]
        assert float((_moved(plain_gatuzen.forward(c2, weights, tokens), ref, scale)[8:] > 20).float().mean()) > 0.9, change
    # the output gate and the shared rotated key part count
    for name in ("l0.mix.g", "l0.canon1"):
        w2 = dict(weights)
        w2[name] = torch.zeros_like(weights[name])
        assert float((_moved(plain_gatuzen.forward(cfg, w2, tokens), ref, scale)[2:] > 20).float().mean()) > 0.9, name
    got = _run(d, dtype, tokens, prompt_len, chunk)
    assert_logits(got, ref, dtype, f"far keys, prompt of {prompt_len}")
    assert_logits(got[:4], ref[:4], dtype, "the first tokens")
    for edge in (63, 64, 65, 127, 128, 639, 640):
        assert_logits(got[edge:edge + 1], ref[edge:edge + 1], dtype, f"position {edge}")


@DTYPES
@pytest.mark.parametrize("prompt_len, chunk", [(500, None), (380, 77), (5, None)])
def test_long_memory_of_the_recurrences(session_tmp, dtype, prompt_len, chunk):
    """Two passes over a gated-linear-attention layer and a state-space layer whose states still hold the first tokens
    after five hundred, each pass with a state of its own; input convolutions of four taps."""
    d = make_gatuzen_dir(session_tmp, MEMORY, seed=6, slow_decay=6.0)
    cfg, weights = plain_inputs(d)
    tokens = random_prompts(cfg["vocab"], [500], seed=7)[0]
    ref = plain_gatuzen.forward(cfg, weights, tokens)
    scale = float(ref.abs().max())
    late = plain_gatuzen.forward(cfg, weights, tokens[300:])          # the same tokens without the first 300
    assert float((_moved(late[100:], ref[400:], scale) > 20).float().mean()) > 0.9
    one = copy.deepcopy(cfg)
    one["loop"]["times"] = 1                                          # a pass less
    assert float((_moved(plain_gatuzen.forward(one, weights, tokens), ref, scale) > 20).float().mean()) > 0.9
    swapped = dict(weights)
    swapped["loop.step"] = weights["loop.step"].flip(0)               # the passes' vectors the other way round
    assert float((_moved(plain_gatuzen.forward(cfg, swapped, tokens), ref, scale) > 20).float().mean()) > 0.9
    for name in ("l0.canon1", "l1.canon2", "l1.mix.conv"):
        w2 = dict(weights)
        w2[name] = weights[name].clone()
        w2[name][:, 0] = 0.0                                          # the tap that reaches furthest back
        assert float((_moved(plain_gatuzen.forward(cfg, w2, tokens), ref, scale)[4:] > 20).float().mean()) > 0.9, name
    for name in ("l1.mix.D", "l1.mix.dt_bias", "l0.mix.a2.b"):
        w2 = dict(weights)
        w2[name] = weights[name] + 0.5
        assert float((_moved(plain_gatuzen.forward(cfg, w2, tokens), ref, scale)[4:] > 20).float().mean()) > 0.9, name
    got = _run(d, dtype, tokens, prompt_len, chunk)
    assert_logits(got, ref, dtype, f"long memory, prompt of {prompt_len}")
    assert_logits(got[:5], ref[:5], dtype, "the first tokens")
