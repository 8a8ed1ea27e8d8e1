"""Small Gatuzen configurations for the tests, and model folders with random weights made so that faults show.

The configurations differ from one another in every size and option: the order of the mixers, a loop over the
first layers, over inner layers and none, one pass and several, norms in one part and in several, input convolutions of
1 to 4 taps and none, layers without feed-forward, one expert of several and several of many, heads that share a group of
the state-space mixer and heads that have their own, key sizes below and above value sizes, a latent plus rotated part
that fills a size the tensor-core attention kernels take and ones that are widened, rotation with and without stretched
frequencies, scales that are no powers of two."""
from __future__ import annotations

import json
from pathlib import Path

import torch


def _moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _latent(heads, dim, rot_dim, vdim, kv_rank, scale, base=10000.0, scaling=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling is not None:
        rot["scaling"] = scaling
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale, "rot": rot}


GATUZEN_A = {
    "architecture": "Gatuzen", "vocab": 160, "width": 64, "embedding": {"scale": 5.5}, "norm": {"eps": 1e-5, "groups": 2},
    "canon": {"taps": 3}, "logit_scale": 0.7, "residual_mult": 0.6, "initializer_range": 0.08,
    "loop": {"start": 0, "stop": 2, "times": 3},
    "layers": [
        {"type": "latent_attention", "mlp": _moe(32, 6, 2),
         "mixer": _latent(4, 16, 8, 24, 40, 0.3, 5000.0, {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0})},
        {"type": "gla", "mixer": {"heads": 3, "dim": 24, "vdim": 16, "tau": 8.0, "decay_rank": 8}, "mlp": None},
        {"type": "mamba2", "mlp": _moe(48, 4, 1),
         "mixer": {"heads": 4, "vdim": 16, "state": 24, "groups": 2, "conv": 3, "norm_groups": 4}},
    ],
}
GATUZEN_B = {
    "architecture": "Gatuzen", "vocab": 200, "width": 96, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-6, "groups": 1},
    "canon": {"taps": 1}, "logit_scale": 1.0, "residual_mult": 1.0, "initializer_range": 0.06,
    "layers": [
        {"type": "mamba2", "mlp": _moe(24, 8, 3),
         "mixer": {"heads": 3, "vdim": 40, "state": 16, "groups": 3, "conv": 2, "norm_groups": 1}},
        {"type": "latent_attention", "mlp": None, "mixer": _latent(2, 48, 32, 40, 96, 0.11)},
        {"type": "gla", "mixer": {"heads": 1, "dim": 72, "vdim": 8, "tau": 1.5, "decay_rank": 4}, "mlp": _moe(40, 9, 4)},
    ],
}
GATUZEN_C = {
    "architecture": "Gatuzen", "vocab": 96, "width": 48, "embedding": {"scale": 0.75}, "norm": {"eps": 1e-6, "groups": 3},
    "canon": {"taps": 4}, "logit_scale": 2.5, "residual_mult": 0.35, "initializer_range": 0.1,
    "loop": {"start": 1, "stop": 2, "times": 1},
    "layers": [
        {"type": "gla", "mixer": {"heads": 2, "dim": 8, "vdim": 40, "tau": 32.0, "decay_rank": 16}, "mlp": _moe(16, 2, 2)},
        {"type": "latent_attention", "mlp": _moe(16, 3, 1),
         "mixer": _latent(20, 8, 2, 8, 22, 0.5, 300.0, {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0})},
        {"type": "mamba2", "mlp": None,
         "mixer": {"heads": 2, "vdim": 24, "state": 40, "groups": 1, "conv": 4, "norm_groups": 3}},
    ],
}
# rows wide enough for the step kernel that keeps a token's row in registers and, in decode steps, also reads for the next
# sublayer (groups of whole 128-number pieces): a block without feed-forward hands its rows straight to the next block,
# and the loop's vector joins the stream in that same kernel
GATUZEN_D = {
    "architecture": "Gatuzen", "vocab": 120, "width": 256, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5, "groups": 2},
    "canon": {"taps": 4}, "logit_scale": 0.8, "residual_mult": 0.5, "initializer_range": 0.05,
    "loop": {"start": 1, "stop": 3, "times": 2},
    "layers": [
        {"type": "gla", "mixer": {"heads": 2, "dim": 16, "vdim": 24, "tau": 4.0, "decay_rank": 8}, "mlp": None},
        {"type": "mamba2", "mlp": _moe(32, 3, 2),
         "mixer": {"heads": 2, "vdim": 32, "state": 16, "groups": 2, "conv": 3, "norm_groups": 2}},
        {"type": "latent_attention", "mlp": None, "mixer": _latent(3, 24, 8, 16, 56, 0.2)},
        {"type": "gla", "mixer": {"heads": 1, "dim": 40, "vdim": 32, "tau": 12.0, "decay_rank": 4}, "mlp": _moe(24, 4, 1)},
    ],
}
CONFIGS = {"A": GATUZEN_A, "B": GATUZEN_B, "C": GATUZEN_C, "D": GATUZEN_D}


def make_gatuzen_dir(tmp_path: Path, config_json: dict, seed: int = 0, slow_decay: float = 3.0, edit=None) -> Path:
    """A model folder with random bfloat16 weights.  Norm weights get a visible spread; the state-space layers' step
    biases are lowered by ``slow_decay`` so that their state remembers hundreds of tokens instead of a handful (the
    gated linear attention's decay biases are made for that already); every row of a routing table names different
    experts.  ``edit(tensors)`` may change the float32 tensors before they are rounded and written."""
    from gpullama3.java_b200.config import config_from_dict
    from gpullama3.java_b200.weights import random_checkpoint, write_safetensors

    cfg = config_from_dict(config_json)
    tag = abs(hash(json.dumps([config_json, seed, slow_decay, getattr(edit, "__name__", None)], sort_keys=True))) % 10 ** 10
    out = Path(tmp_path) / f"gatuzen_{tag}"
    if (out / "model.safetensors").is_file():
        return out
    out.mkdir(parents=True, exist_ok=True)
    where = "cuda" if torch.cuda.is_available() else "cpu"
    tensors = {}
    for n, t in random_checkpoint(cfg, seed, dtype=torch.float32, norm_std=0.2, device=where):
        tensors[n] = t.cpu() if not t.is_floating_point() else t.cpu().to(torch.float32)
    for name in tensors:
        if name.endswith(".dt_bias"):
            tensors[name] = tensors[name] - slow_decay
    if edit is not None:
        edit(tensors)
    (out / "config.json").write_text(json.dumps(cfg.to_dict(), indent=2))
    write_safetensors(out / "model.safetensors",
                      {n: (t.to(torch.bfloat16) if t.is_floating_point() else t.to(torch.int32)) for n, t in tensors.items()})
    return out


def plain_inputs(model_dir: Path):
    """config.json as a dict and the weights by checkpoint name (floats as float32, tables as stored), read with the
    safetensors package (not with the product's reader)."""
    from safetensors.torch import load_file

    cfg = json.loads((Path(model_dir) / "config.json").read_text())
    weights = {k: (v.to(torch.float32) if v.is_floating_point() else v)
               for k, v in load_file(str(Path(model_dir) / "model.safetensors")).items()}
    return cfg, weights


class Reference:
    """The plain implementation's logits of a request and, per position and logit, how far they move when what every
    sublayer reads is rounded to bfloat16 once: where a sublayer's result is small by chance (the first tokens of a
    recurrent layer of few channels, whose result can change sign with one rounding) the norm behind it magnifies any
    rounding, and the plain implementation shows that itself."""

    def __init__(self, logits: torch.Tensor, moved: torch.Tensor):
        self.logits, self.moved = logits, moved

    def __getitem__(self, index):
        return Reference(self.logits[index], self.moved[index])


def reference(cfg, weights, tokens) -> Reference:
    import plain_gatuzen

    exact = plain_gatuzen.forward(cfg, weights, tokens)
    rounded = plain_gatuzen.forward(cfg, weights, tokens, reads=lambda h: h.to(torch.bfloat16).to(h.dtype))
    return Reference(exact, (rounded - exact).abs())


def assert_logits(got: torch.Tensor, ref, dtype, what: str = "") -> None:
    """float32: accumulation-order noise only, at every position.  bfloat16: the engine rounds activations between its
    kernels, the plain implementation does not round at all; what is allowed is a few roundings' worth relative to the
    largest logit (the routing is a table: it cannot flip), plus, against a ``Reference``, a few times what one rounding
    moves the plain implementation's own result at that position."""
    moved = None
    if isinstance(ref, Reference):
        ref, moved = ref.logits, ref.moved.detach().to("cpu", torch.float64)
    got = got.detach().to("cpu", torch.float64)
    ref = ref.detach().to("cpu", torch.float64)
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    scale = float(ref.abs().max()) + 1e-30
    err = (got - ref).abs()
    if dtype == torch.float32:
        # (where one bfloat16 rounding of what the sublayers read moves the plain result far, a 32-bit rounding, 2^-15 of
        # it, is magnified alike: such a position is allowed a few dozen of those)
        allowed = 5e-5 * scale + (1e-3 * moved.amax(dim=-1) if moved is not None else 0.0)
        worst = err.amax(dim=-1)
        over = worst - allowed
        assert float(over.max()) <= 0.0, (f"{what}: max err {float(worst.max()):.3e} vs scale {scale:.3e} "
                                          f"(position {int(over.argmax())})")
        return
    # A sublayer's result is normed before it joins the stream, so where that result is small by chance (a recurrent
    # layer's first tokens, whose state holds one or two outer products of a few channels) the norm magnifies the
    # rounding of the projections; such positions are allowed as a small share, and the typical position is held tighter.
    worst, mean = err.amax(dim=-1), err.mean(dim=-1)
    if moved is None:
        bad = (worst > 0.08 * scale) | (mean > 0.012 * scale)
    else:   # (the engine rounds in several places: a few times what one rounding in the plain implementation does)
        bad = (worst > 0.08 * scale + 6.0 * moved.amax(dim=-1)) | (mean > 0.012 * scale + 6.0 * moved.mean(dim=-1))
    allowed = max(1, int(0.12 * bad.numel())) if bad.numel() >= 3 else 0
    assert int(bad.sum()) <= allowed, (f"{what}: {int(bad.sum())} of {bad.numel()} positions outside "
                                       f"(max err {float(err.max()):.3e}, scale {scale:.3e})")
    typical = 0.04 * scale + (6.0 * float(moved.amax(dim=-1).median()) if moved is not None else 0.0)
    assert float(worst.median()) <= typical, f"{what}: median of the worst errors {float(worst.median()):.3e} vs scale {scale:.3e}"
