"""Typed configuration of the Bisudra decoder, read from ``config.json``.

A Bisudra model is a list of layers over one residual stream.  A sublayer reads the stream itself (no norm in front);
its result is multiplied by a sigmoid gate of the sublayer's own input, passes a layer norm with weight and bias
(``norm.eps``) and is then added.  The mixer reads its input plus a causal convolution of ``canon.taps`` taps over it.  After
the feed-forward a few learned numbers per (token id, layer) (``token_side.dim`` of them) join the stream, gated by it,
projected to its width and RMS-normed.  What a layer hands on is a learned mix of the embedding output and every
layer's result so far.  The output head is the embedding table, behind a last layer norm.

* ``layers[i].type`` names the mixer, ``layers[i].mixer`` gives its sizes.  ``attention``: differential attention, two
  softmax maps per head over the same values (``heads``, ``kv_heads``, per-map query/key size ``dim``, value size ``vdim``,
  score ``scale``, the constant ``diff``, a sliding window ``mask.size``, rotation of the first ``rot.dims`` numbers of
  every map in interleaved pairs with ``rot.base``), with an RMS norm over every map of every query and key head and a
  sigmoid gate on the heads' results;
* ``layers[i].mlp`` is null, ``{"kind": "dense", "ff"}`` (one product up with the square of max(., 0), one down, both
  with biases) or ``{"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}}`` (SiLU-gated experts without
  biases; router logits with a bias, the ``top`` largest chosen, weighted by the softmax over the chosen logits).

A record that is absent (``canon``, ``token_side``, a mixer's ``mask`` or ``rot``) builds the model without that mechanism."""
from __future__ import annotations

from dataclasses import dataclass

from .base import ConfigError, LayerSpec, ModelConfig, PartSpec, as_float, as_int, require_keys
from .registry import register_architecture

MIXER_TYPES = ("attention",)


def _positive(d: dict, key: str, where: str) -> float:
    v = as_float(d, key)
    if not v > 0:
        raise ConfigError(f"{where}: {key} must be positive, got {v}")
    return v


@dataclass(frozen=True)
class BisudraLayer:
    type: str
    mixer: dict        # the mixer's record as config.json has it (checked when read)
    mlp: dict | None   # the feed-forward's record, None for a layer without one


@dataclass(frozen=True)
class BisudraConfig(ModelConfig):
    vocab_size: int
    hidden_size: int
    layers: tuple
    norm_eps: float
    canon_taps: int = 0
    side_dim: int = 0
    initializer_range: float = 0.02
    tie_word_embeddings: bool = True
    stop_token_ids: tuple[int, ...] = ()

    architecture = "Bisudra"

    # ---- reading
    @classmethod
    def from_dict(cls, d: dict) -> "BisudraConfig":
        require_keys(d, ["vocab", "width", "layers", "norm"], "Bisudra config.json")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("Bisudra config.json: 'layers' must be a non-empty list")
        if not isinstance(d["norm"], dict):
            raise ConfigError("Bisudra config.json: 'norm' must be an object with 'eps'")
        require_keys(d["norm"], ["eps"], "Bisudra norm")
        eps = _positive(d["norm"], "eps", "norm")

        def optional_int(key: str, inner: str) -> int:
            record = d.get(key)
            if record is None:
                return 0
            if not isinstance(record, dict):
                raise ConfigError(f"Bisudra config.json: {key!r} must be an object with {inner!r}")
            return as_int(record, inner, minimum=0) if record.get(inner) is not None else 0

        layers = []
        for i, L in enumerate(d["layers"]):
            where = f"layer {i}"
            if not isinstance(L, dict) or not isinstance(L.get("mixer"), dict):
                raise ConfigError(f"{where}: needs 'type' and a 'mixer' object")
            kind = L.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"{where}: unknown mixer type {kind!r}; known: {', '.join(MIXER_TYPES)}")
            mlp = L.get("mlp")
            layers.append(BisudraLayer(kind, cls._checked_attention(dict(L["mixer"]), where),
                                       cls._checked_mlp(mlp, where) if mlp is not None else None))
        eos = d.get("eos_token_id")
        stop = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        return cls(vocab_size=as_int(d, "vocab"), hidden_size=as_int(d, "width"), layers=tuple(layers), norm_eps=eps,
                   canon_taps=optional_int("canon", "taps"), side_dim=optional_int("token_side", "dim"),
                   initializer_range=float(d.get("initializer_range", 0.02)), stop_token_ids=stop)

    @staticmethod
    def _checked_attention(m: dict, where: str) -> dict:
        require_keys(m, ["heads", "kv_heads", "dim", "vdim", "scale", "diff"], where)
        for key in ("heads", "kv_heads", "dim", "vdim"):
            as_int(m, key)
        _positive(m, "scale", where)
        as_float(m, "diff")
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"{where}: heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")
        if m.get("mask") is not None:      # (no mask: every earlier position is visible)
            if not isinstance(m["mask"], dict):
                raise ConfigError(f"{where}: mask must be an object with 'size'")
            require_keys(m["mask"], ["size"], where + " mask")
            as_int(m["mask"], "size")
        if m.get("rot") is not None:       # (no rot: positions enter through the window and the convolution alone)
            if not isinstance(m["rot"], dict):
                raise ConfigError(f"{where}: rot must be an object with 'base' and 'dims'")
            require_keys(m["rot"], ["base", "dims"], where + " rot")
            _positive(m["rot"], "base", where + " rot")
            dims = as_int(m["rot"], "dims", minimum=0)
            if dims % 2 or dims > m["dim"]:
                raise ConfigError(f"{where}: rot.dims {dims} must be even and at most dim {m['dim']}")
        return m

    @staticmethod
    def _checked_mlp(mlp, where: str) -> dict:
        if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
            raise ConfigError(f"{where}: mlp must be null or an object of kind 'dense' or 'moe', got {mlp!r}")
        if mlp["kind"] == "dense":
            require_keys(mlp, ["ff"], where + " mlp")
            as_int(mlp, "ff")
            return dict(mlp)
        require_keys(mlp, ["expert", "router"], where + " mlp")
        ex, ro = mlp["expert"], mlp["router"]
        if not isinstance(ex, dict) or not isinstance(ro, dict):
            raise ConfigError(f"{where} mlp: 'expert' and 'router' must be objects")
        require_keys(ex, ["ff"], where + " mlp.expert")
        require_keys(ro, ["experts", "top"], where + " mlp.router")
        n, top = as_int(ro, "experts"), as_int(ro, "top")
        if top > n:
            raise ConfigError(f"{where} mlp.router: {top} of {n} experts")
        return {"kind": "moe", "expert": {"ff": as_int(ex, "ff")}, "router": {"experts": n, "top": top}}

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "norm": {"eps": self.norm_eps}, "initializer_range": self.initializer_range,
             "layers": [{"type": L.type, "mixer": dict(L.mixer), "mlp": dict(L.mlp) if L.mlp else None} for L in self.layers]}
        if self.canon_taps:
            d["canon"] = {"taps": self.canon_taps}
        if self.side_dim:
            d["token_side"] = {"dim": self.side_dim}
        if self.stop_token_ids:
            d["eos_token_id"] = list(self.stop_token_ids)
        return d

    # ---- the model as data
    def _norm(self) -> PartSpec:
        return PartSpec("norm", "layernorm", {"dim": self.hidden_size, "eps": self.norm_eps})

    def _mixer(self, i: int) -> PartSpec:
        m = self.layers[i].mixer
        rot = m.get("rot") or {}
        if rot.get("dims"):
            position = PartSpec("position", "rope", {"head_dim": m["dim"], "theta": float(rot["base"]), "pairing": "interleaved",
                                                       "rotary_dim": int(rot["dims"])})
        else:
            position = PartSpec("position", "none", {})
        return PartSpec("mixer", "differential_attention", {
            "hidden_size": self.hidden_size, "n_heads": m["heads"], "n_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "value_dim": m["vdim"], "scale": float(m["scale"]), "diff": float(m["diff"]), "norm_eps": self.norm_eps,
            "position": position, "window": (m.get("mask") or {}).get("size"), "output_gate": True})

    def _feed_forward(self, mlp: dict) -> PartSpec:
        if mlp["kind"] == "dense":
            return PartSpec("feed_forward", "dense", {"hidden_size": self.hidden_size, "intermediate_size": mlp["ff"],
                                                      "activation": "relu_squared", "bias": True})
        ro, ex = mlp["router"], mlp["expert"]
        return PartSpec("feed_forward", "routed", {
            "hidden_size": self.hidden_size, "intermediate_size": ex["ff"], "n_experts": ro["experts"], "top": ro["top"],
            "activation": "silu", "weight_eps": 0.0, "router_bias": True})

    def layer_specs(self) -> list[LayerSpec]:
        n = len(self.layers)
        specs = []
        for i, L in enumerate(self.layers):
            parts = {"mixer": self._mixer(i), "mixer_norm": self._norm()}
            if L.mlp is not None:
                parts["feed_forward"] = self._feed_forward(L.mlp)
                parts["feed_forward_norm"] = self._norm()
            specs.append(LayerSpec("gated_residual", parts, {
                "hidden_size": self.hidden_size, "conv_taps": self.canon_taps, "side_dim": self.side_dim,
                "side_columns": (i * self.side_dim, n * self.side_dim), "vocab_size": self.vocab_size,
                "side_eps": self.norm_eps, "depth": (i, n)}))
        return specs

    def final_norm(self) -> PartSpec:
        return self._norm()

    def tensor_names(self) -> dict[str, str]:
        names = {"embedding.table": "embed", "final_norm.weight": "final.norm", "final_norm.bias": "final.norm.b"}
        for i, L in enumerate(self.layers):
            p, c = f"layers.{i}.", f"l{i}."
            names[p + "mixer_norm.weight"], names[p + "mixer_norm.bias"] = c + "norm1", c + "norm1.b"
            names[p + "mixer_gate"], names[p + "mixer_gate_bias"] = c + "rg1", c + "rg1.b"
            names[p + "depth_mix"] = c + "dwa"
            if self.canon_taps:
                names[p + "mixer_conv"] = c + "canon1"
            if self.side_dim:
                names[p + "side_table"] = "side.embed"
                for w in ("gate", "proj", "norm"):
                    names[p + "side_" + w] = c + "side." + w
            if L.mlp is not None:
                names[p + "feed_forward_norm.weight"], names[p + "feed_forward_norm.bias"] = c + "norm2", c + "norm2.b"
                names[p + "feed_forward_gate"], names[p + "feed_forward_gate_bias"] = c + "rg2", c + "rg2.b"
                if L.mlp["kind"] == "dense":
                    names[p + "feed_forward.up"], names[p + "feed_forward.up_bias"] = c + "mlp.up", c + "mlp.up.b"
                    names[p + "feed_forward.down"], names[p + "feed_forward.down_bias"] = c + "mlp.down", c + "mlp.down.b"
                else:
                    names[p + "feed_forward.router"], names[p + "feed_forward.router_bias"] = c + "mlp.router", c + "mlp.router.b"
                    for e in range(L.mlp["router"]["experts"]):
                        for w in ("gate", "up", "down"):
                            names[p + f"feed_forward.e{e}.{w}"] = c + f"mlp.e{e}.{w}"
            m = p + "mixer."
            for w in ("q", "k", "v", "g", "o", "lq1", "lk1", "lq2", "lk2"):
                names[m + w] = c + f"mix.{w}"
            names[m + "q_norm"], names[m + "k_norm"] = c + "mix.q.norm", c + "mix.k.norm"
        return names

    def optional_tensor_names(self) -> set[str]:
        """A layer without a feed-forward reads no second norm and no second gate; a checkpoint may still hold them."""
        return {f"l{i}.{w}" for i, L in enumerate(self.layers) if L.mlp is None for w in ("norm2", "norm2.b", "rg2", "rg2.b")}

    def init_std(self) -> float:
        return self.initializer_range


register_architecture("Bisudra", BisudraConfig)
