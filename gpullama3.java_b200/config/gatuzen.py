"""Typed configuration of the Gatuzen decoder, read from ``config.json``.

A Gatuzen model is a list of layers over one residual stream.  Every sublayer is normed on both sides with an RMS norm in
``norm.groups`` equal parts (``norm.eps``), reads its normed input plus a causal convolution of ``canon.taps`` taps over it,
and joins the stream times ``residual_mult``.  The embedding rows are multiplied with ``embedding.scale``; the logits
with ``logit_scale``; the output head is a matrix of its own.

* ``layers[i].type`` names the mixer, ``layers[i].mixer`` gives its sizes:
  ``gla``: gated linear attention (``heads``, ``dim``, ``vdim``, decay temperature ``tau``);
  ``mamba2``: the state-space mixer with a scalar decay per head (``heads``, ``vdim``, ``state``, ``groups``, ``conv`` taps,
  ``norm_groups``);
  ``latent_attention``: causal softmax attention whose keys and values are products of one cached latent row
  (``heads``, ``dim`` plain and ``rot_dim`` rotated dimensions per head, ``vdim``, ``kv_rank``, score ``scale``, ``rot`` with
  ``base``, ``dims`` and optional ``scaling`` {``factor``, ``original``, ``fast``, ``slow``}), with a gate on its output;
* ``layers[i].mlp`` is null or ``{"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}}``: a mixture of SiLU-gated
  experts chosen by a table from token id to experts, each weighted 1 / top;
* ``loop`` {``start``, ``stop``, ``times``}: layers start .. stop - 1 run ``times`` times in a row with the same weights and a
  cache or state of their own per pass; row t of ``loop.step`` joins the stream right before pass t.

Constants the design fixes stand here: the slope of the rotary magnitude in ln(factor) and the least width of the
frequency ramp."""
from __future__ import annotations

from dataclasses import dataclass

from .base import ConfigError, LayerSpec, ModelConfig, PartSpec, ScheduleEntry, as_float, as_int, require_keys
from .registry import register_architecture

MIXER_TYPES = ("gla", "mamba2", "latent_attention")
ROTARY_MAGNITUDE_SLOPE = 0.1     # cosine and sine are multiplied by 0.1 ln(factor) + 1
ROTARY_MIN_RAMP_WIDTH = 0.001
MIXER_KEYS = {"gla": ["heads", "dim", "vdim", "tau"],
              "mamba2": ["heads", "vdim", "state", "groups", "conv", "norm_groups"],
              "latent_attention": ["heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot"]}
FLOAT_KEYS = ("tau", "scale")


def _positive(d: dict, key: str, where: str) -> float:
    v = as_float(d, key)
    if not v > 0:
        raise ConfigError(f"{where}: {key} must be positive, got {v}")
    return v


@dataclass(frozen=True)
class GatuzenLayer:
    type: str
    mixer: dict        # the mixer's record as config.json has it (checked when read)
    mlp: dict | None   # the feed-forward's record, None for a layer without one


@dataclass(frozen=True)
class GatuzenConfig(ModelConfig):
    vocab_size: int
    hidden_size: int
    layers: tuple
    norm_eps: float
    norm_groups: int = 1
    canon_taps: int = 0
    embed_scale: float = 1.0
    logit_scale: float = 1.0
    residual_mult: float = 1.0
    loop: tuple | None = None          # (start, stop, times)
    initializer_range: float = 0.02
    tie_word_embeddings: bool = False
    stop_token_ids: tuple[int, ...] = ()

    architecture = "Gatuzen"

    # ---- reading
    @classmethod
    def from_dict(cls, d: dict) -> "GatuzenConfig":
        require_keys(d, ["vocab", "width", "layers", "norm"], "Gatuzen config.json")
        if not isinstance(d["layers"], list) or not d["layers"]:
            raise ConfigError("Gatuzen config.json: 'layers' must be a non-empty list")
        if not isinstance(d["norm"], dict):
            raise ConfigError("Gatuzen config.json: 'norm' must be an object with 'eps' (and 'groups')")
        require_keys(d["norm"], ["eps"], "Gatuzen norm")
        eps = _positive(d["norm"], "eps", "norm")
        groups = as_int(d["norm"], "groups") if d["norm"].get("groups") is not None else 1
        width = as_int(d, "width")
        if width % groups:
            raise ConfigError(f"norm: width {width} cannot be cut into {groups} equal parts")

        def number(record, key, default):
            if not isinstance(record, dict) or record.get(key) is None:
                return default
            return as_float(record, key)

        canon = d.get("canon") or {}
        if not isinstance(canon, dict):
            raise ConfigError("Gatuzen config.json: 'canon' must be an object with 'taps'")
        taps = as_int(canon, "taps", minimum=0) if canon.get("taps") is not None else 0
        layers = []
        for i, L in enumerate(d["layers"]):
            where = f"layer {i}"
            if not isinstance(L, dict) or not isinstance(L.get("mixer"), dict):
                raise ConfigError(f"{where}: needs 'type' and a 'mixer' object")
            kind, m = L.get("type"), dict(L["mixer"])
            if kind not in MIXER_TYPES:
                raise ConfigError(f"{where}: unknown mixer type {kind!r}; known: {', '.join(MIXER_TYPES)}")
            require_keys(m, MIXER_KEYS[kind], where)
            for key in MIXER_KEYS[kind]:
                if key in FLOAT_KEYS:
                    _positive(m, key, where)
                elif key != "rot":
                    as_int(m, key, minimum=0 if key == "rot_dim" else 1)
            if kind == "latent_attention":
                m["rot"] = cls._checked_rotation(m["rot"], m["rot_dim"], where)
            if kind == "mamba2" and m["heads"] % m["groups"]:
                raise ConfigError(f"{where}: {m['heads']} heads do not share {m['groups']} groups equally")
            mlp = L.get("mlp")
            if mlp is not None:
                mlp = cls._checked_mlp(mlp, where)
            layers.append(GatuzenLayer(kind, m, mlp))
        loop = d.get("loop")
        if loop is not None:
            if not isinstance(loop, dict):
                raise ConfigError("Gatuzen config.json: 'loop' must be an object with 'start', 'stop' and 'times'")
            require_keys(loop, ["start", "stop", "times"], "Gatuzen loop")
            start, stop, times = as_int(loop, "start", minimum=0), as_int(loop, "stop", minimum=0), as_int(loop, "times")
            if not (start < stop <= len(layers)):
                raise ConfigError(f"loop: layers {start} .. {stop - 1} of {len(layers)}")
            loop = (start, stop, times)
        eos = d.get("eos_token_id")
        stop_ids = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        return cls(vocab_size=as_int(d, "vocab"), hidden_size=width, layers=tuple(layers), norm_eps=eps, norm_groups=groups,
                   canon_taps=taps, embed_scale=number(d.get("embedding"), "scale", 1.0),
                   logit_scale=number(d, "logit_scale", 1.0), residual_mult=number(d, "residual_mult", 1.0), loop=loop,
                   initializer_range=float(d.get("initializer_range", 0.02)), stop_token_ids=stop_ids)

    @staticmethod
    def _checked_rotation(rot, rot_dim: int, where: str) -> dict:
        if not isinstance(rot, dict):
            raise ConfigError(f"{where}: rot must be an object with 'base' and 'dims'")
        require_keys(rot, ["base", "dims"], where + " rot")
        out = {"base": _positive(rot, "base", where + " rot"), "dims": as_int(rot, "dims", minimum=0)}
        if out["dims"] != rot_dim or rot_dim % 2:
            raise ConfigError(f"{where}: the {rot_dim} rotated dimensions are rotated whole, in pairs (rot.dims {out['dims']})")
        s = rot.get("scaling")
        if s is not None:
            if not isinstance(s, dict):
                raise ConfigError(f"{where}: rot.scaling must be an object")
            require_keys(s, ["factor", "original", "fast", "slow"], where + " rot.scaling")
            out["scaling"] = {k: _positive(s, k, where + " rot.scaling") for k in ("factor", "original", "fast", "slow")}
        return out

    @staticmethod
    def _checked_mlp(mlp, where: str) -> dict:
        if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
            raise ConfigError(f"{where}: mlp must be null or an object of kind 'moe', got {mlp!r}")
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
             "embedding": {"scale": self.embed_scale}, "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
             "canon": {"taps": self.canon_taps}, "logit_scale": self.logit_scale, "residual_mult": self.residual_mult,
             "initializer_range": self.initializer_range,
             "layers": [{"type": L.type, "mixer": dict(L.mixer), "mlp": dict(L.mlp) if L.mlp else None} for L in self.layers]}
        if self.loop is not None:
            d["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        if self.stop_token_ids:
            d["eos_token_id"] = list(self.stop_token_ids)
        return d

    # ---- the model as data
    def embedding_scale(self) -> float:
        return self.embed_scale

    def output_scale(self) -> float:
        return self.logit_scale

    def pass_offsets(self) -> int:
        return self.loop[2] if self.loop is not None else 0

    def _norm(self) -> PartSpec:
        return PartSpec("norm", "rmsnorm", {"dim": self.hidden_size, "eps": self.norm_eps, "groups": self.norm_groups})

    def _mixer(self, i: int) -> PartSpec:
        L = self.layers[i]
        m, h = L.mixer, self.hidden_size
        if L.type == "gla":
            return PartSpec("mixer", "gla", {"hidden_size": h, "n_heads": m["heads"], "head_dim": m["dim"],
                                             "value_dim": m["vdim"], "decay_temperature": float(m["tau"]),
                                             "norm_eps": self.norm_eps, "decay_rank": m.get("decay_rank")})
        if L.type == "mamba2":
            return PartSpec("mixer", "ssd", {"hidden_size": h, "n_heads": m["heads"], "value_dim": m["vdim"],
                                             "state_dim": m["state"], "n_groups": m["groups"], "conv_taps": m["conv"],
                                             "norm_eps": self.norm_eps, "norm_groups": m["norm_groups"]})
        rot, position = m["rot"], None
        if m["rot_dim"]:
            s = rot.get("scaling") or {}
            position = PartSpec("position", "yarn", {
                "rotary_dim": m["rot_dim"], "base": rot["base"], "factor": s.get("factor"), "original": s.get("original"),
                "fast": s.get("fast", 32.0), "slow": s.get("slow", 1.0), "magnitude_slope": ROTARY_MAGNITUDE_SLOPE,
                "min_ramp_width": ROTARY_MIN_RAMP_WIDTH})
        return PartSpec("mixer", "latent_attention", {
            "hidden_size": h, "n_heads": m["heads"], "head_dim": m["dim"], "value_dim": m["vdim"], "kv_rank": m["kv_rank"],
            "q_rank": None, "norm_eps": self.norm_eps, "scale": float(m["scale"]), "rot_dim": m["rot_dim"],
            "position": position, "output_gate": True})

    def _feed_forward(self, mlp: dict) -> PartSpec:
        return PartSpec("feed_forward", "routed", {
            "hidden_size": self.hidden_size, "intermediate_size": mlp["expert"]["ff"], "n_experts": mlp["router"]["experts"],
            "top": mlp["router"]["top"], "activation": "silu", "router": "table", "vocab_size": self.vocab_size})

    def layer_specs(self) -> list[LayerSpec]:
        specs = []
        for i, L in enumerate(self.layers):
            parts = {"mixer": self._mixer(i), "mixer_norm": self._norm(), "mixer_out_norm": self._norm()}
            if L.mlp is not None:
                parts.update(feed_forward=self._feed_forward(L.mlp), feed_forward_norm=self._norm(),
                             feed_forward_out_norm=self._norm())
            specs.append(LayerSpec("sandwich", parts, {"hidden_size": self.hidden_size, "residual_mult": self.residual_mult,
                                                       "conv_taps": self.canon_taps}))
        return specs

    def schedule(self) -> list[ScheduleEntry]:
        """Layers before the loop, the looped layers once per pass (a cache entry of their own each time, the pass's
        offset before its first layer), the layers behind it."""
        n = len(self.layers)
        if self.loop is None:
            return [ScheduleEntry(layer=i, cache=i) for i in range(n)]
        start, stop, times = self.loop
        runs = [(i, None) for i in range(start)]
        for t in range(times):
            runs += [(i, t if i == start else None) for i in range(start, stop)]
        runs += [(i, None) for i in range(stop, n)]
        return [ScheduleEntry(layer=i, cache=k, enters=t) for k, (i, t) in enumerate(runs)]

    def final_norm(self) -> PartSpec:
        return self._norm()

    def tensor_names(self) -> dict[str, str]:
        names = {"embedding.table": "embed", "final_norm.weight": "final.norm", "head.weight": "head"}
        if self.loop is not None:
            names["pass_offsets.table"] = "loop.step"
        for i, L in enumerate(self.layers):
            p, c = f"layers.{i}.", f"l{i}."
            names[p + "mixer_norm.weight"], names[p + "mixer_out_norm.weight"] = c + "norm1", c + "norm1b"
            if self.canon_taps:
                names[p + "mixer_conv"] = c + "canon1"
            if L.mlp is not None:
                names[p + "feed_forward_norm.weight"], names[p + "feed_forward_out_norm.weight"] = c + "norm2", c + "norm2b"
                if self.canon_taps:
                    names[p + "feed_forward_conv"] = c + "canon2"
                names[p + "feed_forward.table"] = c + "mlp.table"
                for e in range(L.mlp["router"]["experts"]):
                    for w in ("gate", "up", "down"):
                        names[p + f"feed_forward.e{e}.{w}"] = c + f"mlp.e{e}.{w}"
            m = p + "mixer."
            if L.type == "gla":
                for w in ("q", "k", "v", "g", "o", "norm", "a1", "a2"):
                    names[m + w] = c + f"mix.{w}"
                names[m + "a2_bias"] = c + "mix.a2.b"
            elif L.type == "mamba2":
                for w in ("in", "conv", "dt_bias", "A_log", "D", "norm", "o"):
                    names[m + w] = c + f"mix.{w}"
                names[m + "conv_bias"] = c + "mix.conv.b"
            else:
                for w in ("q", "dkv", "uk", "uv", "g", "o"):
                    names[m + w] = c + f"mix.{w}"
                names[m + "dkv_norm"] = c + "mix.dkv.norm"
        return names

    def optional_tensor_names(self) -> set[str]:
        """A layer without a feed-forward reads no second pair of norms and no second convolution; a checkpoint may
        still hold them."""
        return {f"l{i}.{w}" for i, L in enumerate(self.layers) if L.mlp is None for w in ("norm2", "norm2b", "canon2")}

    def init_std(self) -> float:
        return self.initializer_range


register_architecture("Gatuzen", GatuzenConfig)
