"""Grouped-query causal attention over the paged cache: the mixer of the Llama 3 decoder.

One run: project the normalised input to queries, keys and values with one fused weight
(inference/InferenceCore.java:78-80 of the reference project computes the three separately),
rotate queries and keys and store keys and values at each token's position (:83-101), attend over
everything the sequence has cached up to each token (:106-145), project back and add to the
residual stream (:148-151).  Sizes, the position encoding and an optional window are parameters.

Further parameters, all off for Llama 3: biases of the three projections; an RMS norm without weight over every
query and key head; a score scale other than 1/sqrt(head size); a value size other than the key size; keys and values
taken from the cache another layer writes (the mixer then has no key and value projections).  With any of them on, a
kernel between the projection and the rotation finishes the heads (bias, norm, the scale folded into the queries) and
widens them with zeros to one size the attention kernels take; the output product's columns are widened to match.

More parameters of the same kind: an RMS norm with weights over the whole query projection and the whole key
projection, before they are split into heads (``projection_norm``); first positions that stay visible behind the window
(``keep_first``: i sees j when j <= i and (i - j < window or j < keep_first)); a distance penalty slope_h (i - j) taken
off every score with slope_h = 2^(-``distance_slope_base`` (h + 1) / heads); a learned number per head whose
exponential joins the softmax's denominator (``sink``); values mixed with those the first such layer of the pass made
for the same token, v <- (1 - l) v + l v_first with a learned l, the mixed values being what is cached (``value_mix``:
``"source"`` for that first layer, ``"mixed"`` for the others); and a gate per head, sigmoid(W_g x), on the heads'
outputs (``output_gate``)."""
from __future__ import annotations

import torch

from ..cache.sequence_cache import KVCacheNeed, KVView
from ..config.base import ConfigError
from ..kernels import fast, ops
from ..weights.loader import ParamSpec
from .base import Mixer, PositionEncoding, StepContext, register_mixer
from .linear import Linear


class GroupedQueryAttention(Mixer):
    graph_safe = True
    pad_safe = True

    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int, position: PositionEncoding,
                 window: int | None = None, *, value_dim: int | None = None, bias: bool = False,
                 qk_norm_eps: float | None = None, scale: float | None = None, shares_cache: bool = False,
                 cache_window="own", projection_norm: bool = False, keep_first: int = 0,
                 distance_slope_base: float | None = None, sink: bool = False, value_mix: str | None = None,
                 output_gate: bool = False):
        """``cache_window``: how many of the latest positions the cache entry keeps (``"own"``: this mixer's window);
        a layer whose cache other layers read with a longer window, or with none, is told so here."""
        if value_mix not in (None, "source", "mixed"):
            raise ConfigError(f"value_mix {value_mix!r}: None, 'source' or 'mixed'")
        if projection_norm and qk_norm_eps is None:
            raise ConfigError("projection_norm needs qk_norm_eps")
        if keep_first < 0 or (keep_first and window is None):
            raise ConfigError(f"keep_first {keep_first} needs a window (and cannot be negative)")
        if (value_mix or output_gate or projection_norm) and shares_cache:
            raise ConfigError("a mixer that reads another layer's cache has no values to mix, no gate and no weighted norm")
        self.projection_norm, self.keep_first, self.sink = bool(projection_norm), int(keep_first), bool(sink)
        self.distance_slope_base = float(distance_slope_base) if distance_slope_base is not None else None
        self.value_mix, self.output_gate = value_mix, bool(output_gate)
        # terms that only the attention kernels themselves can apply
        self.has_terms = bool(self.keep_first or self.sink or self.distance_slope_base is not None or self.output_gate)
        if n_heads % n_kv_heads:
            raise ConfigError(f"n_heads {n_heads} must be a multiple of n_kv_heads {n_kv_heads}")
        self.key_dim, self.value_dim = int(head_dim), int(value_dim if value_dim is not None else head_dim)
        self.bias, self.qk_norm_eps, self.shares_cache = bool(bias), qk_norm_eps, bool(shares_cache)
        self.scale = float(scale) if scale is not None else None
        self.finishes_heads = bool(self.bias or qk_norm_eps is not None or scale is not None or shares_cache
                                   or self.value_dim != self.key_dim or value_mix or self.has_terms
                                   or (self.key_dim % ops.HEAD_DIM_STEP != 0 and not position.rotary_dim))
        if self.finishes_heads:
            if min(self.key_dim, self.value_dim) < 1:
                raise ConfigError(f"head sizes must be positive, got {self.key_dim} and {self.value_dim}")
            head_dim = kernel_head_dim(max(self.key_dim, self.value_dim))
            if position.rotary_dim and head_dim != self.key_dim:
                raise ConfigError(f"a rotated head of {self.key_dim} cannot be widened to {head_dim}")
        # what no kernel takes is refused here, when the model is built, not at the first step
        if head_dim % ops.HEAD_DIM_STEP or not (0 < head_dim <= ops.MAX_HEAD_DIM):
            raise ConfigError(f"head_dim {head_dim}: the attention kernels take head sizes in steps of "
                              f"{ops.HEAD_DIM_STEP} up to {ops.MAX_HEAD_DIM}")
        if position.rotary_dim > min(head_dim, ops.MAX_ROTARY_DIM) or position.rotary_dim % 2:
            raise ConfigError(f"rotary_dim {position.rotary_dim} must be even and at most "
                              f"{min(head_dim, ops.MAX_ROTARY_DIM)} (head_dim {head_dim})")
        if window is not None and window < 1:
            raise ConfigError(f"window {window} must be at least 1 (or None for no window)")
        self.hidden_size, self.n_heads, self.n_kv_heads, self.head_dim = hidden_size, n_heads, n_kv_heads, head_dim
        self.position, self.window = position, window
        self.cache_window = window if cache_window == "own" else cache_window
        if self.cache_window is not None and (window is None or self.cache_window < window):
            raise ConfigError(f"a cache that keeps {self.cache_window} positions cannot serve a window of {window}")
        self.q_dim, self.kv_dim = n_heads * head_dim, n_kv_heads * head_dim
        self.qkv: Linear | None = None
        self.o: Linear | None = None
        self.head_bias = None
        self.segments = None
        self.norm_weights = self.sinks = self.slopes = self.mix_weight = None

    def parameters(self):
        H, G, dk, dv = self.n_heads, self.n_kv_heads, self.key_dim, self.value_dim
        p = {"q": ParamSpec((H * dk, self.hidden_size)), "o": ParamSpec((self.hidden_size, H * dv))}
        if not self.shares_cache:
            p["k"] = ParamSpec((G * dk, self.hidden_size))
            p["v"] = ParamSpec((G * dv, self.hidden_size))
        if self.bias:
            for n in ("q", "k", "v") if not self.shares_cache else ("q",):
                p[n + "_bias"] = ParamSpec(p[n].shape[:1], "matrix")
        if self.projection_norm:
            p["q_norm"], p["k_norm"] = ParamSpec((H * dk,), "norm"), ParamSpec((G * dk,), "norm")
        if self.sink:
            p["sink"] = ParamSpec((H,), "normal", 0.0, 1.0)
        if self.value_mix:
            p["vmix"] = ParamSpec((), "normal", 0.5, 0.1)    # (the source layer's is stored too, and not used)
        if self.output_gate:
            p["g"] = ParamSpec((H, self.hidden_size))
        return p

    def children(self):
        return {"position": self.position}

    def cache_need(self):
        return KVCacheNeed(self.n_kv_heads, self.head_dim, self.cache_window, self.keep_first if self.cache_window else 0)

    def plan_decode(self, ctx: StepContext, cache: KVView) -> tuple[int, bool]:
        """How a decode step's attention is launched (``plan_decode_attention``)."""
        return plan_decode_attention(self, ctx, cache)

    def load(self, tensors, dtype, device):
        if self.finishes_heads:
            return self._load_finished(tensors, dtype, device)
        q, k, v, o = (tensors[n].to(device) for n in ("q", "k", "v", "o"))
        common = torch.float32 if (dtype == torch.float32 or torch.float32 in (q.dtype, k.dtype, v.dtype)) else q.dtype
        self.qkv = Linear(torch.cat([q.to(common), k.to(common), v.to(common)], dim=0).contiguous())
        self.o = Linear(o.to(torch.float32 if dtype == torch.float32 else o.dtype).contiguous())

    def _load_finished(self, tensors, dtype, device):
        H, G, dk, dv, D = self.n_heads, self.n_kv_heads, self.key_dim, self.value_dim, self.head_dim
        names = ("q",) if self.shares_cache else ("q", "k", "v")
        mats = [tensors[n].to(device) for n in names]
        if self.output_gate:
            mats.append(tensors["g"].to(device))
        common = torch.float32 if (dtype == torch.float32 or any(m.dtype == torch.float32 for m in mats)) else mats[0].dtype
        rows = sum(m.shape[0] for m in mats)
        if rows % 8:   # the products' rows of 16-bit results start on 16-byte boundaries
            mats.append(torch.zeros((8 - rows % 8, self.hidden_size), dtype=common, device=device))
        self.qkv = Linear(torch.cat([m.to(common) for m in mats], dim=0).contiguous())
        self.value_off, self.gate_off = (H + G) * dk, (H + G) * dk + G * dv
        f32 = lambda n: tensors[n].to(device=device, dtype=torch.float32).contiguous()
        self.norm_weights = torch.cat([f32("q_norm"), f32("k_norm")]) if self.projection_norm else None
        self.sinks = f32("sink") if self.sink else None
        self.mix_weight = f32("vmix").reshape(1) if self.value_mix == "mixed" else None
        self.slopes = None
        if self.distance_slope_base is not None:
            self.slopes = torch.tensor([2.0 ** (-self.distance_slope_base * (h + 1) / H) for h in range(H)],
                                       dtype=torch.float64).to(device=device, dtype=torch.float32)
        o = tensors["o"].to(device)
        o = o.to(torch.float32 if dtype == torch.float32 else o.dtype)
        wide = torch.zeros((self.hidden_size, H, D), dtype=o.dtype, device=device)   # columns of the zeros behind a value head
        wide[:, :, :dv] = o.view(self.hidden_size, H, dv)
        self.o = Linear(wide.view(self.hidden_size, H * D).contiguous())
        if self.bias:
            self.head_bias = torch.cat([tensors[n + "_bias"].to(device=device, dtype=torch.float32) for n in names]).contiguous()
        # the scale is folded into the queries: the attention kernels divide every score by sqrt(their head size)
        mul = (self.scale if self.scale is not None else dk ** -0.5) * D ** 0.5
        norm = 0 if self.qk_norm_eps is None else 2 if self.projection_norm else 1
        wq, wk, per = (0, H * dk, True) if self.projection_norm else (-1, -1, False)
        b = (lambda off: off) if self.bias else (lambda off: -1)
        # without rotation the finished keys and values go straight into their cache pages; with it they go to the
        # dense rows that the rotation kernel reads
        direct = not self.position.rotary_dim
        keys, values = (ops.TO_CACHE_KEYS, ops.TO_CACHE_VALUES) if direct else (ops.TO_ROWS, ops.TO_ROWS)
        segs = [ops.head_row_segment(0, H, dk, 0, D, b(0), norm, wq, mul, weight_per_row=per)]
        if not self.shares_cache:
            segs.append(ops.head_row_segment(H * dk, G, dk, H * D, D, b(H * dk), norm, wk, target=keys, weight_per_row=per))
            # (mixed values: the other layer's rows are handed over as a view that starts at its values)
            segs.append(ops.head_row_segment((H + G) * dk, G, dv, (H + G) * D, D, b((H + G) * dk), target=values,
                                             mix_off=0 if self.value_mix == "mixed" else -1))
        self.segments = ops.head_row_segments(*segs)
        self.query_segment = ops.head_row_segments(segs[0])
        self.writes_direct = direct

    def takes_scaled_rows(self, ctx: StepContext) -> bool:
        return not self.finishes_heads and ctx.all_decode and self.qkv.links_with(ctx.n_tokens, ctx.dtype)

    def forward(self, x, ctx: StepContext, cache: KVView, residual, writes_cache=True, then_norm=None):
        table = ctx.page_tables[cache.group]
        out = ctx.empty((x.shape[0], self.q_dim), ctx.dtype)
        attended = False
        if self.finishes_heads:
            if writes_cache and self.shares_cache:
                raise ConfigError("a mixer without key and value projections cannot write a cache entry")
            # (the rows of a layer whose values later layers mix with theirs outlive the block: they come from the allocator)
            raw = self.qkv.store(x, ctx.dtype, ctx.empty if self.value_mix != "source" else None)
            mix = None
            if self.value_mix == "source":
                ctx.extras[VALUE_MIX_SOURCE] = raw[:, self.value_off:self.value_off + self.n_kv_heads * self.value_dim]
            elif self.value_mix == "mixed":
                if VALUE_MIX_SOURCE not in ctx.extras:
                    raise ConfigError("a layer mixes its values with an earlier layer's, and no earlier layer of the pass left any")
                mix = (ctx.extras[VALUE_MIX_SOURCE], self.mix_weight)
            if self.writes_direct:
                qkv = ctx.empty((x.shape[0], self.q_dim), ctx.dtype)
                ops.head_rows(raw, qkv, self.segments if writes_cache else self.query_segment, self.qk_norm_eps or 0.0,
                              self.head_bias, self.norm_weights, mix=mix if writes_cache else None,
                              cache=(ctx.positions, ctx.seq_ids, table, cache.k, cache.v) if writes_cache else None)
            else:
                qkv = ctx.empty((x.shape[0], self.q_dim + 2 * self.kv_dim), ctx.dtype)   # (a reader leaves the key and value columns unused)
                ops.head_rows(raw, qkv, self.segments, self.qk_norm_eps or 0.0, self.head_bias, self.norm_weights, mix=mix)
                ops.rope_cache_write(qkv, ctx.positions, ctx.seq_ids, table, self.position.inverse_frequencies(x.device),
                                     cache.k, cache.v, self.n_heads, self.n_kv_heads, self.head_dim,
                                     self.position.rotary_dim, self.position.pairing, write_cache=writes_cache)
        elif isinstance(x, torch.Tensor) and not ctx.all_decode:
            # a prompt pass: projection, rotation and cache write as one product where its epilogue can do all three
            qkv = ctx.empty((x.shape[0], self.qkv.out_features), ctx.dtype)
            if not fast.try_projection_with_rope(x, self.qkv.weight, qkv, ctx, table, cache, self, writes_cache):
                self.qkv.into(x, qkv)
                ops.rope_cache_write(qkv, ctx.positions, ctx.seq_ids, table, self.position.inverse_frequencies(x.device),
                                     cache.k, cache.v, self.n_heads, self.n_kv_heads, self.head_dim,
                                     self.position.rotary_dim, self.position.pairing, write_cache=writes_cache)
        else:
            qkv = self.qkv.store(x, ctx.dtype, ctx.empty)  # [T, q_dim + 2 kv_dim]; queries are rotated in place below
            # a decode step: one kernel rotates, writes the cache and attends, where the sizes allow
            attended = fast.try_decode_attention_with_rope(qkv, out, ctx, table, cache, self, writes_cache)
            if not attended:
                ops.rope_cache_write(qkv, ctx.positions, ctx.seq_ids, table, self.position.inverse_frequencies(x.device),
                                     cache.k, cache.v, self.n_heads, self.n_kv_heads, self.head_dim,
                                     self.position.rotary_dim, self.position.pairing, write_cache=writes_cache)
        gate = raw[:, self.gate_off:self.gate_off + self.n_heads] if self.output_gate else None
        if not attended:
            attend(self, qkv, out, ctx, table, cache, gate)
        return self.o.add_to(out, residual, then_norm)


def plan_decode_attention(shape, ctx: StepContext, cache: KVView) -> tuple[int, bool]:
    """How a decode step's attention is launched: into how many spans each sequence's keys are cut, and
    whether the kernel may be scheduled while its predecessor still runs.  Both follow from the number of
    sequences, the mixer's own kv heads and the longest sequence the step must be right for (its cache
    group's ``kv_capacity``: a recorded step is replayed until its page tables are outgrown).  ``shape``: whatever
    has ``n_heads``, ``n_kv_heads``, ``head_dim``, ``window`` and ``keep_first`` as the attention kernels are to see them."""
    capacity = ctx.capacity(cache.group)
    if shape.window:
        capacity = min(capacity, shape.window + shape.keep_first)
    resident = ops.resident_ctas(ctx.device, shape.head_dim, shape.n_heads // shape.n_kv_heads)
    splits = ops.attention_decode_splits(ctx.n_seqs, shape.n_kv_heads, capacity, resident)
    return splits, ops.attention_decode_early_start(ctx.n_seqs, shape.n_kv_heads, capacity, splits)


def attend(shape, qkv: torch.Tensor, out: torch.Tensor, ctx: StepContext, table: torch.Tensor, cache: KVView, gate=None) -> None:
    """Attention of the finished query rows in ``qkv`` over the paged cache into ``out``: a tensor-core kernel where one
    takes the sizes, else the plain kernel (a step of few tokens cuts their keys into spans so that the GPU has CTAs to
    run).  ``shape`` as for ``plan_decode_attention``, with ``plan_decode``, ``has_terms`` and the terms themselves
    (``slopes``, ``sinks``) where it has any."""
    if fast.try_attention(qkv, out, ctx, table, cache, shape, gate):
        return
    rows = qkv.shape[0] * shape.n_heads
    reach = ctx.capacity(cache.group) if not shape.window else min(ctx.capacity(cache.group), shape.window + shape.keep_first)
    splits = 1 if rows >= 1024 else max(1, min(16, 1024 // rows, reach // 512))
    ops.attention_paged(qkv, qkv.shape[1], out, ctx.positions, ctx.seq_ids, table, cache.k, cache.v,
                        shape.n_heads, shape.n_kv_heads, shape.head_dim, shape.window or 0, n_splits=splits,
                        keep_first=shape.keep_first, slopes=getattr(shape, "slopes", None), sinks=getattr(shape, "sinks", None),
                        gate=gate)


VALUE_MIX_SOURCE = "value mix source"   # in a pass's ``ctx.extras``: the first value-mixing layer's own values [T, G dv]


def kernel_head_dim(d: int) -> int:
    """The head size the attention kernels are given for heads of ``d``: the next size the tensor-core kernels take
    (steps of 32 up to 128), beyond that the next step of the plain kernel."""
    step = 32 if d <= 128 else ops.HEAD_DIM_STEP
    return -(-d // step) * step


register_mixer("attention", GroupedQueryAttention)
