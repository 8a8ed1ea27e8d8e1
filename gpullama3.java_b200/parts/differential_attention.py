"""Differential attention: every head attends twice over the same values and keeps the difference.

    q = W_q h  [H heads x 2 maps x d],  k = W_k h  [G kv heads x 2 maps x d],  v = W_v h  [G x dv]
    every (head, map) row of q and k: divided by its root mean square (eps inside the root), times a weight of d numbers
    shared by all heads and maps, then the first ``rotary_dim`` numbers turned by the token's position (the position part)
    a_m = softmax(scale q_m . k_m over the visible keys) v       for the maps m = 1, 2; query head h reads kv head h / (H / G)
    o = a_1 - lambda a_2,   lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff        (one number for the layer)
    o <- o / sqrt(mean(o^2) + eps) * (1 - diff)                                    (per head, over its dv numbers)
    out = W_o (o * sigmoid(W_g h))                                                 (``output_gate``)

How it runs on the kernels every attention mixer shares: a kv head's cache row holds the keys of both maps side by side
([k_1, k_2], widened with zeros to a size the attention kernels take), the 2 H maps are 2 H query heads whose rows are
zero outside their own map's columns ([q_1, 0] and [0, q_2]), so q . k over the whole row is the map's own score, both
maps read the one cached value row of their kv head, and nothing is cached twice.  One kernel between the projection
and attention finishes the rows (norm, weight, scale, rotation, placement, cache write); one behind attention takes the
difference, norms and gates.  lambda is made once at load, in 32 bits; scores, softmax, the norms and the difference are
32-bit in both precisions."""
from __future__ import annotations

import math

import torch

from ..cache.sequence_cache import KVCacheNeed, KVView
from ..config.base import ConfigError
from ..kernels import ops
from ..weights.loader import ParamSpec
from .attention import attend, kernel_head_dim, plan_decode_attention
from .base import Mixer, PositionEncoding, StepContext, register_mixer
from .linear import Linear


class _KernelShape:
    """The layer as the attention kernels see it: 2 H query heads over G kv heads of one widened size."""
    has_terms = False
    keep_first = 0

    def __init__(self, n_heads: int, n_kv_heads: int, head_dim: int, window: int | None):
        self.n_heads, self.n_kv_heads, self.head_dim, self.window = n_heads, n_kv_heads, head_dim, window

    def plan_decode(self, ctx: StepContext, cache: KVView):
        return plan_decode_attention(self, ctx, cache)


class DifferentialAttention(Mixer):
    graph_safe = True
    pad_safe = True

    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int, value_dim: int, scale: float,
                 diff: float, norm_eps: float, position: PositionEncoding, window: int | None = None,
                 output_gate: bool = True):
        """``head_dim``: numbers per map of a query or key head; ``diff``: the constant in lambda and in the factor
        (1 - diff) behind the heads' norm; ``window``: position i sees j with 0 <= i - j < window (None: every j <= i)."""
        if n_heads < 1 or n_kv_heads < 1 or n_heads % n_kv_heads:
            raise ConfigError(f"n_heads {n_heads} must be a multiple of n_kv_heads {n_kv_heads}")
        if min(head_dim, value_dim) < 1:
            raise ConfigError(f"head sizes must be positive, got {head_dim} and {value_dim}")
        if window is not None and window < 1:
            raise ConfigError(f"window {window} must be at least 1 (or None for no window)")
        if position.rotary_dim % 2 or position.rotary_dim > head_dim:
            raise ConfigError(f"rotary_dim {position.rotary_dim} must be even and at most the {head_dim} numbers of a map")
        if position.rotary_dim and position.pairing != 0:
            raise ConfigError("differential attention rotates interleaved pairs (2i, 2i + 1)")
        if head_dim % 2 and position.rotary_dim:
            raise ConfigError(f"a rotated map of {head_dim} numbers must be even")
        self.hidden_size, self.heads, self.kv_heads = int(hidden_size), int(n_heads), int(n_kv_heads)
        self.key_dim, self.value_dim = int(head_dim), int(value_dim)
        self.scale, self.diff, self.eps = float(scale), float(diff), float(norm_eps)
        self.position, self.window, self.output_gate = position, window, bool(output_gate)
        D = kernel_head_dim(max(2 * self.key_dim, self.value_dim))
        if D > ops.MAX_HEAD_DIM:
            raise ConfigError(f"two maps of {head_dim} or values of {value_dim} do not fit the attention kernels' "
                              f"{ops.MAX_HEAD_DIM} numbers per head")
        self.row_dim = D
        self.shape = _KernelShape(2 * self.heads, self.kv_heads, D, window)
        self.qkv: Linear | None = None
        self.o: Linear | None = None
        self.weight = 0.0

    def parameters(self):
        H, G, d, dv, h = self.heads, self.kv_heads, self.key_dim, self.value_dim, self.hidden_size
        p = {"q": ParamSpec((H * 2 * d, h)), "k": ParamSpec((G * 2 * d, h)), "v": ParamSpec((G * dv, h)),
             "o": ParamSpec((h, H * dv)), "q_norm": ParamSpec((d,), "norm"), "k_norm": ParamSpec((d,), "norm")}
        for n in ("lq1", "lk1", "lq2", "lk2"):
            p[n] = ParamSpec((d,), "normal", 0.0, 0.1)
        if self.output_gate:
            p["g"] = ParamSpec((H * dv, h))
        return p

    def children(self):
        return {"position": self.position}

    def cache_need(self):
        return KVCacheNeed(self.kv_heads, self.row_dim, self.window)

    def load(self, tensors, dtype, device):
        H, G, d, dv, D = self.heads, self.kv_heads, self.key_dim, self.value_dim, self.row_dim
        mats = [tensors[n].to(device) for n in (("q", "k", "v", "g") if self.output_gate else ("q", "k", "v"))]
        common = torch.float32 if (dtype == torch.float32 or any(m.dtype == torch.float32 for m in mats)) else mats[0].dtype
        rows = sum(m.shape[0] for m in mats)
        if rows % 8:   # the products' rows of 16-bit results start on 16-byte boundaries
            mats.append(torch.zeros((8 - rows % 8, self.hidden_size), dtype=common, device=device))
        self.qkv = Linear(torch.cat([m.to(common) for m in mats], dim=0).contiguous())
        o = tensors["o"].to(device)
        self.o = Linear(o.to(torch.float32 if dtype == torch.float32 else o.dtype).contiguous())
        f32 = lambda n: tensors[n].to(device=device, dtype=torch.float32).contiguous()
        self.norm_weights = torch.cat([f32("q_norm"), f32("k_norm")])
        # lambda, in 32 bits: two dot products, two exponentials
        first = torch.exp((f32("lq1") * f32("lk1")).sum())
        second = torch.exp((f32("lq2") * f32("lk2")).sum())
        self.weight = float((first - second + torch.tensor(self.diff, dtype=torch.float32, device=device)).item())
        # frequencies of the pairs of one map: those beyond the rotated part are 0 (an angle of 0 leaves a pair as it is)
        self.inv_freq = torch.zeros((max(d // 2, 1),), dtype=torch.float32, device=device)
        self.rotates = self.position.rotary_dim > 0
        if self.rotates:
            self.inv_freq[:self.position.rotary_dim // 2] = self.position.inverse_frequencies(device)[:self.position.rotary_dim // 2]
        # the scale is folded into the queries: the attention kernels divide every score by sqrt(their head size)
        mul = self.scale * math.sqrt(D)
        k_off, v_off = H * 2 * d, (H + G) * 2 * d
        self.gate_off = v_off + G * dv
        rot = self.rotates
        query = [ops.head_row_segment(m * d, H, d, m * D, D, norm=1, weight_off=0, mul=mul, rotate=rot, src_stride=2 * d,
                                      dst_stride=2 * D, lead=m * d) for m in (0, 1)]
        keys = [ops.head_row_segment(k_off + m * d, G, d, m * d, d if m == 0 else D - d, norm=1, weight_off=d, rotate=rot,
                                     src_stride=2 * d, target=ops.TO_CACHE_KEYS, cache_dim=D) for m in (0, 1)]
        values = ops.head_row_segment(v_off, G, dv, 0, D, target=ops.TO_CACHE_VALUES)
        self.segments = ops.head_row_segments(*query, *keys, values)
        self.query_segments = ops.head_row_segments(*query)

    def forward(self, x, ctx: StepContext, cache: KVView, residual, writes_cache=True, then_norm=None):
        H, dv, D = self.heads, self.value_dim, self.row_dim
        T = x.shape[0]
        table = ctx.page_tables[cache.group]
        raw = self.qkv.store(x, ctx.dtype, ctx.empty)
        q = ctx.empty((T, 2 * H * D), ctx.dtype)
        ops.head_rows(raw, q, self.segments if writes_cache else self.query_segments, self.eps, None, self.norm_weights,
                      cache=(ctx.positions, ctx.seq_ids, table, cache.k, cache.v) if writes_cache else None,
                      rotary=(ctx.positions, self.inv_freq) if self.rotates else None)
        maps = ctx.empty((T, 2 * H * D), ctx.dtype)
        attend(self.shape, q, maps, ctx, table, cache)
        out = ctx.empty((T, H * dv), ctx.dtype)
        gate = raw[:, self.gate_off:self.gate_off + H * dv] if self.output_gate else None
        ops.differential_heads(maps, gate, out, H, dv, D, self.weight, 1.0 - self.diff, self.eps)
        return self.o.add_to(out, residual, then_norm)


register_mixer("differential_attention", DifferentialAttention)
