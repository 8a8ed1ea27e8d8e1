"""Latent attention: keys and values of all heads are products of one small cached row per position.

    c_q = norm(W_dq x) ;  q_h = W_uq,h c_q                      queries through a latent of their own
    c   = norm(W_dkv x)                                        the only thing the cache keeps ([kv_rank] per position)
    k_h = W_uk,h c ;  v_h = W_uv,h c ;  score = scale q_h . k_h ;  softmax ;  o_h = sum p v_h ;  W_o on the heads

Since q_h . (W_uk,h c) = (W_uk,h^T q_h) . c and sum p (W_uv,h c) = W_uv,h (sum p c), the cache is never expanded:
the queries are carried into the latent space (one small product per head, all heads in one launch), attention runs with ONE key/value head
whose keys and values are both c (head size kv_rank, all query heads in its group), and the result is carried back
through W_uv,h.  That is grouped-query attention over a paged cache, so the attention kernels and the cache group
of ``GroupedQueryAttention`` serve it; the latent is stored twice, row-wise as the keys and transposed as the values.
Positions do not enter the scores.  The score scale is folded into c_q (everything after it is linear).

Options, all off by default.  ``q_rank=None``: the queries come straight from one projection, q = W_q x.  ``rot_dim`` > 0
with a rotary ``position``: every query head has ``rot_dim`` further dimensions behind its ``head_dim`` plain ones, and
W_dkv x has ``rot_dim`` further rows behind the latent's; both are rotated by the token's position (interleaved pairs;
cosine and sine times the encoding's ``magnitude``) and the rotated row of W_dkv x is one key part shared by all heads:
score = scale (q_plain . W_uk,h c + q_rot . k_rot).  The cache row is then [c | k_rot] as a key and [c | 0] as a value, and a
query in the latent space is [W_uk,h^T q_plain | q_rot]: still one key/value head and the same attention kernels.  The
per-head product that carries the queries has an identity block for the rotated part.  ``output_gate``: the
concatenated heads are multiplied by sigmoid(W_g x) before the output product; its rows ride in the first product."""

from __future__ import annotations

import torch

from ..cache.sequence_cache import KVCacheNeed, KVView
from ..config.base import ConfigError
from ..kernels import fast, ops
from ..weights.loader import ParamSpec
from .attention import kernel_head_dim
from .base import Mixer, StepContext, register_mixer
from .linear import Linear


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


class LatentAttention(Mixer):
    graph_safe = True
    pad_safe = True
    DECODE_GROUP = 16   # query heads per key/value head that the decode attention kernel takes

    def __init__(self, hidden_size: int, n_heads: int, head_dim: int, value_dim: int, kv_rank: int, q_rank: int | None,
                 norm_eps: float, scale: float | None = None, window: int | None = None, rot_dim: int = 0,
                 position=None, output_gate: bool = False):
        self.hidden_size, self.n_heads, self.key_dim, self.value_dim = hidden_size, n_heads, int(head_dim), int(value_dim)
        self.kv_rank, self.q_rank, self.norm_eps = int(kv_rank), (int(q_rank) if q_rank is not None else None), float(norm_eps)
        self.rot_dim, self.position, self.output_gate = int(rot_dim), position, bool(output_gate)
        self.scale = float(scale) if scale is not None else (self.key_dim + self.rot_dim) ** -0.5
        if min(self.kv_rank, self.q_rank or 1, self.key_dim, self.value_dim, n_heads) < 1 or self.rot_dim < 0:
            raise ConfigError("latent attention: every size must be positive")
        if self.rot_dim and (position is None or position.rotary_dim != self.rot_dim or self.rot_dim % 2
                             or position.pairing != 0):
            raise ConfigError(f"latent attention: {self.rot_dim} rotated dimensions need a rotary position encoding of "
                              "that size over interleaved pairs")
        if self.rot_dim and self.q_rank is not None:
            raise ConfigError("latent attention: rotated dimensions go with queries that come straight from a projection")
        # the sizes the attention kernels see: one key/value head as wide as the (widened) latent and the rotated part
        self.head_dim = kernel_head_dim(self.kv_rank + self.rot_dim)
        if self.head_dim > ops.MAX_HEAD_DIM:
            raise ConfigError(f"kv_rank {kv_rank} + rot_dim {rot_dim}: the attention kernels take rows of at most {ops.MAX_HEAD_DIM}")
        if window is not None and window < 1:
            raise ConfigError(f"window {window} must be at least 1 (or None for no window)")
        self.n_kv_heads, self.window = 1, window
        self.q_pad = _pad8(self.q_rank) if self.q_rank is not None else 0

    def children(self):
        return {"position": self.position} if self.position is not None else {}

    def parameters(self):
        H, dk, dv, h, dr = self.n_heads, self.key_dim, self.value_dim, self.hidden_size, self.rot_dim
        p = {"dkv": ParamSpec((self.kv_rank + dr, h)), "dkv_norm": ParamSpec((self.kv_rank,), "norm"),
             "uk": ParamSpec((H * dk, self.kv_rank)), "uv": ParamSpec((H * dv, self.kv_rank)), "o": ParamSpec((h, H * dv))}
        if self.q_rank is not None:
            p.update({"dq": ParamSpec((self.q_rank, h)), "dq_norm": ParamSpec((self.q_rank,), "norm"),
                      "uq": ParamSpec((H * dk, self.q_rank))})
        else:
            p["q"] = ParamSpec((H * (dk + dr), h))
        if self.output_gate:
            p["g"] = ParamSpec((H * dv, h))
        return p

    def cache_need(self):
        return KVCacheNeed(1, self.head_dim, self.window)

    def plan_decode(self, ctx: StepContext, cache: KVView) -> tuple[int, bool]:
        capacity = ctx.capacity(cache.group)
        if self.window:
            capacity = min(capacity, self.window)
        resident = ops.resident_ctas(ctx.device, self.head_dim, min(self.n_heads, self.DECODE_GROUP))
        splits = ops.attention_decode_splits(ctx.n_seqs, 1, capacity, resident)
        return splits, ops.attention_decode_early_start(ctx.n_seqs, 1, capacity, splits)

    def load(self, tensors, dtype, device):
        H, dk, dv, R, D, dr = self.n_heads, self.key_dim, self.value_dim, self.kv_rank, self.head_dim, self.rot_dim
        keep = lambda t: t.to(device).to(torch.float32 if dtype == torch.float32 else t.dtype)
        first = [keep(tensors["dq"] if self.q_rank is not None else tensors["q"]), keep(tensors["dkv"])]
        if self.output_gate:
            first.append(keep(tensors["g"]))
        common = torch.float32 if any(t.dtype == torch.float32 for t in first) else first[0].dtype
        rows, self.first_offsets, at = [], [], 0
        for t in first:     # the first product's rows: queries (or their latent), latent (and rotated key part), gate
            self.first_offsets.append(at)
            rows.append(t.to(common))
            pad = _pad8(t.shape[0]) - t.shape[0]
            if pad:
                rows.append(torch.zeros((pad, t.shape[1]), dtype=common, device=device))
            at += _pad8(t.shape[0])
        self.down = Linear(torch.cat(rows, dim=0).contiguous())
        uk, uv, o = (keep(tensors[n]) for n in ("uk", "uv", "o"))
        self.uq = Linear(keep(tensors["uq"]).contiguous()) if self.q_rank is not None else None
        # head h: queries into the latent space with W_uk,h^T (rows widened with zeros to D), the rotated part carried as
        # it is by an identity block; results back with W_uv,h
        uk_t = torch.zeros((H, D, dk + dr), dtype=uk.dtype, device=device)
        uk_t[:, :R, :dk] = uk.view(H, dk, R).transpose(1, 2)
        if dr:
            uk_t[:, R:R + dr, dk:] = torch.eye(dr, dtype=uk.dtype, device=device)
        uv_w = torch.zeros((H, dv, D), dtype=uv.dtype, device=device)
        uv_w[:, :, :R] = uv.view(H, dv, R)
        self.carry_in, self.carry_out = uk_t.contiguous(), uv_w.contiguous()   # [H, D, dk + dr] and [H, dv, D]
        self.o = Linear(o.contiguous())
        f32 = lambda n: tensors[n].to(device=device, dtype=torch.float32)
        mul = self.scale * D ** 0.5   # the attention kernels divide every score by sqrt(their head size)
        q_at, c_at = self.first_offsets[0], self.first_offsets[1]
        self.gate_at = self.first_offsets[2] if self.output_gate else None
        magnitude = float(getattr(self.position, "magnitude", 1.0)) if dr else 1.0
        seg, TO_K, TO_V = ops.head_row_segment, ops.TO_CACHE_KEYS, ops.TO_CACHE_VALUES
        if self.q_rank is not None:
            qr = self.q_rank
            self.norm_weights = torch.cat([f32("dq_norm"), f32("dkv_norm")]).contiguous()
            self.query_segment = ops.head_row_segments(seg(q_at, 1, qr, 0, self.q_pad, -1, True, 0, mul))   # c_q
            latent_weight = qr
        else:
            self.norm_weights = f32("dkv_norm").contiguous()
            # every head's plain part times the scale, its rotated part turned by the position (and times the scale)
            plain = seg(q_at, H, dk, 0, dk, mul=mul, src_stride=dk + dr, dst_stride=dk + dr)
            turned = seg(q_at + dk, H, dr, dk, dr, mul=mul * magnitude, rotate=True, src_stride=dk + dr, dst_stride=dk + dr)
            self.query_segment = ops.head_row_segments(*([plain, turned] if dr else [plain]))
            latent_weight = 0
        # c, once as (part of) a key row and once as a value row of its cache page; the rotated key part behind it
        latent = [seg(c_at, 1, R, 0, R if dr else D, -1, True, latent_weight, target=TO_K, cache_dim=D if dr else -1),
                  seg(c_at, 1, R, 0, D, -1, True, latent_weight, target=TO_V)]
        if dr:
            latent.append(seg(c_at + R, 1, dr, R, D - R, mul=magnitude, rotate=True, target=TO_K, cache_dim=D))
        self.latent_segments = ops.head_row_segments(*latent)

    def _rotary(self, ctx: StepContext):
        return (ctx.positions, self.position.inverse_frequencies(ctx.device)) if self.rot_dim else None

    def forward(self, x, ctx: StepContext, cache: KVView, residual, writes_cache=True, then_norm=None):
        H, dk, dv, D, T, dr = self.n_heads, self.key_dim, self.value_dim, self.head_dim, x.shape[0], self.rot_dim
        table = ctx.page_tables[cache.group]
        down = self.down.store(x, ctx.dtype, ctx.empty)                       # [T, queries (or q_rank) | kv_rank + rot_dim | gate]
        if writes_cache:
            ops.head_rows(down, None, self.latent_segments, self.norm_eps, None, self.norm_weights,
                          cache=(ctx.positions, ctx.seq_ids, table, cache.k, cache.v), rotary=self._rotary(ctx))
        if self.q_rank is not None:
            c_q = ctx.empty((T, self.q_pad), ctx.dtype)
            ops.head_rows(down, c_q, self.query_segment, self.norm_eps, None, self.norm_weights)
            q = self.uq.store(c_q[:, :self.q_rank], ctx.dtype, ctx.empty)     # [T, H dk]
        else:
            q = ctx.empty((T, H * (dk + dr)), ctx.dtype)
            ops.head_rows(down, q, self.query_segment, self.norm_eps, None, None, rotary=self._rotary(ctx))
        carried = ctx.empty((T, H * D), ctx.dtype)                            # queries in the latent space
        ops.gemm_per_head(q, self.carry_in, carried)
        heads = ctx.empty((T, H * dv), ctx.dtype)
        if ctx.all_decode and H > self.DECODE_GROUP and ops.attention_decode_supported(ctx.dtype, self.DECODE_GROUP, 1, D):
            # the decode kernel takes up to DECODE_GROUP query heads per key/value head: the heads go in groups, each
            # group over the same cached latents
            splits, early = self.plan_decode(ctx, cache)
            for g in range(0, H, self.DECODE_GROUP):
                n = min(self.DECODE_GROUP, H - g)
                part = ctx.empty((T, n * D), ctx.dtype)
                ops.attention_decode(carried[:, g * D:], carried.stride(0), part, ctx.kv_lens, table, cache.k, cache.v, n, 1,
                                     D, self.window or 0, splits, early_start=early)
                ops.gemm_per_head(part, self.carry_out[g:g + n], heads[:, g * dv:(g + n) * dv])
        else:
            out = ctx.empty((T, H * D), ctx.dtype)
            if not fast.try_attention(carried, out, ctx, table, cache, self):
                n_rows = T * H
                splits = 1 if n_rows >= 1024 else max(1, min(16, 1024 // n_rows, ctx.capacity(cache.group) // 512))
                ops.attention_paged(carried, carried.stride(0), out, ctx.positions, ctx.seq_ids, table, cache.k, cache.v,
                                    H, 1, D, self.window or 0, n_splits=splits)
            ops.gemm_per_head(out, self.carry_out, heads)
        if self.output_gate:
            ops.gate_rows(heads, down[:, self.gate_at:], "sigmoid")
        return self.o.add_to(heads, residual, then_norm)


register_mixer("latent_attention", LatentAttention)
