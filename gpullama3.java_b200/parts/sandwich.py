"""A block whose sublayers are normed on both sides, with an optional short convolution over time on what they read.

    h = norm_in(x) ;  h <- h + conv(h) ;  x <- x + mult * norm_out(sublayer(h))        for the mixer, then the feed-forward

``norm_in`` and ``norm_out`` are RMS norms (in groups or over the whole row), ``mult`` is one number for the whole
model, and conv is a causal convolution over the tokens of a sequence on every channel of the normed input,
conv(h)_t = sum_j w[:, j] h_(t - taps + 1 + j), with zeros before the sequence's start; its last taps - 1 inputs are
part of what a run of the block keeps per sequence (32-bit, beside the mixer's own cache or state).  A block built
without the convolution weights has none; one built without a feed-forward has the first line only.

The sublayer's last product adds into a 32-bit row buffer of the pass, as it would into the residual stream; one
kernel then norms that result into the stream, clears the buffer, adds the vector that enters the stream before the
next run (if the schedule names one) and norms the updated stream for whoever reads it next: the feed-forward of
this block, or the block that runs next (handed over as ``x_in``).  Norms, the convolution and the stream are 32-bit
in both precisions; what the convolution hands the sublayer's first product is rounded to the run's type."""
from __future__ import annotations

import torch

from ..cache.sequence_cache import EntryNeeds, StateNeed
from ..config.base import ConfigError
from ..kernels import ops
from ..weights.loader import ParamSpec
from .base import Block, FirstRead, ReadRows, StepContext, all_parts, register_block


class NormThenOffset:
    """What a block is handed as ``then_norm`` when a vector joins the stream between it and the next block, or when
    the next block's first read is left to this one (``read``, a ``FirstRead``)."""

    def __init__(self, norm, offset: torch.Tensor | None, read: FirstRead | None = None):
        self.norm, self.offset, self.read = norm, offset, read

    def row_factor_form(self):
        return None


class SandwichBlock(Block):
    def __init__(self, mixer, mixer_norm, mixer_out_norm, feed_forward=None, feed_forward_norm=None,
                 feed_forward_out_norm=None, *, hidden_size: int, residual_mult: float = 1.0, conv_taps: int = 0):
        """``conv_taps``: taps of the convolution on what each sublayer reads (0: none)."""
        if (feed_forward is None) != (feed_forward_norm is None) or (feed_forward is None) != (feed_forward_out_norm is None):
            raise ConfigError("a feed-forward and its two norms come together")
        if conv_taps and not (1 <= conv_taps <= ops.MAX_CONV_TAPS):
            raise ConfigError(f"conv taps {conv_taps}: the convolution kernel takes 1 to {ops.MAX_CONV_TAPS}")
        given = {"mixer": mixer, "mixer_norm": mixer_norm, "mixer_out_norm": mixer_out_norm, "feed_forward": feed_forward,
                 "feed_forward_norm": feed_forward_norm, "feed_forward_out_norm": feed_forward_out_norm}
        super().__init__(**{k: v for k, v in given.items() if v is not None})
        for k, v in given.items():
            setattr(self, k, v)
        for name, norm in given.items():
            if name.endswith("norm") and norm is not None and not hasattr(norm, "group_form"):
                raise ConfigError(f"{name}: this block takes RMS norms (over the row or in groups)")
        self.hidden_size, self.mult, self.taps = int(hidden_size), float(residual_mult), int(conv_taps)
        self.n_convs = (1 if feed_forward is None else 2) if self.taps else 0
        self.conv_floats = max(self.taps - 1, 0) * self.hidden_size     # per convolution and sequence
        self.conv_weights: list[torch.Tensor] = []

    # ---- parameters of the block itself: the convolutions
    def parameters(self):
        if not self.taps:
            return {}
        std = 0.5 / self.taps ** 0.5
        names = ["mixer_conv"] + (["feed_forward_conv"] if self.feed_forward is not None else [])
        return {n: ParamSpec((self.hidden_size, self.taps), "normal", 0.0, std) for n in names}

    def load(self, tensors, dtype, device):
        self.conv_weights = [tensors[n].to(device=device, dtype=torch.float32).contiguous() for n in self.parameters()]

    # ---- what a run keeps
    def cache_need(self):
        mixer = self.mixer.cache_need()
        if not self.n_convs or self.taps < 2:
            return mixer
        inputs = StateNeed((self.n_convs * self.conv_floats,), torch.float32)
        return EntryNeeds((("mixer", mixer), ("inputs", inputs)) if mixer is not None else (("inputs", inputs),))

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in all_parts(self).values())

    @property
    def pad_safe(self):
        # (with a convolution every token the block sees enters the inputs it keeps)
        return self.n_convs == 0 and all(p.pad_safe for p in all_parts(self).values())

    def first_norm(self):
        return self.mixer_norm

    def takes_scaled_rows(self, ctx: StepContext) -> bool:
        """The block takes its first normed input from the block before it (``x_in``) and leaves the next block's."""
        return True

    def with_offset(self, then_norm, row):
        return NormThenOffset(then_norm, row) if hasattr(then_norm, "group_form") else None

    def _one_kernel(self, ctx: StepContext, norm) -> bool:
        """Whether a step's last kernel may also read for whoever comes next: every sequence brings one token (its
        older inputs then all come from the state), and the rows are of a size that kernel keeps in registers."""
        return bool(self.taps) and ctx.all_decode and ops.sandwich_step_conv_fits(self.hidden_size, norm.group_form()[2])

    def _conv_state(self, which: int, inputs) -> torch.Tensor:
        if self.taps < 2:     # (one tap reads no earlier input: the kernels never look at the state)
            return self.conv_weights[which].view(1, -1)
        return inputs.data[:, which * self.conv_floats:(which + 1) * self.conv_floats]

    def first_read(self, ctx: StepContext, cache, writes_cache: bool):
        if not self._one_kernel(ctx, self.mixer_norm):
            return None
        inputs = cache.get("inputs") if isinstance(cache, dict) else None
        if self.taps > 1 and inputs is None:
            return None
        return FirstRead(self.conv_weights[0], self._conv_state(0, inputs), bool(writes_cache))

    def with_read(self, then_norm, read):
        if then_norm is None or read is None or not self.taps or read.weight.shape != (self.hidden_size, self.taps):
            return then_norm
        if isinstance(then_norm, NormThenOffset):
            then_norm.read = read
            return then_norm
        return NormThenOffset(then_norm, None, read) if hasattr(then_norm, "group_form") else then_norm

    # ---- one run
    def _read(self, normed: torch.Tensor, which: int, ctx: StepContext, inputs, writes: bool) -> torch.Tensor:
        """h + conv(h) of the normed rows (float32), rounded to the run's type for the sublayer's first product."""
        if not self.taps:
            return normed
        out = ctx.empty(normed.shape, ctx.dtype)
        state = self._conv_state(which, inputs)
        ops.causal_conv(normed, self.conv_weights[which], state, ctx.slots_dev, ctx.seq_ids, ctx.cu_seqlens, out,
                        self.hidden_size, add_input=True, update_state=writes and self.taps > 1)
        return out

    def forward(self, residual, ctx: StepContext, cache, writes_cache=True, x_in=None, then_norm=None):
        mixer_cache, inputs = cache, None
        if isinstance(cache, dict):
            mixer_cache, inputs = cache.get("mixer"), cache.get("inputs")
        # between norm and convolution the rows stay 32-bit; without a convolution they go straight to the product
        between = torch.float32 if self.taps else ctx.dtype
        y = ctx.extras.get("sandwich sublayer result")
        if y is None:
            y = ctx.extras["sandwich sublayer result"] = torch.zeros(residual.shape, dtype=torch.float32, device=residual.device)
        if isinstance(x_in, ReadRows):
            h = x_in.data    # (the block before this one has read for it: normed, convolved, the state moved on)
        else:
            if x_in is not None and x_in.dtype != between:
                x_in = None      # (handed over by a block that reads differently: norm again)
            x = x_in if x_in is not None else self.mixer_norm.forward(residual, between, alloc=ctx.empty)
            h = self._read(x, 0, ctx, inputs, writes_cache)
        self.mixer.forward(h, ctx, mixer_cache, y, writes_cache)
        last = self.mixer_out_norm
        if self.feed_forward is not None:
            if self._one_kernel(ctx, self.feed_forward_norm) and _agree(last, self.feed_forward_norm):
                read = FirstRead(self.conv_weights[1], self._conv_state(1, inputs), bool(writes_cache))
                h = self._step(y, last, residual, None, self.feed_forward_norm, between, ctx.empty, read, ctx).data
            else:
                h = self._read(self._step(y, last, residual, None, self.feed_forward_norm, between, ctx.empty), 1, ctx, inputs,
                               writes_cache)
            self.feed_forward.forward(h, ctx, y)
            last = self.feed_forward_out_norm
        offset = read = None
        if isinstance(then_norm, NormThenOffset):
            then_norm, offset, read = then_norm.norm, then_norm.offset, then_norm.read
        if then_norm is not None and not (hasattr(then_norm, "group_form") and _agree(then_norm, last)):
            assert offset is None    # (with_offset only wraps norms this block can apply)
            then_norm = read = None
        # (rows handed to the next block outlive this block's workspace: they come from the allocator)
        return self._step(y, last, residual, offset, then_norm, between,
                          lambda shape, dtype: torch.empty(shape, dtype=dtype, device=residual.device), read, ctx)

    def _step(self, y, out_norm, residual, offset, next_norm, dtype, alloc, read: FirstRead | None = None, ctx=None):
        """The sublayer's result into the stream; returns ``next_norm`` of the updated stream (with ``read``: a
        ``ReadRows`` of that norm's rows read for whoever comes next), or None without a norm."""
        w, eps, groups = out_norm.group_form()
        if read is not None and next_norm is not None and _agree(out_norm, next_norm) and self._one_kernel(ctx, next_norm):
            out = alloc(tuple(residual.shape), ctx.dtype)
            ops.sandwich_step_conv(y, w, self.mult, residual, eps, groups, next_norm.group_form()[0], out, read.weight,
                                   read.state, ctx.slots_dev, offset=offset, update_state=read.writes and self.taps > 1)
            return ReadRows(out)
        if next_norm is None:
            ops.sandwich_step(y, w, self.mult, residual, eps, groups, offset=offset)
            return None
        if not _agree(out_norm, next_norm):
            ops.sandwich_step(y, w, self.mult, residual, eps, groups, offset=offset)
            return next_norm.forward(residual, dtype, alloc=alloc)
        out = alloc(tuple(residual.shape), dtype)
        ops.sandwich_step(y, w, self.mult, residual, eps, groups, offset=offset, next_weight=next_norm.group_form()[0], out=out)
        return out


def _agree(a, b) -> bool:
    """Whether two norms cut their rows alike (one kernel can then apply both)."""
    return a.group_form()[1:] == b.group_form()[1:] and a.dim == b.dim


register_block("sandwich", SandwichBlock)
