"""A block whose sublayers read the residual stream itself and whose results are gated, normed and then added.

    h = x ;  h' = h + conv(h)                         (optional: a causal convolution over time on what the mixer reads)
    x <- x + norm_1( mixer(h') * sigmoid(W_1 h + b_1) )
    h = x
    x <- x + norm_2( feed_forward(h) * sigmoid(W_2 h + b_2) )                      (a layer may have no feed-forward)
    e = table[token][this layer's columns] ;  y = W_p (gelu_tanh(W_s x) * e) ;  x <- x + w_s * y / rms(y)      (optional:
        a few learned numbers per (token id, layer), gated by the stream, projected to its width and normed)
    level[i + 1] = x ;  x <- sum_(j <= i + 1) c[j] level[j]                         (optional: level[0] is what the first
        block of the pass was handed, level[j + 1] the result of the j-th block; the next block, or the final norm,
        reads a learned mix of all of them)

conv(h)_t = sum_j w[:, j] h_(t - taps + 1 + j) with zeros before the sequence's start; its last taps - 1 inputs are part
of what a run of the block keeps per sequence (32-bit, beside the mixer's cache).  norm_1 and norm_2 are the norm parts
the block is built with (layer norms with weight and bias, or RMS norms); the gates read the sublayer's own input before
the convolution.  A sublayer's last product adds into a 32-bit row buffer of the pass; one kernel then gates and norms
that result into the stream, clears the buffer and leaves the updated stream in the run's type for the products that
read it next (the gate's, the feed-forward's, the next block's); the last such kernel of a layer also files the layer's
result as a level and leaves the mix over the levels as the stream, and in a step in which every sequence brings one
token it applies the next block's input convolution too (that block then launches none).  The stream, the gates' logits and sigmoid, the norms,
the convolution with its state and the mix over the levels are 32-bit in both precisions."""
from __future__ import annotations

import torch

from ..cache.sequence_cache import EntryNeeds, StateNeed
from ..config.base import ConfigError
from ..kernels import ops
from ..weights.loader import ParamSpec
from .base import Block, FirstRead, StepContext, all_parts, register_block
from .linear import Linear

SUBLAYER_RESULT = "gated residual sublayer result"   # in a pass's ``ctx.extras``: float32 [T, width], zero between uses
DEPTH_LEVELS = "gated residual depth levels"         # float32 [levels, T, width]: what every block of the pass left


class StreamRows:
    """What a block hands the next one: the residual stream as it now stands, in the run's type; ``read``: what the next
    block's mixer reads (its convolution applied, its state moved on), when this block's last kernel did that too."""

    def __init__(self, data: torch.Tensor, read: torch.Tensor | None = None):
        self.data, self.read = data, read


class NoNorm:
    """What the block answers when asked for its first norm: it has none (its sublayers read the stream itself), but it
    takes part in the hand-over between blocks, which is keyed on that question."""

    def row_factor_form(self):
        return None


class ReadAhead:
    """``then_norm`` of a block whose successor offered its first read (a ``FirstRead``): no norm, only the read."""

    def __init__(self, read: FirstRead):
        self.read = read

    def row_factor_form(self):
        return None


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


def _reads_rows_of(read: FirstRead, width: int) -> bool:
    """Whether a first read is a convolution over rows of ``width`` numbers with 32-bit weights and state."""
    return (read.weight.dim() == 2 and read.weight.shape[0] == width and read.weight.dtype == torch.float32
            and read.state.dtype == torch.float32)


class GatedResidualBlock(Block):
    def __init__(self, mixer, mixer_norm, feed_forward=None, feed_forward_norm=None, *, hidden_size: int, conv_taps: int = 0,
                 side_dim: int = 0, side_columns: tuple[int, int] = (0, 0), vocab_size: int = 0, side_eps: float = 1e-5,
                 depth: tuple[int, int] | None = None):
        """``conv_taps``: taps of the convolution on what the mixer reads (0: none).  ``side_dim``: numbers per (token id,
        layer) of the token input (0: none), which are columns ``side_columns[0]`` .. + side_dim of a table
        [vocab_size, side_columns[1]] that all layers share.  ``depth``: (this block's place among the blocks of a pass
        whose results are mixed, how many such blocks the pass has); None: the block leaves its own result."""
        if (feed_forward is None) != (feed_forward_norm is None):
            raise ConfigError("a feed-forward and the norm of its result come together")
        if conv_taps and not (1 <= conv_taps <= ops.MAX_CONV_TAPS):
            raise ConfigError(f"conv taps {conv_taps}: the convolution kernel takes 1 to {ops.MAX_CONV_TAPS}")
        if side_dim and not (vocab_size > 0 and 0 <= side_columns[0] and side_columns[0] + side_dim <= side_columns[1]):
            raise ConfigError(f"token input: columns {side_columns[0]} .. + {side_dim} of a table [{vocab_size}, {side_columns[1]}]")
        if depth is not None and not (0 <= depth[0] < depth[1]):
            raise ConfigError(f"depth {depth}: a place among the blocks of a pass and their number")
        given = {"mixer": mixer, "mixer_norm": mixer_norm, "feed_forward": feed_forward, "feed_forward_norm": feed_forward_norm}
        super().__init__(**{k: v for k, v in given.items() if v is not None})
        for k, v in given.items():
            setattr(self, k, v)
        for name in ("mixer_norm", "feed_forward_norm"):
            if given[name] is not None and not hasattr(given[name], "weight"):
                raise ConfigError(f"{name}: this block takes norms with a weight per channel (and a bias, or none)")
        self.hidden_size, self.taps, self.side_dim = int(hidden_size), int(conv_taps), int(side_dim)
        self.side_columns, self.vocab_size, self.side_eps = (int(side_columns[0]), int(side_columns[1])), int(vocab_size), float(side_eps)
        self.depth = None if depth is None else (int(depth[0]), int(depth[1]))
        self.conv_floats = max(self.taps - 1, 0) * self.hidden_size
        self.conv_weight = None

    # ---- parameters of the block itself
    def parameters(self):
        h = self.hidden_size
        p = {}
        if self.taps:
            p["mixer_conv"] = ParamSpec((h, self.taps), "normal", 0.0, 0.5 / self.taps ** 0.5)
        names = ["mixer"] + (["feed_forward"] if self.feed_forward is not None else [])
        for n in names:
            p[n + "_gate"] = ParamSpec((h, h))
            p[n + "_gate_bias"] = ParamSpec((h,), "normal", 0.0, 0.5)
        if self.side_dim:
            p["side_table"] = ParamSpec((self.vocab_size, self.side_columns[1]), "normal", 0.0, 1.0)
            p["side_gate"] = ParamSpec((self.side_dim, h))
            p["side_proj"] = ParamSpec((h, self.side_dim))
            p["side_norm"] = ParamSpec((h,), "norm")
        if self.depth is not None:
            p["depth_mix"] = ParamSpec((self.depth[0] + 2,), "normal", 1.0 / (self.depth[0] + 2), 0.2)
        return p

    def load(self, tensors, dtype, device):
        run = lambda w: w.to(device).to(torch.float32 if dtype == torch.float32 else w.dtype).contiguous()
        f32 = lambda n: tensors[n].to(device=device, dtype=torch.float32).contiguous()
        h = self.hidden_size
        if self.taps:
            self.conv_weight = f32("mixer_conv")
        self.gates, self.gate_biases = [Linear(run(tensors["mixer_gate"]))], [f32("mixer_gate_bias")]
        if self.feed_forward is not None:
            self.gates.append(Linear(run(tensors["feed_forward_gate"])))
            self.gate_biases.append(f32("feed_forward_gate_bias"))
        if self.side_dim:
            n, lo = self.side_dim, self.side_columns[0]
            self.side_k = _pad8(n)     # rows of 16-bit numbers that products read start on 16-byte boundaries
            self.side_table = run(tensors["side_table"][:, lo:lo + n])
            gate, proj = run(tensors["side_gate"]), run(tensors["side_proj"])
            wide_gate = torch.zeros((self.side_k, h), dtype=gate.dtype, device=device)
            wide_gate[:n] = gate
            wide_proj = torch.zeros((h, self.side_k), dtype=proj.dtype, device=device)
            wide_proj[:, :n] = proj
            self.side_gate, self.side_proj, self.side_norm = Linear(wide_gate), Linear(wide_proj), f32("side_norm")
        if self.depth is not None:
            self.depth_mix = f32("depth_mix")
            self.first_level = torch.ones((1,), dtype=torch.float32, device=device)

    # ---- what a run keeps
    def cache_need(self):
        mixer = self.mixer.cache_need()
        if self.taps < 2:
            return mixer
        inputs = StateNeed((self.conv_floats,), torch.float32)
        return EntryNeeds((("mixer", mixer), ("inputs", inputs)) if mixer is not None else (("inputs", inputs),))

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in all_parts(self).values())

    @property
    def pad_safe(self):
        # (with a convolution every token the block sees enters the inputs it keeps)
        return self.taps < 2 and all(p.pad_safe for p in all_parts(self).values())

    def takes_scaled_rows(self, ctx: StepContext) -> bool:
        """The block takes the stream in the run's type from the block before it (``x_in``) and leaves it for the next."""
        return True

    def first_norm(self):
        return NoNorm()

    def first_read(self, ctx: StepContext, cache, writes_cache: bool):
        """In a step in which every sequence brings one token all older inputs of the convolution come from the state:
        the block before may then read for this block's mixer in its own last kernel."""
        if not (self.taps and ctx.all_decode):
            return None
        inputs = cache.get("inputs") if isinstance(cache, dict) else None
        if self.taps > 1 and inputs is None:
            return None
        state = inputs.data if self.taps > 1 else self.conv_weight.view(1, -1)
        return FirstRead(self.conv_weight, state, bool(writes_cache))

    def with_read(self, then_norm, read):
        if read is None or not _reads_rows_of(read, self.hidden_size):
            return then_norm
        return ReadAhead(read) if isinstance(then_norm, NoNorm) else then_norm

    # ---- one run
    def forward(self, residual, ctx: StepContext, cache, writes_cache=True, x_in=None, then_norm=None):
        T, h = residual.shape
        mixer_cache, inputs = cache, None
        if isinstance(cache, dict):
            mixer_cache, inputs = cache.get("mixer"), cache.get("inputs")
        y = ctx.extras.get(SUBLAYER_RESULT)
        if y is None:
            y = ctx.extras[SUBLAYER_RESULT] = torch.zeros((T, h), dtype=torch.float32, device=residual.device)
        x = x_in.data if isinstance(x_in, StreamRows) else None
        levels = None
        if self.depth is not None:
            index, total = self.depth
            levels = ctx.extras.get(DEPTH_LEVELS)
            if levels is None or index == 0:
                # the first block of the pass: what it was handed is level 0 (the same kernel leaves the stream in the run's type)
                levels = ctx.extras[DEPTH_LEVELS] = torch.empty((total + 1, T, h), dtype=torch.float32, device=residual.device)
                x = ctx.empty((T, h), ctx.dtype)
                ops.depth_average(levels, 0, self.first_level, residual, cast=x)
            elif levels.shape[0] < index + 2:
                raise ConfigError(f"block {index} of a pass follows blocks that keep {levels.shape[0]} levels")
        if x is None:
            x = ctx.empty((T, h), ctx.dtype)
            ops.cast_rows(residual, x)
        # what the next block reads outlives this block's workspace: it comes from the allocator
        last = torch.empty((T, h), dtype=ctx.dtype, device=residual.device)
        stages = ["mixer"] + (["feed_forward"] if self.feed_forward is not None else []) + (["side"] if self.side_dim else [])

        def cast_behind(stage: str):
            """Where the kernel that ends ``stage`` leaves the updated stream in the run's type."""
            return ctx.empty((T, h), ctx.dtype) if stage != stages[-1] else last

        def mix_behind(stage: str) -> dict:
            """The layer's last kernel also files the layer's result as a level and leaves the mix over the levels, and
            in a step of one token per sequence reads for the next block's mixer."""
            if stage != stages[-1]:
                return {}
            more = dict(read=ahead) if ahead is not None else {}
            if self.depth is not None:
                more.update(levels=levels, n=self.depth[0] + 1, coefficients=self.depth_mix)
            return more

        ahead = None      # the next block's mixer input, if this block's last kernel is to make it
        if isinstance(then_norm, ReadAhead) and ctx.all_decode:
            r = then_norm.read
            ahead = (r.weight, r.state, ctx.slots_dev, r.writes and r.weight.shape[1] > 1,
                     torch.empty((T, h), dtype=ctx.dtype, device=residual.device))
        read = x
        if self.taps and isinstance(x_in, StreamRows) and x_in.read is not None:
            read = x_in.read     # (the block before this one has read for it: convolved, the state moved on)
        elif self.taps:
            read = ctx.empty((T, h), ctx.dtype)
            state = inputs.data if self.taps > 1 else self.conv_weight.view(1, -1)   # (one tap reads no earlier input)
            ops.causal_conv(residual, self.conv_weight, state, ctx.slots_dev, ctx.seq_ids, ctx.cu_seqlens, read, h,
                            add_input=True, update_state=bool(writes_cache) and self.taps > 1)
        self.mixer.forward(read, ctx, mixer_cache, y, writes_cache)
        x = self._join(y, x, 0, self.mixer_norm, residual, ctx, cast=cast_behind("mixer"), **mix_behind("mixer"))
        if self.feed_forward is not None:
            y_bias = None
            if hasattr(self.feed_forward, "result_bias"):    # (its last bias joins in the kernel that reads the result anyway)
                self.feed_forward.forward(x, ctx, y, add_result_bias=False)
                y_bias = self.feed_forward.result_bias()
            else:
                self.feed_forward.forward(x, ctx, y)
            x = self._join(y, x, 1, self.feed_forward_norm, residual, ctx, y_bias=y_bias, cast=cast_behind("feed_forward"),
                           **mix_behind("feed_forward"))
        if self.side_dim:
            a = self.side_gate.store(x, ctx.dtype, ctx.empty)
            g = ctx.empty((T, self.side_k), ctx.dtype)
            ops.token_gate_rows(a, ctx.tokens, self.side_table, g, self.side_dim)
            self.side_proj.add_to(g, y)
            ops.gated_norm_step(y, self.side_norm, None, residual, self.side_eps, center=False, cast=cast_behind("side"),
                                **mix_behind("side"))
        return StreamRows(last, ahead[4] if ahead is not None else None)

    def _join(self, y, x, which: int, norm, residual, ctx: StepContext, y_bias=None, cast=None, **mix):
        """The sublayer's result ``y`` times its gate (a product over the sublayer's input ``x``), normed, into the
        stream; returns ``cast``, which then holds the updated stream in the run's type."""
        bias = getattr(norm, "bias", None)
        w = norm.weight if norm.weight.dtype == torch.float32 else norm.group_form()[0]
        r = self.gates[which].store(x, torch.float32, ctx.empty)    # (the gate's logits leave their product in 32 bits)
        ops.gated_norm_step(y, w, bias, residual, norm.eps, gate=r, gate_bias=self.gate_biases[which], y_bias=y_bias, cast=cast,
                            center=bias is not None, **mix)
        return cast


register_block("gated_residual", GatedResidualBlock)
