"""Arrangements of mixer, feed-forward and norms in one layer."""

from __future__ import annotations

from typing import Mapping, Optional

import torch

from tokensprint_b200 import ops
from tokensprint_b200.parts.base import (
    Block,
    BuildContext,
    CacheNeed,
    LayerCache,
    Normed,
    PartSpec,
    PreNormed,
    ResidualNorm,
    Rounded,
    StepContext,
    TensorSpec,
    build_part,
    register_part,
)


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    """h = h + Mixer(Norm_a(h)); h = h + FeedForward(Norm_f(h))  (engine/nn/layers.py:111-121).

    The residual stream is float32.  Each branch output is handed on as `pending` and
    added by the next norm in the same pass that norms it, so a residual sum never costs
    a pass over memory of its own.  A layer without a feed-forward ends with its mixer.
    """

    def __init__(self, ctx: BuildContext, *, mixer: PartSpec, mixer_norm: PartSpec, feed_forward: Optional[PartSpec] = None,
                 ffn_norm: Optional[PartSpec] = None) -> None:
        if (feed_forward is None) != (ffn_norm is None):
            raise ValueError("pre_norm block: a feed-forward and its norm come together")
        self.dtype = ctx.dtype
        self.mixer = build_part("mixer", mixer, ctx)
        self.feed_forward = None if feed_forward is None else build_part("feed_forward", feed_forward, ctx)
        self.mixer_norm = build_part("norm", mixer_norm, ctx)
        self.ffn_norm = None if ffn_norm is None else build_part("norm", ffn_norm, ctx)
        self._parts = tuple(p for p in (self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward) if p is not None)
        self.graph_safe = all(p.graph_safe for p in self._parts)
        # the block itself only hands tensors on; before a part that reads them by other means
        # than this package's ops, products that still wait in a chain are launched
        self.reads_through_ops = True

    def tensor_specs(self) -> list[TensorSpec]:
        return [s for p in self._parts for s in p.tensor_specs()]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for p in self._parts:
            p.load(tensors)

    def entry_norm(self):
        return self.mixer_norm

    def forward(self, hidden, pending, step: StepContext, cache: LayerCache):
        """`pending`: None, the last branch output not yet added to `hidden`, or a PreNormed that
        stands for mixer_norm(hidden) (the part before prepared it; `hidden` is then complete).

        Where mixer and feed-forward offer it (`folds_norms`, and `can_fold` for this step), the
        norms and residual sums between them are folded into their products: the mixer's last
        product adds into `hidden` and prepares the feed-forward's input, the feed-forward's last
        product does the same for `step.norm_after`.  Otherwise every norm is a step of its own."""
        T = hidden.shape[0]
        if isinstance(pending, Rounded):  # the block before handed on rounded rows, no branch: nothing to add
            pending = None
        after_block, norm_after = step.weight_after, step.norm_after
        mixer_folds = self.mixer.folds_norms and self.mixer.can_fold(T, self.dtype)
        ffn_folds = self.feed_forward is not None and self.feed_forward.folds_norms and self.feed_forward.can_fold(T, self.dtype)

        if isinstance(pending, PreNormed) and mixer_folds:
            x = pending
        elif isinstance(pending, Normed):  # the block before ran this block's first norm with its last kernel
            x = pending.x
        else:
            x = torch.empty(hidden.shape, device=hidden.device, dtype=self.dtype)
            self._before(self.mixer_norm)
            self.mixer_norm.forward(hidden, None if isinstance(pending, PreNormed) else pending, x)
        if self.feed_forward is None:
            self._before(self.mixer)
            return self.mixer.forward(x, step, cache)
        step.weight_after = self.feed_forward.first_weight()
        ffn_norm = self.ffn_norm.params()
        self._before(self.mixer)
        if mixer_folds and ffn_folds and ffn_norm is not None:
            x = self.mixer.forward(x, step, cache, fold=ResidualNorm(hidden, ffn_norm))
        else:
            mixed = self.mixer.forward(x, step, cache)
            x = torch.empty(hidden.shape, device=hidden.device, dtype=self.dtype)
            self._before(self.ffn_norm)
            self.ffn_norm.forward(hidden, mixed, x)
        step.weight_after = after_block
        next_norm = norm_after.params() if norm_after is not None else None
        self._before(self.feed_forward)
        if ffn_folds and next_norm is not None:
            return self.feed_forward.forward(x, step, fold=ResidualNorm(hidden, next_norm))
        return self.feed_forward.forward(x, step)

    @staticmethod
    def _before(part) -> None:
        if not part.reads_through_ops:
            ops.flush_gemm_chain()

    def first_weight(self):
        return self.mixer.first_weight()


@register_part("block", "post_norm")
class PostNormBlock(Block):
    """h = h + Norm_a(Mixer(h)); h = h + Norm_f(FeedForward(h)); h = h + Norm_e(Extra(h)).

    The norm sits on each sublayer's output and the sublayers read the residual stream itself.
    `feed_forward` and `extra` (a second feed-forward-like sublayer, for instance a per-layer
    token input) may each be absent.  The residual stream is float32; a sublayer reads its rows
    rounded to the compute dtype, which the norm kernel of the sublayer before writes in the same
    pass that adds into the stream (`Norm.forward_branch`), and the last one hands them to the
    next block as a `Rounded`.
    """

    def __init__(self, ctx: BuildContext, *, mixer: PartSpec, mixer_norm: PartSpec, feed_forward: Optional[PartSpec] = None,
                 ffn_norm: Optional[PartSpec] = None, extra: Optional[PartSpec] = None, extra_norm: Optional[PartSpec] = None) -> None:
        if (feed_forward is None) != (ffn_norm is None) or (extra is None) != (extra_norm is None):
            raise ValueError("post_norm block: a sublayer and its norm come together")
        self.dtype = ctx.dtype
        self.mixer = build_part("mixer", mixer, ctx)
        self.mixer_norm = build_part("norm", mixer_norm, ctx)
        self.feed_forward = None if feed_forward is None else build_part("feed_forward", feed_forward, ctx)
        self.ffn_norm = None if ffn_norm is None else build_part("norm", ffn_norm, ctx)
        self.extra = None if extra is None else build_part("feed_forward", extra, ctx)
        self.extra_norm = None if extra_norm is None else build_part("norm", extra_norm, ctx)
        self._parts = tuple(p for p in (self.mixer, self.mixer_norm, self.feed_forward, self.ffn_norm, self.extra, self.extra_norm) if p is not None)
        self.graph_safe = all(p.graph_safe for p in self._parts)
        self.reads_through_ops = True

    def tensor_specs(self) -> list[TensorSpec]:
        return [s for p in self._parts for s in p.tensor_specs()]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for p in self._parts:
            p.load(tensors)

    def first_weight(self):
        return self.mixer.first_weight()

    def _rows(self, hidden: torch.Tensor, pending) -> torch.Tensor:
        """The stream's rows in the compute dtype: the stream itself in a float32 run, else what the
        sublayer before left, else a rounding pass."""
        if self.dtype == torch.float32:
            return hidden
        if isinstance(pending, Rounded) and pending.x.dtype == self.dtype:
            return pending.x
        x = torch.empty(hidden.shape, device=hidden.device, dtype=self.dtype)
        ops.round_rows(hidden, x)
        return x

    def _add(self, norm, branch: torch.Tensor, hidden: torch.Tensor):
        PreNormBlock._before(norm)
        if self.dtype == torch.float32:
            norm.forward_branch(branch, hidden)
            return hidden
        x = torch.empty(hidden.shape, device=hidden.device, dtype=self.dtype)
        norm.forward_branch(branch, hidden, x)
        return x

    def forward(self, hidden, pending, step: StepContext, cache: LayerCache):
        if isinstance(pending, torch.Tensor):  # a branch that the block before did not add
            ops.residual_add(hidden, pending)
            pending = None
        x = self._rows(hidden, pending)
        after_block = step.weight_after
        step.weight_after = None
        PreNormBlock._before(self.mixer)
        x = self._add(self.mixer_norm, self.mixer.forward(x, step, cache), hidden)
        for part, norm in ((self.feed_forward, self.ffn_norm), (self.extra, self.extra_norm)):
            if part is None:
                continue
            PreNormBlock._before(part)
            branch = part.forward(x, step, residual=hidden) if part.wants_residual else part.forward(x, step)
            x = self._add(norm, branch, hidden)
        step.weight_after = after_block
        return None if self.dtype == torch.float32 else Rounded(x)


@register_part("block", "sandwich_norm")
class SandwichNormBlock(Block):
    """h = h + s_a * Norm_ao(Mixer(Norm_a(h))); h = h + s_f * Norm_fo(FeedForward(Norm_f(h))).

    Every sublayer stands between two norms, and what its output norm leaves is multiplied
    channel by channel by a learned scale (`mixer_scale`, `ffn_scale`: names of [width] vectors,
    or None) before it joins the float32 stream.  The feed-forward with its norms and scale may be
    absent.  The output norms are plain RMS norms; one kernel runs such a norm on the branch, the
    scale, the sum into the stream and the norm that reads the stream next (this block's
    feed-forward norm, or the first norm of the block that follows, which is then handed the
    finished rows as a `Normed`).

    `mixer_conv` / `ffn_conv` (names of [width, conv_taps] tensors): the sublayer does not read its
    normed input h but h + conv(h), a short causal convolution over time on every channel (the last
    tap weighs the current token, zeros before a sequence's start).  The last conv_taps - 1 normed
    inputs of either sublayer are then part of a request's state: the block keeps them in a slot of
    its own (`state_need`), so prompts may be cut anywhere."""

    def __init__(self, ctx: BuildContext, *, mixer: PartSpec, mixer_norm: PartSpec, mixer_out_norm: PartSpec, hidden_size: int,
                 mixer_scale: Optional[str] = None, feed_forward: Optional[PartSpec] = None, ffn_norm: Optional[PartSpec] = None,
                 ffn_out_norm: Optional[PartSpec] = None, ffn_scale: Optional[str] = None, mixer_conv: Optional[str] = None,
                 ffn_conv: Optional[str] = None, conv_taps: int = 0) -> None:
        if not ((feed_forward is None) == (ffn_norm is None) == (ffn_out_norm is None)):
            raise ValueError("sandwich_norm block: a feed-forward comes with both of its norms")
        if feed_forward is None and ffn_scale is not None:
            raise ValueError("sandwich_norm block: a scale without its feed-forward")
        self.dtype, self.hidden_size = ctx.dtype, int(hidden_size)
        self.mixer = build_part("mixer", mixer, ctx)
        self.mixer_norm = build_part("norm", mixer_norm, ctx)
        self.mixer_out_norm = build_part("norm", mixer_out_norm, ctx)
        self.feed_forward = None if feed_forward is None else build_part("feed_forward", feed_forward, ctx)
        self.ffn_norm = None if ffn_norm is None else build_part("norm", ffn_norm, ctx)
        self.ffn_out_norm = None if ffn_out_norm is None else build_part("norm", ffn_out_norm, ctx)
        self.scale_names = {"mixer": mixer_scale, "ffn": ffn_scale}
        if feed_forward is None and ffn_conv is not None:
            raise ValueError("sandwich_norm block: an input convolution without its feed-forward")
        self.conv_names = {"mixer": mixer_conv, "ffn": ffn_conv}
        self.conv_taps = int(conv_taps)
        if (mixer_conv is not None or ffn_conv is not None) and self.conv_taps < 1:
            raise ValueError("sandwich_norm block: input convolutions need conv_taps >= 1")
        self.conv_weights: dict[str, Optional[torch.Tensor]] = {"mixer": None, "ffn": None}
        # the slot's layout: the mixer's kept inputs [conv_taps - 1, width], then the feed-forward's
        self._conv_floats = (self.conv_taps - 1) * self.hidden_size if self.conv_taps > 1 else 0
        self._conv_offset = {"mixer": 0, "ffn": self._conv_floats if mixer_conv is not None else 0}
        self.mixer_scale: Optional[torch.Tensor] = None
        self.ffn_scale: Optional[torch.Tensor] = None
        self._parts = tuple(p for p in (self.mixer_norm, self.mixer, self.mixer_out_norm, self.ffn_norm, self.feed_forward, self.ffn_out_norm)
                            if p is not None)
        self.graph_safe = all(p.graph_safe for p in self._parts)
        self.reads_through_ops = True

    def tensor_specs(self) -> list[TensorSpec]:
        specs = [s for p in self._parts for s in p.tensor_specs()]
        specs += [TensorSpec(name, (self.hidden_size,), "vector") for name in self.scale_names.values() if name is not None]
        specs += [TensorSpec(name, (self.hidden_size, self.conv_taps), "vector") for name in self.conv_names.values() if name is not None]
        return specs

    def state_need(self):
        convs = sum(1 for name in self.conv_names.values() if name is not None)
        if not convs or not self._conv_floats:
            return None
        return CacheNeed(kind="none", state_shape=(convs * self._conv_floats,), state_dtype=torch.float32)

    def _input_conv(self, which: str, x: torch.Tensor, step: StepContext, cache: LayerCache) -> torch.Tensor:
        """x + conv(x) for the sublayer `which` (x itself where it has no convolution)."""
        w = self.conv_weights[which]
        if w is None:
            return x
        state = None
        if self._conv_floats:
            if cache.block_state is None:
                raise ops.KernelError("sandwich_norm block: its input convolutions need the block's state slots (none were bound)")
            first = self._conv_offset[which]
            state = cache.block_state.view(cache.block_state.shape[0], -1)[:, first:first + self._conv_floats]
        out = torch.empty(x.shape, device=x.device, dtype=self.dtype)
        ops.causal_conv(x, w, None, state, step.state_slots, step.cu_seqlens_q, step.seq_index, step.num_seqs, out, add_input=True)
        return out

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        for p in self._parts:
            p.load(tensors)
        if self.scale_names["mixer"] is not None:
            self.mixer_scale = tensors[self.scale_names["mixer"]]
        if self.scale_names["ffn"] is not None:
            self.ffn_scale = tensors[self.scale_names["ffn"]]
        for which, name in self.conv_names.items():
            if name is not None:
                self.conv_weights[which] = tensors[name].t().contiguous()  # tap by tap, as the kernel reads them
        for norm in (self.mixer_out_norm, self.ffn_out_norm):
            if norm is not None and norm.params() is None:
                raise ValueError("sandwich_norm block: the norm on a sublayer's output must be a plain RMS norm")

    def entry_norm(self):
        return self.mixer_norm

    def first_weight(self):
        return self.mixer.first_weight()

    def _close(self, branch: torch.Tensor, out_norm, scale: Optional[torch.Tensor], hidden: torch.Tensor, next_norm):
        """Output norm, scale and the sum into the stream; with `next_norm` (a plain RMS norm) also
        that norm of the new rows, which are returned."""
        p = out_norm.params()
        nxt = next_norm.params() if next_norm is not None else None
        if nxt is None:
            ops.branch_norm_add(branch, p.weight, scale, hidden, p.eps)
            return None
        out = torch.empty(hidden.shape, device=hidden.device, dtype=self.dtype)
        ops.branch_norm_add(branch, p.weight, scale, hidden, p.eps, next_weight=nxt.weight, out=out, next_eps=nxt.eps)
        return out

    def forward(self, hidden, pending, step: StepContext, cache: LayerCache):
        after_block, norm_after = step.weight_after, step.norm_after
        if isinstance(pending, torch.Tensor):  # a branch that the block before did not add
            ops.residual_add(hidden, pending)
            pending = None
        if isinstance(pending, Normed):
            x = pending.x
        else:  # the stream is complete (nothing pending, or rows prepared for a kernel this block does not use)
            x = torch.empty(hidden.shape, device=hidden.device, dtype=self.dtype)
            PreNormBlock._before(self.mixer_norm)
            self.mixer_norm.forward(hidden, None, x)
        ffn_first = self.feed_forward.first_weight() if self.feed_forward is not None else None
        step.weight_after = ffn_first if ffn_first is not None else after_block
        x = self._input_conv("mixer", x, step, cache)
        PreNormBlock._before(self.mixer)
        branch = self.mixer.forward(x, step, cache)
        step.weight_after = after_block
        if self.feed_forward is not None:
            x = self._close(branch, self.mixer_out_norm, self.mixer_scale, hidden, self.ffn_norm)
            if x is None:  # a feed-forward norm of another kind: a step of its own
                x = torch.empty(hidden.shape, device=hidden.device, dtype=self.dtype)
                PreNormBlock._before(self.ffn_norm)
                self.ffn_norm.forward(hidden, None, x)
            x = self._input_conv("ffn", x, step, cache)
            PreNormBlock._before(self.feed_forward)
            branch = self.feed_forward.forward(x, step)
            out = self._close(branch, self.ffn_out_norm, self.ffn_scale, hidden, norm_after)
        else:
            out = self._close(branch, self.mixer_out_norm, self.mixer_scale, hidden, norm_after)
        return None if out is None else Normed(out)
