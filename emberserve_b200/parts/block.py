"""Residual blocks.

Pre-norm: ``h += mixer(norm1(h)); h += ffn(norm2(h))`` (a layer without a feed-forward is its first half);
behind the sub-layers a block may run parts that act on the stream itself (``stream_parts``, in order).
Sandwich (a norm before AND behind every sub-layer, optionally a short convolution before the
mixer, optionally no feed-forward): ``h += norm1b(mixer(conv(norm1(h)))); h += norm2b(ffn(norm2(h)))``.

Shared-input (``SharedInputBlock``): both sub-layers read norms of the SAME stream and their outputs join it
together, times a constant: ``h += m * (mixer(norm1(h)) + ffn(norm2(h)))``.

Written on the pair (delta, residual) so that each norm performs the add that precedes
it (``emberserve/model/qwen2.py:122-164``): the block receives the previous block's
output `delta`, which has not been added to the stream yet, and returns its own.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from emberserve_b200 import kernels as K
from emberserve_b200.parts.base import (Block, CacheNeed, NormedDelta, Part, ScaledSum, StepContext, StreamPart,
                                        build_part, register_part)


@dataclass(frozen=True)
class PreNormBlockSpec:
    mixer: Any
    feed_forward: Any  # None: the block is its mixer alone
    mixer_norm: Any
    ffn_norm: Any
    kind: str = "prenorm"
    stream_parts: tuple = ()  # specs of category "stream", run in order behind the sub-layers


@register_part("block", "prenorm")
class PreNormBlock(Block):
    def __init__(self, spec: PreNormBlockSpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        self.mixer_norm = build_part("norm", spec.mixer_norm, prefix + ".mixer_norm", self.shared)
        self.mixer = build_part("mixer", spec.mixer, prefix + ".mixer", self.shared)
        self.ffn = self.ffn_norm = None
        if spec.feed_forward is not None:
            self.ffn_norm = build_part("norm", spec.ffn_norm, prefix + ".ffn_norm", self.shared)
            self.ffn = build_part("feed_forward", spec.feed_forward, prefix + ".ffn", self.shared)
        self.stream_parts = [build_part("stream", sp, f"{prefix}.stream{j}", self.shared)
                             for j, sp in enumerate(spec.stream_parts)]

    def children(self) -> dict[str, Part]:
        out = {"mixer_norm": self.mixer_norm, "mixer": self.mixer}
        if self.ffn is not None:
            out.update(ffn_norm=self.ffn_norm, ffn=self.ffn)
        for j, part in enumerate(self.stream_parts):
            out[f"stream{j}"] = part
        return out

    def cache_need(self) -> CacheNeed | None:
        return self.mixer.cache_need()

    def entry_norm(self):
        return self.mixer_norm if self.mixer.splits_norms else None

    def forward(self, delta: torch.Tensor | None, residual: torch.Tensor, ctx: StepContext,
                cache: Any) -> torch.Tensor:
        if not self.stream_parts:
            return self._sublayers(delta, residual, ctx, cache)
        ctx.extra["next_norm"] = None  # (the stream parts stand between this block's last product and that norm)
        if delta is not None and any(type(p).on_entry is not StreamPart.on_entry for p in self.stream_parts):
            raise TypeError(f"{self.prefix}: its stream parts read the stream on entry, so the block before "
                            f"must leave nothing to be added")
        for part in self.stream_parts:
            part.on_entry(residual, ctx)
        delta = self._sublayers(delta, residual, ctx, cache)
        for part in self.stream_parts:
            delta = part.forward(delta, residual, ctx)
        return delta

    def _sublayers(self, delta: torch.Tensor | None, residual: torch.Tensor, ctx: StepContext,
                   cache: Any) -> torch.Tensor:
        # A sub-layer whose successor takes `ScaledRows` is asked to begin the norm that follows
        # it in its last product (ctx.extra["norm_behind"]); what it returns says whether it did.
        after_ffn = ctx.extra.pop("next_norm", None)  # the next block's entry norm, from the decoder
        x = self.mixer_norm.forward(delta, residual, ctx)
        if self.ffn is None:
            ctx.extra["norm_behind"] = (after_ffn.split_request(residual, ctx)
                                        if after_ffn is not None and self.mixer.splits_norms else None)
            a = self.mixer.forward(x, ctx, cache)
            ctx.extra["norm_behind"] = None
            return a
        ctx.extra["norm_behind"] = (self.ffn_norm.split_request(residual, ctx)
                                    if self.mixer.splits_norms and self.ffn.splits_norms else None)
        a = self.mixer.forward(x, ctx, cache)
        y = self.ffn_norm.forward(a, residual, ctx)
        ctx.extra["norm_behind"] = (after_ffn.split_request(residual, ctx)
                                    if after_ffn is not None and self.ffn.splits_norms else None)
        out = self.ffn.forward(y, ctx)
        ctx.extra["norm_behind"] = None
        return out


@dataclass(frozen=True)
class SandwichBlockSpec:
    mixer: Any
    mixer_norm: Any
    mixer_post_norm: Any
    feed_forward: Any | None = None  # None: the block is its mixer alone
    ffn_norm: Any | None = None
    ffn_post_norm: Any | None = None
    mixer_conv: Any | None = None  # spec of a "conv" part that filters what the mixer reads
    kind: str = "sandwich"


@register_part("block", "sandwich")
class SandwichBlock(Block):
    """A sub-layer's output passes a norm of its own before it joins the stream.  That norm, the
    32-bit add and the norm in front of the NEXT sub-layer are one kernel: the block hands its
    output on as a `NormedDelta`, and the norm that receives it does all three.  What the block
    keeps between steps is the mixer's cache entry and, with a convolution, its state: two entries
    per layer call."""

    def __init__(self, spec: SandwichBlockSpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        self.mixer_norm = build_part("norm", spec.mixer_norm, prefix + ".mixer_norm", self.shared)
        self.mixer = build_part("mixer", spec.mixer, prefix + ".mixer", self.shared)
        self.mixer_post_norm = build_part("norm", spec.mixer_post_norm, prefix + ".mixer_post_norm", self.shared)
        self.conv = (build_part("conv", spec.mixer_conv, prefix + ".mixer_conv", self.shared)
                     if spec.mixer_conv is not None else None)
        self.ffn = self.ffn_norm = self.ffn_post_norm = None
        if spec.feed_forward is not None:
            if spec.ffn_norm is None or spec.ffn_post_norm is None:
                raise ValueError(f"{prefix}: a feed-forward needs its two norms")
            self.ffn_norm = build_part("norm", spec.ffn_norm, prefix + ".ffn_norm", self.shared)
            self.ffn = build_part("feed_forward", spec.feed_forward, prefix + ".ffn", self.shared)
            self.ffn_post_norm = build_part("norm", spec.ffn_post_norm, prefix + ".ffn_post_norm", self.shared)
        self._conv_state = self.conv is not None and self.conv.cache_need() is not None

    def children(self) -> dict[str, Part]:
        out = {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "mixer_post_norm": self.mixer_post_norm}
        if self.conv is not None:
            out["mixer_conv"] = self.conv
        if self.ffn is not None:
            out.update(ffn_norm=self.ffn_norm, ffn=self.ffn, ffn_post_norm=self.ffn_post_norm)
        return out

    def cache_need(self):
        need = self.mixer.cache_need()
        if not self._conv_state:
            return need
        state = self.conv.cache_need()
        return (need, state) if need is not None else state

    def forward(self, delta, residual: torch.Tensor, ctx: StepContext, cache: Any):
        ctx.extra.pop("next_norm", None)
        mixer_cache, conv_cache = cache, None
        if self._conv_state:
            mixer_cache, conv_cache = cache if isinstance(cache, tuple) else (None, cache)
        x = self.mixer_norm.forward(delta, residual, ctx)
        if self.conv is not None:
            x = self.conv.forward(x, ctx, conv_cache)
        a = NormedDelta(self.mixer.forward(x, ctx, mixer_cache), self.mixer_post_norm)
        if self.ffn is None:
            return a
        y = self.ffn_norm.forward(a, residual, ctx)
        return NormedDelta(self.ffn.forward(y, ctx), self.ffn_post_norm)


@dataclass(frozen=True)
class SharedInputBlockSpec:
    mixer: Any
    mixer_norm: Any  # spec of a one-group RMS norm ("rmsnorm_grouped")
    feed_forward: Any | None = None  # None: the block is its mixer alone
    ffn_norm: Any | None = None
    residual_mult: float = 1.0  # m: what the block adds to the stream is multiplied by it
    kind: str = "shared_input"


@register_part("block", "shared_input")
class SharedInputBlock(Block):
    """``h += m * (mixer(norm1(h)) + ffn(norm2(h)))``: the two norms differ in their gains only, so one
    kernel adds what the block before left (a tensor or a `ScaledSum`) into the 32-bit stream, takes
    the root mean square once and writes both normed inputs.  The block hands its own outputs on as a
    `ScaledSum`, unrounded: a mixer may itself return a `ScaledSum` (two mixers side by side with
    weights), whose terms are then multiplied by m."""

    def __init__(self, spec: SharedInputBlockSpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        self.mixer_norm = build_part("norm", spec.mixer_norm, prefix + ".mixer_norm", self.shared)
        self.mixer = build_part("mixer", spec.mixer, prefix + ".mixer", self.shared)
        self.ffn = self.ffn_norm = None
        if spec.feed_forward is not None:
            if spec.ffn_norm is None:
                raise ValueError(f"{prefix}: a feed-forward needs its norm")
            self.ffn_norm = build_part("norm", spec.ffn_norm, prefix + ".ffn_norm", self.shared)
            self.ffn = build_part("feed_forward", spec.feed_forward, prefix + ".ffn", self.shared)
        for norm in (self.mixer_norm, self.ffn_norm):
            if norm is not None and (getattr(norm.spec, "kind", None) != "rmsnorm_grouped" or norm.spec.groups != 1):
                raise ValueError(f"{prefix}: the two norms share their statistics, so each is a one-group RMS norm")
        if self.ffn_norm is not None and (self.ffn_norm.spec.eps != self.mixer_norm.spec.eps
                                          or self.ffn_norm.spec.gain_offset != self.mixer_norm.spec.gain_offset):
            raise ValueError(f"{prefix}: the two norms must agree in eps and gain offset")

    def children(self) -> dict[str, Part]:
        out = {"mixer_norm": self.mixer_norm, "mixer": self.mixer}
        if self.ffn is not None:
            out.update(ffn_norm=self.ffn_norm, ffn=self.ffn)
        return out

    def cache_need(self):
        return self.mixer.cache_need()

    def scratch_elements_per_token(self) -> int:
        return 2 * self.mixer_norm.spec.dim

    def forward(self, delta, residual: torch.Tensor, ctx: StepContext, cache: Any):
        ctx.extra.pop("next_norm", None)
        ctx.extra["norm_behind"] = None
        ns = self.mixer_norm.spec
        if delta is None:
            terms = []
        elif isinstance(delta, ScaledSum):
            terms = delta.terms
        elif isinstance(delta, torch.Tensor):
            terms = [(delta, 1.0)]
        else:
            raise TypeError(f"{self.prefix}: cannot take a delta of type {type(delta).__name__}")
        n = residual.shape[0]
        x1 = ctx.scratch("normed", (n, ns.dim), ctx.dtype)
        x2 = ctx.scratch("normed_second", (n, ns.dim), ctx.dtype) if self.ffn is not None else None
        K.add_scaled_norm2(terms, residual, self.mixer_norm.weight, None if self.ffn is None else self.ffn_norm.weight,
                           ns.gain_offset, ns.eps, x1, x2)
        m = float(self.spec.residual_mult)
        a = self.mixer.forward(x1, ctx, cache)
        out = a.scaled(m) if isinstance(a, ScaledSum) else ScaledSum([(a, m)])
        if self.ffn is not None:
            out = ScaledSum(out.terms + [(self.ffn.forward(x2, ctx), m)])
        if len(out.terms) > 3:
            raise ValueError(f"{self.prefix}: at most three terms join the stream at once")
        return out
