"""Two mixers side by side: both read the same input; the block's mixer output is the mean of the two
outputs, each first RMS-normed over the model width with a gain of its own:

``y = (rms(left(x)) * g_left + rms(right(x)) * g_right) / 2``.

With ``combine="weighted"`` there are no norms and no gains: the output is ``left_scale * left(x) + right_scale *
right(x)``, handed on as a `ScaledSum` so that the block adds both terms into the 32-bit stream itself.

What the pair keeps between steps is what its members keep, side by side (the layer call then
names one cache entry per member that keeps something).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from emberserve_b200 import kernels as K
from emberserve_b200.parts.base import (Mixer, ParamSpec, Part, ScaledSum, Source, StepContext, build_part,
                                        register_part)


@dataclass(frozen=True)
class ParallelMixersSpec:
    hidden: int
    left: Any  # mixer specs
    right: Any
    eps: float = 0.0
    left_gain_name: str | None = None  # checkpoint tensors [hidden] (combine "normed_mean")
    right_gain_name: str | None = None
    kind: str = "parallel_mixers"
    combine: str = "normed_mean"  # or "weighted": left_scale * left + right_scale * right
    left_scale: float = 1.0
    right_scale: float = 1.0


def _as_tuple(need) -> tuple:
    return () if need is None else (need if isinstance(need, tuple) else (need,))


@register_part("mixer", "parallel_mixers")
class ParallelMixers(Mixer):
    left_gain: torch.Tensor
    right_gain: torch.Tensor

    def __init__(self, spec: ParallelMixersSpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        if spec.combine not in ("normed_mean", "weighted"):
            raise ValueError(f"combine {spec.combine!r}: 'normed_mean' or 'weighted'")
        if spec.combine == "normed_mean" and (spec.left_gain_name is None or spec.right_gain_name is None):
            raise ValueError("the normed mean of two mixers needs a gain for each")
        self.left = build_part("mixer", spec.left, prefix + ".left", self.shared)
        self.right = build_part("mixer", spec.right, prefix + ".right", self.shared)
        self._needs = (self.left.cache_need(), self.right.cache_need())

    def children(self) -> dict[str, Part]:
        return {"left": self.left, "right": self.right}

    def cache_need(self):
        flat = _as_tuple(self._needs[0]) + _as_tuple(self._needs[1])
        return None if not flat else (flat[0] if len(flat) == 1 else flat)

    def param_specs(self) -> dict[str, ParamSpec]:
        s: ParallelMixersSpec = self.spec
        if s.combine == "weighted":
            return {}
        return {"left_gain": ParamSpec((s.hidden,), [Source(s.left_gain_name)], init="ones"),
                "right_gain": ParamSpec((s.hidden,), [Source(s.right_gain_name)], init="ones")}

    def scratch_elements_per_token(self) -> int:
        return 2 * self.spec.hidden

    def _split(self, cache) -> tuple[Any, Any]:
        handles = list(_as_tuple(cache))
        out = []
        for need in self._needs:
            k = len(_as_tuple(need))
            mine, handles = handles[:k], handles[k:]
            out.append(None if need is None else (tuple(mine) if isinstance(need, tuple) else mine[0]))
        return out[0], out[1]

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: Any) -> torch.Tensor:
        s: ParallelMixersSpec = self.spec
        left_cache, right_cache = self._split(cache)
        a = self.left.forward(x, ctx, left_cache)
        if s.combine == "weighted":
            # (members of different kinds write to scratch buffers of different names)
            if type(self.left) is type(self.right):
                a = ctx.scratch("parallel_left", tuple(a.shape), a.dtype).copy_(a)
            b = self.right.forward(x, ctx, right_cache)
            return ScaledSum([(a, float(s.left_scale)), (b, float(s.right_scale))])
        if type(self.left) is type(self.right):  # two parts of one kind share their scratch buffers by name
            a = ctx.scratch("parallel_left", tuple(a.shape), a.dtype).copy_(a)
        b = self.right.forward(x, ctx, right_cache)
        out = ctx.scratch("parallel_out", (ctx.num_tokens, s.hidden), ctx.dtype)
        K.norm_mean2(a, b, self.left_gain, self.right_gain, s.eps, out)
        return out
