"""A short causal convolution over time on every channel, by default added to its input:

``out[t] = h[t] + sum_j w[:, j] * h[t - taps + 1 + j]`` with ``h = 0`` before a request's
first token; with ``identity=False`` the input itself is not added, and a bias per channel may be.  The last ``taps - 1`` inputs of a request are state that lives between steps
(``FixedState((taps - 1, width))``, float32), so a portion of a prompt or a single decoded
token continues where the step before stopped.  A block puts it between a norm and a mixer.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from emberserve_b200 import kernels as K
from emberserve_b200.parts.base import (FixedState, FixedStateHandle, ParamSpec, Part, Source, StepContext,
                                        register_part)


@dataclass(frozen=True)
class CausalTapsSpec:
    width: int
    taps: int
    weight_name: str  # checkpoint tensor [width, taps]; column taps - 1 multiplies the current input
    kind: str = "causal_taps"
    identity: bool = True  # add the input to the convolution's output
    bias_name: str | None = None  # checkpoint tensor [width]
    # the weight as several checkpoint tensors stacked along the channels: (name, first channel, end);
    # when given, `weight_name` only labels the part
    weight_parts: tuple = ()


@register_part("conv", "causal_taps")
class CausalTaps(Part):
    weight: torch.Tensor
    bias: torch.Tensor | None = None

    def __init__(self, spec: CausalTapsSpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        if spec.taps < 1:
            raise ValueError(f"a convolution needs at least one tap, got {spec.taps}")

    def param_specs(self) -> dict[str, ParamSpec]:
        s: CausalTapsSpec = self.spec
        sources = ([Source(name, (lo, hi)) for name, lo, hi in s.weight_parts] if s.weight_parts
                   else [Source(s.weight_name)])
        specs = {"weight": ParamSpec((s.width, s.taps), sources)}
        if s.bias_name is not None:
            specs["bias"] = ParamSpec((s.width,), [Source(s.bias_name)], init="bias")
        return specs

    def cache_need(self) -> FixedState | None:
        s: CausalTapsSpec = self.spec
        return FixedState((s.taps - 1, s.width), "float32") if s.taps > 1 else None

    def scratch_elements_per_token(self) -> int:
        return self.spec.width

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: FixedStateHandle | None) -> torch.Tensor:
        s: CausalTapsSpec = self.spec
        out = ctx.scratch("taps_out", (ctx.num_tokens, s.width), ctx.dtype)
        K.causal_taps(x, self.weight, None if cache is None else cache.state,
                      None if cache is None else cache.slots, ctx.cu_q, ctx.row_of_token, out, ctx.num_rows,
                      bias=self.bias, identity=s.identity)
        return out
