"""Parts that act on the residual stream itself, behind a layer's sub-layers (category ``stream``;
a pre-norm block lists them in ``stream_parts`` and runs them in order).

``TokenSideInput`` -- an input of the layer's own from a second embedding table.  The table
``[vocab, layers * dim]`` is one tensor for the whole model (``TokenTable``, a shared part); layer i
reads the columns ``[i * dim, (i + 1) * dim)`` of the token's row e and adds

    g = gelu_tanh(Wg x) * e;   y = Wp g;   x += y / sqrt(mean(y^2) + eps) * gain

to the stream x (as it stands after the layer's sub-layers).  The two products run on the stream
rounded to the activation type; the norm and the sum are 32-bit.

``DepthAverage`` -- the stream that goes on to the next layer is a weighted sum over the stream's
states at ALL depths so far: with X_0 the embedding output and X_(d+1) the result of the layer at depth
d, the layer at depth d hands on ``sum_j w[j] X_j`` over j = 0 .. d + 1, with d + 2 weights of its own.
The states live in a 32-bit scratch buffer ``[depths + 1, tokens, width]`` of the step; the part at
depth 0 stores X_0 when its block is entered.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from emberserve_b200 import kernels as K
from emberserve_b200.parts.base import (NormedDelta, ParamSpec, Part, Source, StepContext, StreamPart, build_part,
                                        register_part)
from emberserve_b200.parts.linear import linear
from emberserve_b200.parts.norm import GroupedRMSNorm, GroupedRMSNormSpec


@dataclass(frozen=True)
class TokenTableSpec:
    vocab_size: int
    width: int  # columns of the table: all layers' parts side by side
    name: str  # checkpoint tensor [vocab_size, width]
    kind: str = "token_table"


@register_part("stream", "token_table")
class TokenTable(Part):
    """A second embedding table that several layers read column ranges of; it does nothing by itself."""

    table: torch.Tensor

    def param_specs(self) -> dict[str, ParamSpec]:
        s: TokenTableSpec = self.spec
        return {"table": ParamSpec((s.vocab_size, s.width), [Source(s.name)])}


@dataclass(frozen=True)
class TokenSideInputSpec:
    hidden: int
    dim: int  # numbers of the token's row that this layer reads
    column: int  # the first of them
    table: TokenTableSpec
    eps: float
    gate_name: str  # [dim, hidden]
    proj_name: str  # [hidden, dim]
    norm_name: str  # [hidden], a plain gain
    kind: str = "token_side_input"


@register_part("stream", "token_side_input")
class TokenSideInput(StreamPart):
    wgate: torch.Tensor
    wproj: torch.Tensor

    def __init__(self, spec: TokenSideInputSpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        if spec.dim <= 0 or spec.column < 0 or spec.column + spec.dim > spec.table.width:
            raise ValueError(f"{prefix}: columns [{spec.column}, {spec.column + spec.dim}) of a table of "
                             f"{spec.table.width}")
        self.table_part = self.shared.get("stream", spec.table)
        self.out_norm = build_part("norm", GroupedRMSNormSpec(spec.hidden, 1, spec.eps, spec.norm_name),
                                   prefix + ".out_norm", self.shared)

    def children(self) -> dict[str, Part]:
        return {"out_norm": self.out_norm}

    def param_specs(self) -> dict[str, ParamSpec]:
        s: TokenSideInputSpec = self.spec
        return {"wgate": ParamSpec((s.dim, s.hidden), [Source(s.gate_name)]),
                "wproj": ParamSpec((s.hidden, s.dim), [Source(s.proj_name)])}

    def scratch_elements_per_token(self) -> int:
        return 2 * self.spec.hidden + 2 * self.spec.dim

    def forward(self, delta: Any, residual: torch.Tensor, ctx: StepContext) -> NormedDelta:
        s: TokenSideInputSpec = self.spec
        n = residual.shape[0]
        if isinstance(delta, NormedDelta):
            raise TypeError(f"{self.prefix}: reads the stream itself, so what precedes it must be added plainly")
        xb = ctx.scratch("side_x", (n, s.hidden), ctx.dtype)
        K.add_cast(delta, residual, xb)
        z = ctx.scratch("side_z", (n, s.dim), ctx.dtype)
        linear(xb, self.wgate, None, z, ctx.scratch)
        g = ctx.scratch("side_g", (n, s.dim), ctx.dtype)
        K.token_gate(z, self.table_part.table, s.column, ctx.tokens, g, deferred=ctx.deferred)
        y = ctx.scratch("side_y", (n, s.hidden), ctx.dtype)
        linear(g, self.wproj, None, y, ctx.scratch)
        return NormedDelta(y, self.out_norm)  # whoever receives it norms, scales and adds in one kernel


@dataclass(frozen=True)
class DepthAverageSpec:
    hidden: int
    depth: int  # 0 for the first layer; the part owns depth + 2 weights
    depths: int  # layers of the model that average (the history holds depths + 1 states)
    weight_name: str  # [depth + 2]
    kind: str = "depth_average"


@register_part("stream", "depth_average")
class DepthAverage(StreamPart):
    weight: torch.Tensor

    def __init__(self, spec: DepthAverageSpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        if not 0 <= spec.depth < spec.depths:
            raise ValueError(f"{prefix}: depth {spec.depth} of {spec.depths}")
        self._w32: torch.Tensor | None = None

    def param_specs(self) -> dict[str, ParamSpec]:
        s: DepthAverageSpec = self.spec
        return {"weight": ParamSpec((s.depth + 2,), [Source(s.weight_name)], init="ones")}

    def bind(self, params: dict[str, torch.Tensor]) -> None:
        super().bind(params)
        self._w32 = self.weight.float().contiguous()

    def _history(self, residual: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        n, h = residual.shape
        return ctx.scratch("depth_history", (self.spec.depths + 1, n, h), torch.float32)

    def on_entry(self, residual: torch.Tensor, ctx: StepContext) -> None:
        if self.spec.depth == 0:  # the stream as the first layer receives it is state 0
            K.depth_mix(None, None, 0.0, residual, self._history(residual, ctx), None, 1)

    def forward(self, delta: Any, residual: torch.Tensor, ctx: StepContext) -> None:
        s: DepthAverageSpec = self.spec
        x, gain, eps = delta, None, 0.0
        if isinstance(delta, NormedDelta):
            post = delta.norm
            if not isinstance(post, GroupedRMSNorm) or post.spec.groups != 1:
                raise TypeError(f"{self.prefix}: a delta normed by {type(post).__name__} cannot be taken")
            x, gain, eps = delta.x, post.gain, post.spec.eps
        K.depth_mix(x, gain, eps, residual, self._history(residual, ctx), self._w32, s.depth + 2)
        return None
