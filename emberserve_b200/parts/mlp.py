"""Dense feed-forwards.  Gated: ``down(act(gate(x)) * up(x))``, no biases; act is SiLU (SwiGLU)
unless the spec names another (``relu``, ``gelu_tanh``, ``swiglu_capped``: see
``kernels.GLU_ACTIVATIONS``), which takes the unfused kernels.  With `token_gate_name` ([1, hidden]) the
output of every token is multiplied by ``sigmoid(x . wg)``: the gate is one more column of the gate/up
product and is applied to the activation (one number per row passes the down projection unchanged).
Ungated (``DenseMLP``): ``down(act(up(x)))`` with act one of ``kernels.UNARY_ACTIVATIONS``
(``relu2`` is the square of relu).

gate and up are one fused projection whose first I output columns are the gate and the
last I the up part (``emberserve/model/qwen2.py:48-61``); the activation is
``silu(g) * u`` computed in 32 bits (``emberserve/model/ops.py:84-87``).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from emberserve_b200 import kernels as K
from emberserve_b200.parts.base import FeedForward, ParamSpec, Source, StepContext, register_part
from emberserve_b200.parts.linear import gated_linear, linear


@dataclass(frozen=True)
class SwiGLUSpec:
    hidden: int
    intermediate: int
    # checkpoint names of the three projections, without ".weight"
    gate_name: str
    up_name: str
    down_name: str
    kind: str = "swiglu"
    activation: str = "silu"  # one of kernels.GLU_ACTIVATIONS
    weight_suffix: str = ".weight"  # what follows the three names in the checkpoint
    act_limit: float = 0.0  # the two constants of "swiglu_capped"
    act_alpha: float = 1.0
    token_gate_name: str | None = None  # full name of a [1, hidden] tensor: the output times sigmoid(x . wg)


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    splits_norms = True
    wgu: torch.Tensor
    wdown: torch.Tensor

    def __init__(self, spec: SwiGLUSpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        if spec.activation not in K.GLU_ACTIVATIONS:
            raise ValueError(f"activation {spec.activation!r}: one of {sorted(K.GLU_ACTIVATIONS)}")

    def param_specs(self) -> dict[str, ParamSpec]:
        s: SwiGLUSpec = self.spec
        i = s.intermediate
        srcs = [Source(s.gate_name + s.weight_suffix, (0, i)), Source(s.up_name + s.weight_suffix, (i, 2 * i))]
        rows = 2 * i
        if s.token_gate_name is not None:  # (padded so that a row of the product stays 16-byte aligned)
            srcs.append(Source(s.token_gate_name, (2 * i, 2 * i + 1)))
            rows = 2 * i + 8
        return {
            "wgu": ParamSpec((rows, s.hidden), srcs),
            "wdown": ParamSpec((s.hidden, i), [Source(s.down_name + s.weight_suffix)]),
        }

    def streamed_params(self) -> list[str]:
        return ["wgu", "wdown"]

    def scratch_elements_per_token(self) -> int:
        # ffn_act, ffn_out, and gate_up for the steps in which no fused kernel takes the sizes
        return 3 * self.spec.intermediate + self.spec.hidden + (8 if self.spec.token_gate_name is not None else 0)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        s: SwiGLUSpec = self.spec
        n = x.shape[0]
        act = ctx.scratch("ffn_act", (n, s.intermediate), ctx.dtype)
        if s.activation != "silu" or s.token_gate_name is not None:
            # (the kernels with the activation in their epilogue know SiLU only)
            gu = ctx.scratch("gate_up", (n, self.wgu.shape[0]), ctx.dtype)
            linear(x, self.wgu, None, gu, ctx.scratch)
            K.glu_act(gu, act, s.activation, s.act_limit, s.act_alpha, row_gate=s.token_gate_name is not None)
        elif not gated_linear(x, self.wgu, act):  # both projections and SiLU in one kernel, where one takes the sizes
            gu = ctx.scratch("gate_up", (n, 2 * s.intermediate), ctx.dtype)
            linear(x, self.wgu, None, gu, ctx.scratch)
            K.silu_mul(gu, act)
        y = ctx.scratch("ffn_out", (n, s.hidden), ctx.dtype)
        # (the norm behind this feed-forward, if the down projection's product may begin it)
        return linear(act, self.wdown, None, y, ctx.scratch, ctx.extra.get("norm_behind"))


@dataclass(frozen=True)
class DenseMLPSpec:
    hidden: int
    intermediate: int
    up_name: str  # checkpoint tensor [intermediate, hidden]
    down_name: str  # checkpoint tensor [hidden, intermediate]
    activation: str = "relu2"  # one of kernels.UNARY_ACTIVATIONS
    kind: str = "dense_mlp"


@register_part("feed_forward", "dense_mlp")
class DenseMLP(FeedForward):
    """``down(act(up(x)))`` without gate and without biases; the activation is computed in 32 bits
    from the rounded projection and rounded once."""

    wup: torch.Tensor
    wdown: torch.Tensor

    def __init__(self, spec: DenseMLPSpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        if spec.activation not in K.UNARY_ACTIVATIONS:
            raise ValueError(f"activation {spec.activation!r}: one of {sorted(K.UNARY_ACTIVATIONS)}")

    def param_specs(self) -> dict[str, ParamSpec]:
        s: DenseMLPSpec = self.spec
        return {"wup": ParamSpec((s.intermediate, s.hidden), [Source(s.up_name)]),
                "wdown": ParamSpec((s.hidden, s.intermediate), [Source(s.down_name)])}

    def streamed_params(self) -> list[str]:
        return ["wup", "wdown"]

    def scratch_elements_per_token(self) -> int:
        return 2 * self.spec.intermediate + self.spec.hidden

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        s: DenseMLPSpec = self.spec
        n = x.shape[0]
        up = ctx.scratch("ffn_up", (n, s.intermediate), ctx.dtype)
        linear(x, self.wup, None, up, ctx.scratch)
        act = ctx.scratch("ffn_act", (n, s.intermediate), ctx.dtype)
        K.unary_act(up, act, s.activation)
        y = ctx.scratch("ffn_out", (n, s.hidden), ctx.dtype)
        return linear(act, self.wdown, None, y, ctx.scratch)
