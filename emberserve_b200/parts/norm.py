"""RMSNorm fused with the residual add that precedes it.

``y = weight * cast(r * rsqrt(mean(r^2) + eps))`` with ``r = residual + delta``
(``emberserve/model/ops.py:51-63``, ``emberserve/model/qwen2.py:30-45``).  The residual
stream is held in 32 bits; the sum and the statistics are 32-bit.
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import torch

from emberserve_b200 import kernels as K
from emberserve_b200.parts.base import (Norm, NormedDelta, NormRequest, ParamSpec, ScaledRows, ScaledSum, Source,
                                        StepContext, register_part)


# EMBERSERVE_SPLIT_NORMS=0 keeps the norm a kernel of its own in every step (for comparisons).
_SPLIT_NORMS = os.environ.get("EMBERSERVE_SPLIT_NORMS", "1") != "0"


@dataclass(frozen=True)
class RMSNormSpec:
    dim: int
    eps: float
    weight_name: str  # checkpoint tensor of the gain, [dim]
    kind: str = "rmsnorm"


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    weight: torch.Tensor

    def param_specs(self) -> dict[str, ParamSpec]:
        s: RMSNormSpec = self.spec
        return {"weight": ParamSpec((s.dim,), [Source(s.weight_name)], init="ones")}

    def scratch_elements_per_token(self) -> int:
        return self.spec.dim  # "normed" (the rows before the head are fewer)

    def split_request(self, residual: torch.Tensor, ctx: StepContext) -> NormRequest | None:
        # In bfloat16 steps of few rows the norm is split between the products around it: the one
        # before adds into the residual, applies the gain and begins the sum of squares, the one
        # behind multiplies its rows by rsqrt(mean + eps).  (Roundings then differ from the
        # kernel's: residual * gain is rounded once, the scale is applied to a float32 result.)
        if (ctx.dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16 and residual.is_cuda
                and ctx.num_tokens <= K.GEMM_NORM_ROWS and _SPLIT_NORMS):
            return NormRequest(residual, self.weight, self.spec.eps)
        return None

    def forward(self, delta: torch.Tensor | None, residual: torch.Tensor, ctx: StepContext,
                rows: torch.Tensor | None = None) -> torch.Tensor:
        if isinstance(delta, ScaledRows):  # begun by the product before: the product behind finishes it
            assert rows is None
            return delta
        s: RMSNormSpec = self.spec
        n = residual.shape[0] if rows is None else rows.numel()
        out = ctx.scratch("normed" if rows is None else "normed_rows", (n, s.dim), ctx.dtype)
        K.add_rmsnorm(delta, residual, self.weight, out, s.eps, rows=rows)
        return out


@dataclass(frozen=True)
class GroupedRMSNormSpec:
    dim: int
    groups: int  # the width is cut into this many equal consecutive parts, each with its own statistics
    eps: float
    weight_name: str  # checkpoint tensor of the gain, [dim]
    kind: str = "rmsnorm_grouped"
    gain_offset: float = 0.0  # the gain is the stored tensor plus this (1.0: a weight stored around zero)


@register_part("norm", "rmsnorm_grouped")
class GroupedRMSNorm(Norm):
    """RMSNorm in groups: ``y[g] = x[g] / sqrt(mean(x[g]^2) + eps)`` for each of `groups` equal
    consecutive parts g of the vector, then ``y * weight`` over the whole (groups = 1 is the plain
    RMSNorm, with the gain applied to the unrounded 32-bit value).  All of it in 32 bits.

    `forward` takes these kinds of `delta`: None, a tensor (added to the stream as it is), a
    `NormedDelta` whose own norm is a GroupedRMSNorm: then ``residual += thatnorm(delta.x)`` and
    this norm of the new residual are one kernel; or a `ScaledSum`, whose terms are added into the
    32-bit residual first (of every row, also when only some rows are normed)."""

    weight: torch.Tensor

    def __init__(self, spec: GroupedRMSNormSpec, prefix: str, shared=None) -> None:
        super().__init__(spec, prefix, shared)
        if spec.groups <= 0 or spec.dim % spec.groups:
            raise ValueError(f"a norm over {spec.dim} numbers cannot have {spec.groups} equal groups")

    def param_specs(self) -> dict[str, ParamSpec]:
        s: GroupedRMSNormSpec = self.spec
        return {"weight": ParamSpec((s.dim,), [Source(s.weight_name)], init="ones")}

    def scratch_elements_per_token(self) -> int:
        return self.spec.dim

    def bind(self, params: dict[str, torch.Tensor]) -> None:
        super().bind(params)
        # the gain as the kernels read it: with an offset, the 32-bit sum (the stored tensor stays as loaded)
        self.gain = self.weight if not self.spec.gain_offset else self.weight.float() + self.spec.gain_offset

    def normalize_stream(self, residual: torch.Tensor, ctx: StepContext) -> None:
        s: GroupedRMSNormSpec = self.spec
        if s.groups != 1:
            raise NotImplementedError(f"{self.prefix}: the stream is normed in place as one group only")
        K.stream_norm(residual, self.weight, s.gain_offset, s.eps)

    def forward(self, delta, residual: torch.Tensor, ctx: StepContext,
                rows: torch.Tensor | None = None) -> torch.Tensor:
        s: GroupedRMSNormSpec = self.spec
        n = residual.shape[0] if rows is None else rows.numel()
        out = ctx.scratch("normed" if rows is None else "normed_rows", (n, s.dim), ctx.dtype)
        if isinstance(delta, ScaledSum):
            K.add_scaled_norm2(delta.terms, residual, None, None, 0.0, s.eps, None, None)
            delta = None
        x, gain, groups, eps = delta, None, 1, 0.0
        if isinstance(delta, NormedDelta):
            post = delta.norm
            if not isinstance(post, GroupedRMSNorm):
                raise TypeError(f"{self.prefix}: a delta normed by {type(post).__name__} cannot be taken")
            x, gain, groups, eps = delta.x, post.gain, post.spec.groups, post.spec.eps
            if gain.dtype != self.gain.dtype:  # (the kernel reads both gains as one type)
                gain = gain.to(self.gain.dtype)
        K.add_norm_grouped(x, gain, groups, eps, residual, self.gain, s.groups, s.eps, out, rows=rows)
        return out
